"""Drives the reference's own ``stickbreaking`` (oracle/_ref/sb_ref.py, put there by build_ref.py) over a packed
batch.  TEST INFRASTRUCTURE ONLY: used by the CPU arm of the benchmark and by tests; never by the product.

The driving follows the reference's tests (tests/test_varlen.py:11-43): the token axis is split by the sequence
lengths, every piece gets ``mask = triu(0)`` (``triu(1)`` when the current token may be attended) and
``cum_weight = tril(-1)``, gradients come from autograd.  Unlike those tests the two results ``o`` and ``rem``
are kept apart and ``rem`` receives its own upstream gradient.
"""
import importlib.util
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF_FILE = os.path.join(HERE, "_ref", "sb_ref.py")


def available():
    return os.path.isfile(REF_FILE)


def load():
    spec = importlib.util.spec_from_file_location("sb_ref_reference", REF_FILE)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.stickbreaking


def fwd_bwd(stickbreaking, q, k, v, do, drem, lengths, attend_current=False):
    """q, k, v, do: float32 CPU tensors [H, T, D]; drem [H, T].  Returns (o, rem, dq, dk, dv)."""
    q, k, v = (x.detach().clone().requires_grad_() for x in (q, k, v))
    outs, rems = [], []
    start = 0
    for L in lengths:
        sl = slice(start, start + L)
        ones = torch.ones(L, L, dtype=torch.bool)
        mask = ones.triu(1 if attend_current else 0)
        cm = torch.ones(L, L).tril(-1)
        o, rem = stickbreaking(q[None, :, sl], k[None, :, sl], v[None, :, sl], mask, cm)
        outs.append(o[0])
        rems.append(rem[0])
        start += L
    o, rem = torch.cat(outs, 1), torch.cat(rems, 1)
    dq, dk, dv = torch.autograd.grad([o, rem], [q, k, v], [do[:, :start], drem[:, :start]])
    return o.detach(), rem.detach(), dq, dk, dv

"""Builds tests/golden/*.npz by running the REFERENCE's dense implementation on seeded inputs.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It imports ``stickbreaking_attention/sb_ref.py`` (function ``stickbreaking``) from that checkout, drives it per
sequence exactly as the reference's ``tests/test_varlen.py:11-28`` does (but keeps ``o`` and ``rem`` separate),
and differentiates with autograd for upstream gradients (do, drem).  Only outputs and a digest of the inputs are
stored; the inputs are regenerated from their seed by ``cases.make_inputs``.
"""
import importlib.util
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from cases import CASES, digest, inv_temp_of, make_inputs  # noqa: E402


def load_reference(root):
    path = os.path.join(root, "stickbreaking_attention", "sb_ref.py")
    spec = importlib.util.spec_from_file_location("sb_ref_reference", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.stickbreaking


def run_case(stickbreaking, spec):
    q, k, v, do, drem = [torch.from_numpy(x.copy()) for x in make_inputs(spec)]
    D = spec["D"]
    inv_temp = inv_temp_of(spec)
    # the reference hard-codes 1/sqrt(D) (sb_ref.py:12): other temperatures go through a rescaled q
    qscale = inv_temp * math.sqrt(D)
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    outs_o, outs_r = [], []
    a = 0
    for L in spec["lengths"]:
        b = a + L
        mask = torch.ones(L, L).triu(1 if spec["attend_current"] else 0).bool()
        cm = torch.ones(L, L).tril(-1)
        o, rem = stickbreaking((q[:, a:b] * qscale)[None], k[None, :, a:b], v[None, :, a:b], mask, cm)
        outs_o.append(o[0])
        outs_r.append(rem[0])
        a = b
    o = torch.cat(outs_o, 1)
    rem = torch.cat(outs_r, 1)
    dq, dk, dv = torch.autograd.grad([o, rem], [q, k, v], [do, drem])
    return dict(o=o.detach().numpy(), rem=rem.detach().numpy(), dq=dq.numpy(), dk=dk.numpy(), dv=dv.numpy())


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <checkout of speedcell4/stickbreaking-attention>")
    root = sys.argv[1]
    stickbreaking = load_reference(root)
    torch.manual_seed(0)
    for name, spec in CASES.items():
        out = run_case(stickbreaking, spec)
        out["input_digest"] = np.array(digest(make_inputs(spec)))
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(name, {k: (v.shape if hasattr(v, "shape") else v) for k, v in out.items()})


if __name__ == "__main__":
    main()

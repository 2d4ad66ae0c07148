"""Seeded input generators shared by the fixture builder and the tests (no reference import here)."""
import hashlib
import math

import numpy as np
import torch

# name -> specification of a packed varlen case
CASES = {
    # first configuration of the benchmark list: fp32, 4 heads, 512 tokens, head_dim 64, three sequences
    "c1": dict(H=4, D=64, lengths=[128, 192, 192], seed=0, dist="normal", attend_current=False, bf16=False),
    "c1_attend": dict(H=2, D=64, lengths=[128, 192, 192], seed=0, dist="normal", attend_current=True, bf16=False),
    # input distribution of the reference's own tests (tests/test_varlen.py:85-95), ragged multi-sequence pack
    "reftest_ragged": dict(H=3, D=32, lengths=[70, 1, 129, 56], seed=1337, dist="reftest", attend_current=False,
                           bf16=True),
    "reftest_ragged_attend": dict(H=3, D=32, lengths=[70, 1, 129, 56], seed=1337, dist="reftest",
                                  attend_current=True, bf16=True),
    "tiny_edges": dict(H=2, D=16, lengths=[1, 2, 63, 64, 65], seed=7, dist="normal", attend_current=False,
                       bf16=False),
    # temperature different from 1/sqrt(D)
    "temp": dict(H=2, D=64, lengths=[100, 156], seed=3, dist="normal", attend_current=False, bf16=True,
                 inv_temp=0.07),
    "d128": dict(H=1, D=128, lengths=[300, 84], seed=11, dist="normal", attend_current=False, bf16=True),
}


def make_inputs(spec):
    """q, k, v, do [H,T,D] and drem [H,T] as float32 numpy arrays (bf16-representable when spec['bf16'])."""
    g = torch.Generator().manual_seed(spec["seed"])
    H, D = spec["H"], spec["D"]
    T = sum(spec["lengths"])

    def randn(*shape):
        return torch.randn(*shape, generator=g, dtype=torch.float32)

    if spec["dist"] == "normal":
        q, k, v = randn(H, T, D), randn(H, T, D), randn(H, T, D)
    else:  # the reference tests: negative-mean logits
        v = 0.25 * randn(H, T, D)
        q = 0.25 * (randn(H, T, D) + 1)
        k = 0.25 * (randn(H, T, D) - 1)
    do = randn(H, T, D)
    drem = randn(H, T)
    if spec["bf16"]:
        q, k, v, do, drem = [x.to(torch.bfloat16).float() for x in (q, k, v, do, drem)]
    return [x.numpy() for x in (q, k, v, do, drem)]


def inv_temp_of(spec):
    return spec.get("inv_temp", 1.0 / math.sqrt(spec["D"]))


def digest(arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a, dtype=np.float32).tobytes())
    return h.hexdigest()

"""The operators under torch.compile: one opaque registered operator per launcher, no graph break, same results."""
import numpy as np
import pytest
import torch

from tests.util import synth

pytestmark = pytest.mark.gpu


def _grads(fn, q, k, v, do, dr):
    q, k, v = (x.clone().requires_grad_() for x in (q, k, v))
    o, rem = fn(q, k, v)
    dq, dk, dv = torch.autograd.grad([o, rem], [q, k, v], [do, dr])
    return [x.detach() for x in (o, rem, dq, dk, dv)]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_varlen_compiled_matches_eager(dtype):
    from stickbreaking_attention_b200 import sb_attn_varlen
    lengths = [130, 257, 64, 61]
    H, T, D = 2, sum(lengths), 64
    q, k, v, do, dr = (torch.from_numpy(x).to("cuda", dtype) for x in synth(H, T, D, 5))
    cu = torch.tensor(np.cumsum(lengths), dtype=torch.int32, device="cuda")

    def fn(q, k, v):
        return sb_attn_varlen(q, k, v, cu, max(lengths), zero_start=False)

    eager = _grads(fn, q, k, v, do, dr)
    compiled = _grads(torch.compile(fn, backend="aot_eager", fullgraph=True), q, k, v, do, dr)
    for a, b in zip(eager, compiled):
        assert torch.equal(a, b)


def test_batched_compiled_matches_eager():
    from stickbreaking_attention_b200 import sb_attn
    B, H, T, D = 2, 2, 200, 64
    g = torch.Generator().manual_seed(3)
    q, k, v, do = (torch.randn(B, H, T, D, generator=g).to("cuda", torch.bfloat16) for _ in range(4))
    dr = torch.randn(B, H, T, generator=g).to("cuda", torch.bfloat16)

    def fn(q, k, v):
        return sb_attn(q, k, v, attend_current=True)

    eager = _grads(fn, q, k, v, do, dr)
    compiled = _grads(torch.compile(fn, backend="aot_eager", fullgraph=True), q, k, v, do, dr)
    for a, b in zip(eager, compiled):
        assert torch.equal(a, b)


def test_fused_remainder_compiled_matches_eager():
    from stickbreaking_attention_b200 import sb_attn_varlen
    lengths = [200, 130, 182]
    H, T, D = 2, sum(lengths), 128
    q, k, v, do, dr = (torch.from_numpy(x).to("cuda", torch.bfloat16) for x in synth(H, T, D, 6))
    cu = torch.tensor(np.cumsum(lengths), dtype=torch.int32, device="cuda")

    def fn(q, k, v):
        return sb_attn_varlen(q, k, v, cu, max(lengths), zero_start=False, fuse_remainder=True)

    eager = _grads(fn, q, k, v, do, dr)
    compiled = _grads(torch.compile(fn, backend="aot_eager", fullgraph=True), q, k, v, do, dr)
    for a, b in zip(eager, compiled):
        assert torch.equal(a, b)

"""The allocation-free forward (sbattn_fwd_static) against the ordinary forward, through the C ABI.

Some callers cannot allocate device memory when they call into the library -- a serving process whose pool already
owns the GPU, a plugin that may not use its host's allocator -- so the library offers one forward whose scratch is a
fixed array inside the library.  This file is collected last on purpose: if it fails, `pytest -x` has already run
every other test.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _params(q, k, v, cu, max_len, inv_temp, o, rem, nla):
    from stickbreaking_attention_b200 import ops
    p = ops._base_params(q, False, cu, max_len, inv_temp, False, False)
    p.q, p.k, p.v, p.o = (ops._mat(t, False) for t in (q, k, v, o))
    p.rem, p.neg_log_acc = ops._vec(rem, False), ops._vec(nla, False)
    return p


def _forward(entry, q, k, v, cu, max_len, inv_temp, with_workspace):
    from stickbreaking_attention_b200 import _lib, ops
    o = torch.empty_like(q)
    rem = torch.zeros(q.shape[:-1], dtype=q.dtype, device=q.device)
    nla = torch.zeros(q.shape[:-1], dtype=torch.float32, device=q.device)
    p = _params(q, k, v, cu, max_len, inv_temp, o, rem, nla)
    ws = None
    if with_workspace:
        fwd_bytes, _ = ops._workspace_sizes(p)
        ws = torch.empty(fwd_bytes, dtype=torch.uint8, device=q.device)
        p.fwd_workspace, p.fwd_workspace_bytes = ws.data_ptr(), fwd_bytes
    _lib.check(getattr(_lib.lib(), entry)(ctypes.byref(p)), entry)
    torch.cuda.synchronize()
    ops.check_status(q.device)
    return o, rem, nla


@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 128), (torch.float32, 64)])
def test_static_forward_matches_ordinary_forward_twice(dtype, D):
    lengths = [300, 45, 129, 550]
    H, T = 3, sum(lengths)
    g = torch.Generator().manual_seed(3)
    cu = torch.tensor(np.cumsum(lengths), device="cuda", dtype=torch.int32)
    it = 1 / math.sqrt(D)
    for call in range(2):  # two calls in a row share the built-in scratch: the second must not see stale state
        q, k, v = (torch.randn(H, T, D, generator=g).to(dtype).cuda() for _ in range(3))
        want = _forward("sbattn_fwd", q, k, v, cu, max(lengths), it, True)
        got = _forward("sbattn_fwd_static", q, k, v, cu, max(lengths), it, False)
        tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
        for name, a, b in zip(("o", "rem"), got, want):
            assert torch.isfinite(a.float()).all(), (call, name)
            assert (a.float() - b.float()).abs().max().item() <= tol, (call, name)
        # same kernels on the same data: identical bits (neg_log_acc is -inf where the remainder underflowed to 0)
        for name, a, b in zip(("o", "rem", "neg_log_acc"), got, want):
            assert torch.equal(a, b), (call, name)


def test_static_forward_rejects_oversized_problem():
    from stickbreaking_attention_b200 import _lib
    q = torch.zeros(1, 128, 64, device="cuda", dtype=torch.bfloat16)
    n_seqs = 200_000  # the sequence table alone exceeds the 1 MiB scratch
    cu = torch.zeros(n_seqs, device="cuda", dtype=torch.int32)
    o, rem = torch.empty_like(q), torch.zeros(1, 128, device="cuda", dtype=torch.bfloat16)
    nla = torch.zeros(1, 128, device="cuda", dtype=torch.float32)
    p = _params(q, q, q, cu, 128, 0.125, o, rem, nla)
    assert _lib.lib().sbattn_static_scratch_bytes() == 1 << 20
    assert _lib.lib().sbattn_fwd_static(ctypes.byref(p)) == -7


def test_static_forward_leaves_device_memory_untouched():
    """The property the entry point exists for: once the first call on the device has looked the scratch array up, a
    call neither takes nor returns device memory.  Free memory as the driver reports it (cudaMemGetInfo, which sees
    every allocation of the process, whoever made it) is the same before and after the call, and so is what PyTorch's
    allocator holds, since the outputs were allocated beforehand."""
    from stickbreaking_attention_b200 import _lib, ops
    lengths = [200, 312, 129]
    H, T, D = 4, sum(lengths), 128
    g = torch.Generator().manual_seed(11)
    q, k, v = (torch.randn(H, T, D, generator=g).bfloat16().cuda() for _ in range(3))
    cu = torch.tensor(np.cumsum(lengths), device="cuda", dtype=torch.int32)
    o = torch.empty_like(q)
    rem = torch.zeros(H, T, dtype=q.dtype, device="cuda")
    nla = torch.zeros(H, T, dtype=torch.float32, device="cuda")
    p = _params(q, k, v, cu, max(lengths), 1 / math.sqrt(D), o, rem, nla)
    fwd_static = _lib.lib().sbattn_fwd_static
    _lib.check(fwd_static(ctypes.byref(p)), "first call: looks up the scratch address, loads the kernels")
    torch.cuda.synchronize()
    ops.check_status(q.device)
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    _lib.check(fwd_static(ctypes.byref(p)), "second call")
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)
    assert torch.cuda.memory_reserved() == reserved_before
    ops.check_status(q.device)
    assert torch.isfinite(o.float()).all()

"""GPU parity: the CUDA path (through the public Python API, hence the C ABI) against the reference fixtures and the
numpy oracle on the same seeded inputs."""
import math
import os

import numpy as np
import pytest
import torch

from cases import CASES, inv_temp_of, make_inputs
from util import (TOL_BF16, TOL_F32, assert_close, oracle_varlen, rounded, run_batched, run_varlen, synth)
from oracle import sb_oracle as orc

pytestmark = pytest.mark.gpu
NAMES = ("o", "rem", "dq", "dk", "dv")
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def gold(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    return [z[k].astype(np.float64) for k in NAMES]


@pytest.mark.parametrize("name", sorted(CASES))
def test_fixture_float32_mode(name):
    """float32 inputs: max-abs <= 1e-5 against the reference's own outputs."""
    spec = CASES[name]
    ins = make_inputs(spec)
    got = run_varlen(*ins, spec["lengths"], inv_temp_of(spec), spec["attend_current"], torch.float32)
    assert_close(NAMES, got, gold(name), TOL_F32, name)


@pytest.mark.parametrize("name", sorted(n for n in CASES if CASES[n]["bf16"]))
@pytest.mark.parametrize("path", ["auto", "simt"])
def test_fixture_bf16(name, path):
    """bf16 inputs (the fixtures of these cases were produced from bf16-representable values): max-abs <= 2e-2."""
    import stickbreaking_attention_b200 as sb
    spec = CASES[name]
    ins = make_inputs(spec)
    sb.set_path(path)
    try:
        got = run_varlen(*ins, spec["lengths"], inv_temp_of(spec), spec["attend_current"], torch.bfloat16)
    finally:
        sb.set_path("auto")
    assert_close(NAMES, got, gold(name), TOL_BF16, name)


@pytest.mark.parametrize("zero_start,cu_dtype", [(False, torch.int64), (True, torch.int32), (False, torch.int32)])
def test_cu_seqlens_conventions(zero_start, cu_dtype):
    spec = CASES["tiny_edges"]
    ins = make_inputs(spec)
    got = run_varlen(*ins, spec["lengths"], inv_temp_of(spec), False, torch.float32, zero_start=zero_start,
                     cu_dtype=cu_dtype, max_seqlens=None if zero_start else "given")
    assert_close(NAMES, got, gold("tiny_edges"), TOL_F32)


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, TOL_BF16), (torch.float16, TOL_BF16), (torch.float32, TOL_F32)])
@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("attend_current", [False, True])
def test_ragged_pack_against_oracle(dtype, tol, D, attend_current):
    lengths = [1, 127, 128, 129, 300, 2, 64, 513, 255]
    H, T = 3, sum(lengths)
    ins = [rounded(x, dtype) for x in synth(H, T, D, seed=5)]
    it = 1 / math.sqrt(D)
    got = run_varlen(*ins, lengths, it, attend_current, dtype)
    want = oracle_varlen(*ins, lengths, it, attend_current)
    assert_close(NAMES, got, want, tol, f"D={D}")


@pytest.mark.parametrize("B,H,T,D", [(2, 3, 500, 50), (1, 2, 256, 16), (2, 1, 512, 32), (2, 2, 640, 64),
                                     (1, 3, 1024, 128)])
@pytest.mark.parametrize("attend_current", [False, True])
def test_batched_reference_distribution(B, H, T, D, attend_current):
    """Shapes and input distribution of the reference's tests/test_attn.py:40-59 (including head_dim 50, T 500)."""
    ins = synth(B * H, T, D, seed=1337, dist="reftest")
    ins = [rounded(x, torch.bfloat16) for x in ins]
    ins4 = [x.reshape((B, H) + x.shape[1:]) for x in ins]
    it = 1 / math.sqrt(D)
    got = run_batched(*ins4, it, attend_current, torch.bfloat16)
    want = orc.sb_batched_fwd_bwd(*ins4, it, attend_current)
    assert_close(NAMES, got, want, TOL_BF16, f"{B,H,T,D}")


def test_reference_test_quantity_single_sequence():
    """What the reference's tests/test_varlen.py:97-112 checks: o + rem*v and its gradients, eps 0.05 there."""
    from stickbreaking_attention_b200 import sb_attn_varlen
    H, T, D = 3, 4096, 128
    q, k, v, do, _ = [rounded(x, torch.bfloat16) for x in synth(H, T, D, seed=1337, dist="reftest")]
    tq, tk, tv = (torch.from_numpy(x).cuda().bfloat16().requires_grad_() for x in (q, k, v))
    tdo = torch.from_numpy(do).cuda().bfloat16()
    cu = torch.tensor([T], device="cuda", dtype=torch.int64)
    o, rem = sb_attn_varlen(tq, tk, tv, cu, T, inv_temp=1 / math.sqrt(D), zero_start=False)
    out = o + rem[..., None] * tv
    dq, dk, dv = torch.autograd.grad(out, (tq, tk, tv), tdo)
    drem = (do * v).sum(-1)
    ro, rrem, rdq, rdk, rdv = orc.sb_varlen_fwd_bwd(q, k, v, do, drem, [T], 1 / math.sqrt(D))
    rout = ro + rrem[..., None] * v
    rdv = rdv + rrem[..., None] * do
    for n, g, w in zip(("out", "dq", "dk", "dv"), (out, dq, dk, dv), (rout, rdq, rdk, rdv)):
        err = np.abs(g.detach().double().cpu().numpy() - w).max()
        assert err < TOL_BF16 * 1.5, (n, err)


def test_strided_inputs_token_major():
    """The reference's benchmark passes [T,H,D] tensors permuted to [H,T,D] (benchmarks/varlen.py:44-46)."""
    from stickbreaking_attention_b200 import sb_attn_varlen
    lengths = [200, 312]
    H, T, D = 4, 512, 64
    q, k, v, do, drem = [rounded(x, torch.bfloat16) for x in synth(H, T, D, seed=9)]
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x.transpose(1, 0, 2))).cuda().bfloat16()
    tq, tk, tv = (dev(x).requires_grad_() for x in (q, k, v))
    cu = torch.tensor(np.cumsum(lengths), device="cuda")
    o, rem = sb_attn_varlen(tq.permute(1, 0, 2), tk.permute(1, 0, 2), tv.permute(1, 0, 2), cu, max(lengths),
                            zero_start=False)
    tdo = torch.from_numpy(do).cuda().bfloat16()
    tdr = torch.from_numpy(drem).cuda().bfloat16()
    dq, dk, dv = torch.autograd.grad([o, rem], [tq, tk, tv], [tdo, tdr])
    got = [o, rem] + [x.permute(1, 0, 2) for x in (dq, dk, dv)]
    got = [x.detach().double().cpu().numpy() for x in got]
    want = oracle_varlen(q, k, v, do, drem, lengths, 1 / math.sqrt(D), False)
    assert_close(NAMES, got, want, TOL_BF16)


def test_outputs_at_16_byte_aligned_addresses():
    """A C-ABI caller may hand over result buffers that are 16-byte but not 32-byte aligned (rows of D + 8 elements,
    first column skipped): the epilogues then fall back from 256-bit to 128-bit stores.  Same bits as the dense call."""
    from stickbreaking_attention_b200 import ops
    lengths = [150, 300, 62]
    H, T, D = 2, 512, 128
    q, k, v, do, drem = (torch.from_numpy(x).cuda().bfloat16() for x in synth(H, T, D, seed=11))
    cu = torch.tensor(np.cumsum(lengths), dtype=torch.int32, device="cuda")
    scale = 1 / math.sqrt(D)
    o, rem, nla, ws = ops.varlen_fwd(q, k, v, cu, max(lengths), scale)
    dq, dk, dv = ops.varlen_bwd(do, drem, q, k, v, cu, max(lengths), ws, scale)
    odd = lambda: torch.full((H, T, D + 8), 7.0, dtype=torch.bfloat16, device="cuda")[..., 8:]
    o2, rem2, nla2 = odd(), torch.zeros_like(rem), torch.zeros_like(nla)
    assert o2.data_ptr() % 32 == 16 and o2.stride(1) == D + 8
    fb, bb = ops.workspace_bytes(False, cu.numel(), H, T, max(lengths))
    ws2 = torch.empty(fb, dtype=torch.uint8, device="cuda")
    ops._forward_into(q, k, v, False, cu, max(lengths), scale, False, False, o2, rem2, nla2, ws2)
    dq2, dk2, dv2 = odd(), odd(), odd()
    ops._backward_into(do, drem, q, k, v, False, cu, max(lengths), ws2, scale, False, 0, dq2, dk2, dv2,
                       torch.empty(bb, dtype=torch.uint8, device="cuda"))
    torch.cuda.synchronize()
    ops.check_status()
    for a_, b_ in [(o, o2), (rem, rem2), (dq, dq2), (dk, dk2), (dv, dv2)]:
        assert torch.equal(a_, b_)


def test_rows_sum_to_one_and_linearity_full_size():
    """Size-independent properties on the 16384-token benchmark pack: with v = 1 every o entry equals 1 - rem,
    and o is linear in v."""
    from stickbreaking_attention_b200 import sb_attn_varlen
    lengths = [2943, 3503, 2192, 1807, 3696, 649, 1594]
    H, T, D = 4, sum(lengths), 128
    g = torch.Generator().manual_seed(0)
    q = torch.randn(H, T, D, generator=g).cuda().bfloat16()
    k = torch.randn(H, T, D, generator=g).cuda().bfloat16()
    v1 = torch.randn(H, T, D, generator=g).cuda().bfloat16()
    cu = torch.tensor(np.cumsum(lengths), device="cuda")
    ones = torch.ones_like(v1)
    o_ones, rem = sb_attn_varlen(q, k, ones, cu, max(lengths), zero_start=False)
    assert (o_ones.float() - (1 - rem.float())[..., None]).abs().max() < 2e-2
    o1, rem1 = sb_attn_varlen(q, k, v1, cu, max(lengths), zero_start=False)
    o2, _ = sb_attn_varlen(q, k, v1 * 2, cu, max(lengths), zero_start=False)
    assert torch.equal(rem, rem1)
    assert (o2.float() - 2 * o1.float()).abs().max() < 4e-2
    # first row of every sequence attends nothing
    starts = [0] + list(np.cumsum(lengths)[:-1])
    assert torch.all(o1[:, starts] == 0) and torch.all(rem1[:, starts] == 1)


def test_bitwise_deterministic():
    lengths = [700, 324]
    H, T, D = 2, 1024, 128
    ins = [rounded(x, torch.bfloat16) for x in synth(H, T, D, seed=21)]
    a = run_varlen(*ins, lengths, 0.1, False, torch.bfloat16)
    b = run_varlen(*ins, lengths, 0.1, False, torch.bfloat16)
    for x, y in zip(a, b):
        assert np.array_equal(x, y)


def test_bad_seqlens_reported_not_faulting():
    """Sequence ends that decrease or run past the token count set a status bit; nothing is computed, nothing faults."""
    import stickbreaking_attention_b200 as sb
    from stickbreaking_attention_b200 import sb_attn_varlen
    H, T, D = 1, 256, 64
    q = torch.randn(H, T, D, device="cuda", dtype=torch.bfloat16)
    sb.check_status()
    for ends in ([200, 100], [100, 300]):
        cu = torch.tensor(ends, device="cuda")
        with pytest.raises(ValueError):
            sb_attn_varlen(q, q, q, cu, 256, zero_start=False)
            sb.check_status()
    assert sb.check_status() == 0
    o, rem = sb_attn_varlen(q, q, q, torch.tensor([100, 256], device="cuda"), 256, zero_start=False)
    assert sb.check_status() == 0 and torch.isfinite(o.float()).all()


def test_tensor_core_path_is_taken():
    """Forcing the tcgen05 kernels must succeed for bf16/f16 with head_dim 32, 64 or 128 and be refused otherwise."""
    import stickbreaking_attention_b200 as sb
    from stickbreaking_attention_b200 import sb_attn_varlen
    from stickbreaking_attention_b200._lib import SbAttnError
    cu = torch.tensor([300], device="cuda")
    sb.set_path("tensor")
    try:
        for D in (64, 128):
            q = torch.randn(2, 300, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
            o, rem = sb_attn_varlen(q, q, q, cu, 300, zero_start=False)
            (o.float().sum() + rem.float().sum()).backward()
            assert torch.isfinite(q.grad.float()).all()
        q = torch.randn(2, 300, 50, device="cuda", dtype=torch.bfloat16)  # rows of 100 bytes: not whole 16-byte units
        with pytest.raises(SbAttnError):
            sb_attn_varlen(q, q, q, cu, 300, zero_start=False)
        q = torch.randn(2, 300, 64, device="cuda", dtype=torch.float32)
        with pytest.raises(SbAttnError):
            sb_attn_varlen(q, q, q, cu, 300, zero_start=False)
    finally:
        sb.set_path("auto")


@pytest.mark.parametrize("D", [32])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_tensor_path_head_dim_32(D, dtype):
    """Head dim 32 (the reference's test grid has 16 and 32, tests/test_attn.py:42; 16 stays on the fp32 kernels) on the
    tcgen05 kernels, which work on 64 or 128 columns that TMA pads with zeros: packed layout with ragged sequences,
    against the oracle; then the batched layout and the fused remainder on the same path."""
    import stickbreaking_attention_b200 as sb
    lengths = [1, 130, 257, 64, 300, 127]
    H, T = 3, sum(lengths)
    ins = [rounded(x, dtype) for x in synth(H, T, D, seed=40 + D)]
    it = 1 / math.sqrt(D)
    sb.set_path("tensor")
    try:
        got = run_varlen(*ins, lengths, it, D == 32, dtype)
        want = oracle_varlen(*ins, lengths, it, D == 32)
        assert_close(NAMES, got, want, TOL_BF16, f"tensor path D={D}")
        B, Hb, Tb = 2, 2, 200
        ins4 = [rounded(x, dtype) for x in synth(B * Hb, Tb, D, seed=41 + D, dist="reftest")]
        ins4 = [x.reshape((B, Hb) + x.shape[1:]) for x in ins4]
        got = run_batched(*ins4, it, False, dtype)
        want = orc.sb_batched_fwd_bwd(*ins4, it, False)
        assert_close(NAMES, got, want, TOL_BF16, f"tensor path batched D={D}")
    finally:
        sb.set_path("auto")


def test_broadcast_head_falls_back():
    """k and v expanded over the heads (stride 0, multi-query attention): a tensor map cannot describe them, so the
    fp32-arithmetic kernels take the call; same results as with materialised copies."""
    from stickbreaking_attention_b200 import sb_attn_varlen
    lengths = [150, 106]
    H, T, D = 4, 256, 64
    q, k, v, do, drem = [rounded(x, torch.bfloat16) for x in synth(H, T, D, seed=77)]
    k[:] = k[:1]
    v[:] = v[:1]
    tq = torch.from_numpy(q).cuda().bfloat16()
    tk1, tv1 = (torch.from_numpy(x[:1]).cuda().bfloat16() for x in (k, v))
    cu = torch.tensor(np.cumsum(lengths), device="cuda")
    o, rem = sb_attn_varlen(tq, tk1.expand(H, T, D), tv1.expand(H, T, D), cu, max(lengths), zero_start=False)
    want = oracle_varlen(q, k, v, do, drem, lengths, 1 / math.sqrt(D), False)
    got = [x.detach().double().cpu().numpy() for x in (o, rem)]
    assert_close(("o", "rem"), got, want[:2], TOL_BF16, "broadcast k, v")


def test_forward_after_fp32_path_feeds_tensor_backward():
    """The forward and the backward choose their kernels independently (by the alignment of their own operands): an
    output buffer the tensor-core forward cannot write sends the forward to the fp32-arithmetic kernels, whose carries the
    tensor-core backward must be able to use."""
    from stickbreaking_attention_b200 import ops
    lengths = [300, 212]
    H, T, D = 2, 512, 64
    ins = [rounded(x, torch.bfloat16) for x in synth(H, T, D, seed=91)]
    q, k, v, do, drem = (torch.from_numpy(x).cuda().bfloat16() for x in ins)
    cu = torch.tensor(np.cumsum(lengths), dtype=torch.int32, device="cuda")
    scale = 1 / math.sqrt(D)
    o = torch.empty(H, T, D + 2, dtype=torch.bfloat16, device="cuda")[..., 2:]  # rows start 4 bytes off a 16-byte boundary
    rem = torch.empty(H, T, dtype=torch.bfloat16, device="cuda")
    nla = torch.empty(H, T, dtype=torch.float32, device="cuda")
    fb, bb = ops.workspace_bytes(False, cu.numel(), H, T, max(lengths))
    ws = torch.empty(fb, dtype=torch.uint8, device="cuda")
    ops._forward_into(q, k, v, False, cu, max(lengths), scale, False, False, o, rem, nla, ws)
    dq, dk, dv = ops.varlen_bwd(do, drem, q, k, v, cu, max(lengths), ws, scale)
    torch.cuda.synchronize()
    ops.check_status()
    want = oracle_varlen(*ins, lengths, scale, False)
    got = [x.detach().double().cpu().numpy() for x in (o, rem, dq, dk, dv)]
    assert_close(NAMES, got, want, TOL_BF16, "fp32-path forward, tensor-core backward")


def test_uncovered_tokens_get_zero_remainder():
    """rem and neg_log_acc of tokens behind the last sequence are zero although the caller's buffers are not cleared."""
    from stickbreaking_attention_b200 import ops
    H, T, D = 2, 300, 64
    q = torch.randn(H, T, D, device="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([100, 180], dtype=torch.int32, device="cuda")
    o, rem, nla, _ = ops.varlen_fwd(q, q, q, cu, 100, 0.125, no_grad=True)
    torch.cuda.synchronize()
    assert torch.all(rem[:, 180:] == 0) and torch.all(nla[:, 180:] == 0)
    assert torch.all(rem[:, 0] == 1) and torch.all(rem[:, 100] == 1)


def test_recomputed_carries_give_the_same_gradients():
    """set_carry_policy('recompute') keeps nothing quadratic in the sequence length between forward and backward;
    results are the same bits as with saved carries, in both layouts."""
    import stickbreaking_attention_b200 as sb
    lengths = [700, 324, 129]
    H, T, D = 2, sum(lengths), 128
    ins = [rounded(x, torch.bfloat16) for x in synth(H, T, D, seed=23)]
    ins4 = [x.reshape((1, H) + x.shape[1:]) for x in ins]
    want = run_varlen(*ins, lengths, 0.1, False, torch.bfloat16)
    want4 = run_batched(*ins4, 0.1, True, torch.bfloat16)
    sb.set_carry_policy("recompute")
    try:
        got = run_varlen(*ins, lengths, 0.1, False, torch.bfloat16)
        got4 = run_batched(*ins4, 0.1, True, torch.bfloat16)
    finally:
        sb.set_carry_policy("save")
    for x, y in zip(want + want4, got + got4):
        assert np.array_equal(x, y)


@pytest.mark.parametrize("lengths", [[300, 200], [272, 129, 255]])
@pytest.mark.parametrize("D", [32, 64, 128])
@pytest.mark.parametrize("path", ["tensor", "simt"])
def test_non_finite_rows_outside_a_sequence_do_not_leak(path, D, lengths):
    """NaN in the rows behind the ragged end of a sequence (the pad behind the last sequence; the sequences that follow)
    must not reach the sequence's results: the kernels load whole 128-row tiles, and a zero weight does not silence a
    NaN.  Sequences of two and three tiles, so that off-diagonal steps see the ragged query tile too; ends in either
    64-row half of a tile, on a multiple of 16 rows, one row into a tile and one row short of one."""
    import stickbreaking_attention_b200 as sb
    H, T = 2, 768
    ends = np.cumsum(lengths)
    for poisoned in ("pad", "neighbour"):
        ins = [rounded(x, torch.bfloat16) for x in synth(H, T, D, seed=41)]
        lo, hi = (ends[-1], T) if poisoned == "pad" else (ends[0], T)
        clean = [x[:, :lo].copy() for x in ins]
        for x in ins:
            x[:, lo:hi] = np.nan
        sb.set_path(path)
        try:
            got = run_varlen(*ins, lengths, 0.1, False, torch.bfloat16)
        finally:
            sb.set_path("auto")
        kept = lengths if poisoned == "pad" else lengths[:1]
        want = oracle_varlen(*clean, kept, 0.1, False)
        assert_close(NAMES, [x[:, :lo] for x in got], want, TOL_BF16, f"NaN in the {poisoned}, {path} path, D={D}")


def test_empty_and_no_grad():
    from stickbreaking_attention_b200 import sb_attn_varlen
    q = torch.randn(2, 0, 64, device="cuda", dtype=torch.bfloat16)
    o, rem = sb_attn_varlen(q, q, q, torch.zeros(0, device="cuda", dtype=torch.int64), 0, zero_start=False)
    assert o.shape == (2, 0, 64) and rem.shape == (2, 0)
    q = torch.randn(2, 130, 64, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        o, rem = sb_attn_varlen(q, q, q, torch.tensor([0, 130], device="cuda"), 130)
    assert torch.isfinite(o.float()).all()


def test_tokens_outside_all_sequences_get_zero_gradients():
    """A pack whose last end is below T: the uncovered rows of dq, dk, dv are zero and covered rows are unaffected."""
    from stickbreaking_attention_b200 import sb_attn_varlen
    H, T, D = 2, 400, 64
    lengths = [150, 130]  # 280 of 400 tokens covered
    q, k, v, do, drem = [rounded(x, torch.bfloat16) for x in synth(H, T, D, seed=31)]
    tq, tk, tv = (torch.from_numpy(x).cuda().bfloat16().requires_grad_() for x in (q, k, v))
    cu = torch.tensor(np.cumsum(lengths), device="cuda")
    o, rem = sb_attn_varlen(tq, tk, tv, cu, max(lengths), zero_start=False)
    dq, dk, dv = torch.autograd.grad([o[:, :280], rem[:, :280]], [tq, tk, tv],
                                     [torch.from_numpy(do[:, :280]).cuda().bfloat16(),
                                      torch.from_numpy(drem[:, :280]).cuda().bfloat16()])
    for g in (dq, dk, dv):
        assert torch.all(g[:, 280:] == 0)
    want = oracle_varlen(q[:, :280], k[:, :280], v[:, :280], do[:, :280], drem[:, :280], lengths, 1 / math.sqrt(D), False)
    got = [x.detach().double().cpu().numpy()[:, :280] for x in (o, rem, dq, dk, dv)]
    assert_close(NAMES, got, want, TOL_BF16)


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_tensor_path_agrees_with_fp32_arithmetic_path_on_random_packs(seed):
    """Random ragged packs (many short sequences next to long ones, both head dims, both 16-bit types, both
    diagonal conventions): the tcgen05 kernels against the fp32-arithmetic kernels of the same library on the same
    16-bit inputs.  Sized beyond what the numpy oracle finishes quickly; exercises item transitions of the
    persistent kernels (sequences of 1 ... 3 tiles) and several items per block."""
    from stickbreaking_attention_b200 import get_path, sb_attn_varlen, set_path
    rng = np.random.default_rng(seed)
    D = [64, 128][seed % 2]
    dtype = [torch.bfloat16, torch.float16][(seed // 2) % 2]
    attend_current = bool(seed % 2)
    lengths = [int(x) for x in rng.integers(1, 400, size=40)] + [1500, 129, 128, 127, 1, 2600]
    H, T = 5, sum(lengths)
    g = torch.Generator().manual_seed(seed)
    q, k, v, do = (torch.randn(H, T, D, generator=g).to("cuda", dtype) for _ in range(4))
    dr = torch.randn(H, T, generator=g).to("cuda", dtype)
    cu = torch.tensor(np.cumsum(lengths), dtype=torch.int32, device="cuda")
    res = {}
    old = get_path()
    try:
        for path in ("tensor", "simt"):
            set_path(path)
            tq, tk, tv = (x.clone().requires_grad_() for x in (q, k, v))
            o, rem = sb_attn_varlen(tq, tk, tv, cu, max(lengths), zero_start=False, attend_current=attend_current)
            res[path] = [x.detach().float() for x in (o, rem) + torch.autograd.grad([o, rem], [tq, tk, tv], [do, dr])]
    finally:
        set_path(old)
    # both sides are rounded to 16 bits on output: allow one unit in the last place of bfloat16 on top of the bar
    for name, a_, b_ in zip(NAMES, res["tensor"], res["simt"]):
        excess = ((a_ - b_).abs() - (TOL_BF16 + b_.abs() * 2.0 ** -7)).max().item()
        assert excess <= 0, (name, excess)

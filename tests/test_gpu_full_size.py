"""GPU parity at the benchmark's full sizes (training shape, 65536-token sequence, 131072-token log-normal pack),
checked where the CPU oracle can follow: whole (head, sequence) pairs for sequences up to 4096 tokens, row slabs of
long sequences for o / rem / dq, and windows for dk / dv where the input distribution makes attention local."""
import math
import os
import sys

import numpy as np
import pytest
import torch

from util import TOL_BF16, assert_close
from oracle import sb_oracle as orc

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NAMES = ("o", "rem", "dq", "dk", "dv")


def make(H, T, D, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    q, k, v = ((torch.randn(H, T, D, generator=g) * scale).bfloat16() for _ in range(3))
    do = torch.randn(H, T, D, generator=g).bfloat16()
    drem = torch.randn(H, T, generator=g).bfloat16()
    return q, k, v, do, drem


def run(q, k, v, do, drem, lengths, it):
    from stickbreaking_attention_b200 import check_status, sb_attn_varlen
    tq, tk, tv = (x.cuda().requires_grad_() for x in (q, k, v))
    cu = torch.tensor(np.cumsum(lengths), device="cuda", dtype=torch.int32)
    o, rem = sb_attn_varlen(tq, tk, tv, cu, max(lengths), inv_temp=it, zero_start=False)
    dq, dk, dv = torch.autograd.grad([o, rem], [tq, tk, tv], [do.cuda(), drem.cuda()])
    torch.cuda.synchronize()
    check_status()
    return [x.detach().float().cpu().numpy().astype(np.float64) for x in (o, rem, dq, dk, dv)]


def f64(*xs):
    return [x.float().numpy().astype(np.float64) for x in xs]


def test_benchmark_pack_16384_every_sequence():
    """Config 2 at its own size: the seeded 16384-token pack of the default benchmark (head_dim 128, bf16, 2 of the 32
    heads, drem != 0), every sequence of both heads in full against the oracle.  Gradients reach magnitude 4 ... 5 here,
    where rounding the exact value to bfloat16 alone costs up to 1.5e-2 of the 2e-2 bar (measured on the oracle's own
    results: dq 1.3e-2, dv 1.5e-2), so the bar applies to the error beyond the output rounding (see assert_close)."""
    sys.path.insert(0, ROOT)
    import bench
    lengths = bench.workload("c2")["lengths"]
    assert lengths == [2943, 3503, 2192, 1807, 3696, 649, 1594]
    H, D, T = 2, 128, sum(lengths)
    q, k, v, do, drem = make(H, T, D, seed=0)
    it = 1 / math.sqrt(D)
    got = run(q, k, v, do, drem, lengths, it)
    start = 0
    for L in lengths:
        sl = (slice(None), slice(start, start + L))
        want = orc.sb_dense_bwd(*f64(q[sl], k[sl], v[sl], do[sl]), f64(drem[sl])[0], it)
        assert_close(NAMES, [x[sl] for x in got], want, TOL_BF16, f"c2 sequence at {start} len {L}", out_half_ulp=2.0 ** -8)
        start += L


def test_training_shape_8x4096():
    """Config 3: 8 sequences of 4096 tokens, head_dim 128 (4 of the 32 heads; one sequence checked in full)."""
    lengths = [4096] * 8
    H, D, T = 4, 128, 8 * 4096
    q, k, v, do, drem = make(H, T, D, seed=0)
    it = 1 / math.sqrt(D)
    got = run(q, k, v, do, drem, lengths, it)
    for h, s in ((0, 0), (3, 7), (1, 4)):
        a, b = s * 4096, (s + 1) * 4096
        sl = (slice(h, h + 1), slice(a, b))
        want = orc.sb_dense_bwd(*f64(q[sl], k[sl], v[sl], do[sl]), f64(drem[sl])[0], it)
        assert_close(NAMES, [x[sl] for x in got], want, TOL_BF16, f"head {h} seq {s}")


def test_long_context_65536():
    """Config 4: one 65536-token sequence, inputs 0.5*N(0,1) (2 of the 8 heads).  o, rem, dq on row slabs against
    the oracle with all keys to their left; dk, dv on windows: with these inputs beta is about 1/2, weights fall off
    like 2^-(i-j), so keys more than 256 positions away contribute less than 1e-70."""
    L, H, D = 65536, 2, 128
    q, k, v, do, drem = make(H, L, D, seed=0, scale=0.5)
    it = 1 / math.sqrt(D)
    got = run(q, k, v, do, drem, [L], it)
    Q, K, V, DO = f64(q, k, v, do)
    DR = f64(drem)[0]
    for lo, hi in ((0, 256), (30000, 30256), (65280, 65536)):
        o, rem = orc.sb_rows_fwd(Q, K, V, 0, lo, hi, it)
        dq = orc.sb_rows_dq(Q, K, V, DO, DR, 0, lo, hi, it)
        assert_close(("o", "rem", "dq"), [got[0][:, lo:hi], got[1][:, lo:hi], got[2][:, lo:hi]], [o, rem, dq], TOL_BF16,
                     f"rows {lo}:{hi}")
    for a, b in ((0, 512), (40000, 40512), (65024, 65536)):
        w0, w1 = max(0, a - 256), min(L, b + 256)
        sl = (slice(None), slice(w0, w1))
        res = orc.sb_dense_bwd(Q[sl], K[sl], V[sl], DO[sl], DR[sl], it)
        inner = slice(a - w0, b - w0)
        assert_close(("dk", "dv"), [got[3][:, a:b], got[4][:, a:b]], [res[3][:, inner], res[4][:, inner]], TOL_BF16,
                     f"keys {a}:{b}")


def test_lognormal_pack_131072():
    """Config 5: 70 sequences, 131072 tokens (2 of the 64 heads): every sequence up to 2048 tokens in full, the
    16384-token sequence on row slabs."""
    sys.path.insert(0, ROOT)
    import bench
    lengths = bench.workload("c5")["lengths"]
    H, D, T = 2, 128, sum(lengths)
    q, k, v, do, drem = make(H, T, D, seed=0)
    it = 1 / math.sqrt(D)
    got = run(q, k, v, do, drem, lengths, it)
    Q, K, V, DO = f64(q, k, v, do)
    DR = f64(drem)[0]
    ends = np.cumsum(lengths)
    starts = ends - np.asarray(lengths)
    checked = 0
    for a, b, L in zip(starts, ends, lengths):
        sl = (slice(None), slice(int(a), int(b)))
        if L <= 2048:
            want = orc.sb_dense_bwd(Q[sl], K[sl], V[sl], DO[sl], DR[sl], it)
            assert_close(NAMES, [x[sl] for x in got], want, TOL_BF16, f"sequence at {a} len {L}")
            checked += 1
        elif L == 16384:
            for lo, hi in ((0, 128), (8000, 8200), (16200, 16384)):
                o, rem = orc.sb_rows_fwd(Q, K, V, int(a), lo, hi, it)
                dq = orc.sb_rows_dq(Q, K, V, DO, DR, int(a), lo, hi, it)
                g = [got[0][:, a + lo:a + hi], got[1][:, a + lo:a + hi], got[2][:, a + lo:a + hi]]
                assert_close(("o", "rem", "dq"), g, [o, rem, dq], TOL_BF16, f"long sequence rows {lo}:{hi}")
    assert checked >= 40

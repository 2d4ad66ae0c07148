"""fuse_remainder=True: the first result is o + rem * v, formed in the kernels' epilogues; gradients flow through the
sum.  Checked against the CPU oracle (out = o + rem v; upstream gradient of rem becomes drem + do . v; dv gains
rem * do) in both layouts, and against the same expression built from the unfused operator."""
import math

import numpy as np
import pytest
import torch

from util import TOL_BF16, assert_close, rounded, synth
from oracle import sb_oracle as orc

pytestmark = pytest.mark.gpu
NAMES = ("out", "rem", "dq", "dk", "dv")


def _close(got, want):
    # both sides end in 16-bit roundings of differently associated sums: the bar plus one unit in the last place
    for name, a_, b_ in zip(NAMES, got, want):
        a_, b_ = a_.float(), b_.float()
        excess = ((a_ - b_).abs() - (TOL_BF16 + b_.abs() * 2.0 ** -7)).max().item()
        assert excess <= 0, (name, excess)


def _run(fn, q, k, v, dout, dr):
    q, k, v = (x.clone().requires_grad_() for x in (q, k, v))
    out, rem = fn(q, k, v)
    return [x.detach() for x in (out, rem) + torch.autograd.grad([out, rem], [q, k, v], [dout, dr])]


def _oracle_fused(q, k, v, dout, dr, lengths, it, attend_current):
    """float64 oracle of out = o + rem v and of its gradients for upstream (dout, dr): the operator itself receives
    do = dout and drem = dr + dout . v (the path through rem v), and dv gains rem * dout (the direct path)."""
    q, k, v, dout, dr = (np.asarray(x, dtype=np.float64) for x in (q, k, v, dout, dr))
    drem_eff = dr + (dout * v).sum(-1)
    o, rem, dq, dk, dv = orc.sb_varlen_fwd_bwd(q, k, v, dout, drem_eff, orc.ends_from_lengths(lengths), it, attend_current,
                                               np.float64)
    return o + rem[..., None] * v, rem, dq, dk, dv + rem[..., None] * dout


@pytest.mark.parametrize("D,dtype,attend_current", [(128, torch.bfloat16, False), (64, torch.float16, True)])
def test_varlen_fused_against_oracle(D, dtype, attend_current):
    from stickbreaking_attention_b200 import check_status, sb_attn_varlen
    lengths = [300, 1, 129, 640, 77, 128]
    H, T = 3, sum(lengths)
    ins = [rounded(x, dtype) for x in synth(H, T, D, 21)]
    q, k, v, dout, dr = (torch.from_numpy(x).to("cuda", dtype) for x in ins)
    cu = torch.tensor(np.cumsum(lengths), dtype=torch.int64, device="cuda")
    it = 1 / math.sqrt(D)
    got = _run(lambda q, k, v: sb_attn_varlen(q, k, v, cu, max(lengths), zero_start=False, attend_current=attend_current,
                                              fuse_remainder=True), q, k, v, dout, dr)
    check_status()
    want = _oracle_fused(*ins, lengths, it, attend_current)
    assert_close(NAMES, [x.double().cpu().numpy() for x in got], want, TOL_BF16, f"fused packed D={D}")


def test_varlen_fused_ignores_nan_behind_the_last_sequence():
    """The fused kernels with NaN in the pad behind the last sequence (the epilogues read v and dO rows themselves)."""
    from stickbreaking_attention_b200 import check_status, sb_attn_varlen
    lengths = [300, 200]
    H, T, D, used = 2, 640, 128, 500
    ins = [rounded(x, torch.bfloat16) for x in synth(H, T, D, 23)]
    clean = [x[:, :used].copy() for x in ins]
    for x in ins:
        x[:, used:] = np.nan
    q, k, v, dout, dr = (torch.from_numpy(x).to("cuda", torch.bfloat16) for x in ins)
    cu = torch.tensor(np.cumsum(lengths), dtype=torch.int64, device="cuda")
    got = _run(lambda q, k, v: sb_attn_varlen(q, k, v, cu, max(lengths), inv_temp=0.1, zero_start=False, fuse_remainder=True),
               q, k, v, dout, dr)
    check_status()
    want = _oracle_fused(*clean, lengths, 0.1, False)
    assert_close(NAMES, [x.double().cpu().numpy()[:, :used] for x in got], want, TOL_BF16, "fused packed, NaN pad")


def test_batched_fused_against_oracle():
    from stickbreaking_attention_b200 import check_status, sb_attn
    B, H, T, D = 2, 2, 300, 128
    ins = [rounded(x, torch.bfloat16) for x in synth(B * H, T, D, 4)]
    q, k, v, dout, dr = (torch.from_numpy(x.reshape((B, H) + x.shape[1:])).to("cuda", torch.bfloat16) for x in ins)
    got = _run(lambda q, k, v: sb_attn(q, k, v, fuse_remainder=True), q, k, v, dout, dr)
    check_status()
    # one sequence per (batch, head): the oracle sees B*H heads of one T-token sequence
    want = _oracle_fused(*ins, [T], 1 / math.sqrt(D), False)
    got = [x.double().cpu().numpy().reshape((B * H,) + tuple(x.shape[2:])) for x in got]
    assert_close(NAMES, got, want, TOL_BF16, "fused batched")


@pytest.mark.parametrize("D,dtype,attend_current", [(128, torch.bfloat16, False), (64, torch.float16, True)])
def test_varlen_fused_matches_composed(D, dtype, attend_current):
    from stickbreaking_attention_b200 import sb_attn_varlen
    lengths = [300, 1, 129, 640, 77, 128]
    H, T = 3, sum(lengths)
    q, k, v, dout, dr = (torch.from_numpy(x).to("cuda", dtype) for x in synth(H, T, D, 21))
    cu = torch.tensor(np.cumsum(lengths), dtype=torch.int64, device="cuda")

    def composed(q, k, v):
        o, rem = sb_attn_varlen(q, k, v, cu, max(lengths), zero_start=False, attend_current=attend_current)
        return o.float() + rem.float()[..., None] * v.float(), rem

    def fused(q, k, v):
        return sb_attn_varlen(q, k, v, cu, max(lengths), zero_start=False, attend_current=attend_current,
                              fuse_remainder=True)

    want = _run(composed, q, k, v, dout.float(), dr)
    got = _run(fused, q, k, v, dout, dr)
    _close(got, want)


def test_batched_fused_matches_composed():
    from stickbreaking_attention_b200 import sb_attn
    B, H, T, D = 2, 2, 300, 128
    g = torch.Generator().manual_seed(4)
    q, k, v, dout = (torch.randn(B, H, T, D, generator=g).to("cuda", torch.bfloat16) for _ in range(4))
    dr = torch.randn(B, H, T, generator=g).to("cuda", torch.bfloat16)

    def composed(q, k, v):
        o, rem = sb_attn(q, k, v)
        return o.float() + rem.float()[..., None] * v.float(), rem

    want = _run(composed, q, k, v, dout.float(), dr)
    got = _run(lambda q, k, v: sb_attn(q, k, v, fuse_remainder=True), q, k, v, dout, dr)
    _close(got, want)


def test_fused_falls_back_for_float32_inputs():
    """The fp32-arithmetic kernels have no fused epilogue: the Python layer forms the sum itself, same results."""
    from stickbreaking_attention_b200 import sb_attn_varlen
    lengths = [100, 156]
    H, T, D = 2, 256, 64
    q, k, v, dout, dr = (torch.from_numpy(x).cuda() for x in synth(H, T, D, 8))
    cu = torch.tensor(np.cumsum(lengths), dtype=torch.int32, device="cuda")
    want = _run(lambda q, k, v: (lambda o, rem: (o + rem[..., None] * v, rem))(
        *sb_attn_varlen(q, k, v, cu, max(lengths), zero_start=False)), q, k, v, dout, dr)
    got = _run(lambda q, k, v: sb_attn_varlen(q, k, v, cu, max(lengths), zero_start=False, fuse_remainder=True),
               q, k, v, dout, dr)
    for a_, b_ in zip(got, want):
        assert torch.equal(a_, b_)

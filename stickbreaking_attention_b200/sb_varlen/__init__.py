"""Packed variable-length stick-breaking attention with the reference's Python interface
(stickbreaking_attention/sb_varlen/__init__.py:23-81)."""
import math

import torch

from ..ops import fusable, get_carry_policy, varlen_bwd, varlen_fwd


class StickBreakingAttention(torch.autograd.Function):
    """Same argument order and return values as the reference's Function (sb_varlen/__init__.py:26,48)."""

    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, max_seqlens, inv_temp, attend_current, fuse_remainder=False):
        no_grad = not any(ctx.needs_input_grad[:3])
        ctx.recompute = not no_grad and get_carry_policy() == "recompute"  # see ops.set_carry_policy
        o, rem, neg_log_acc, workspace = varlen_fwd(q, k, v, cu_seqlens, max_seqlens, inv_temp,
                                                    attend_current=attend_current, no_grad=no_grad or ctx.recompute,
                                                    fuse_remainder=fuse_remainder)
        ctx.save_for_backward(q, k, v, cu_seqlens, rem if ctx.recompute else workspace, rem)
        ctx.fuse_remainder = fuse_remainder
        ctx.logit_scale = inv_temp
        ctx.max_seqlens = max_seqlens
        ctx.attend_current = attend_current
        return o, rem

    @staticmethod
    def backward(ctx, do, drem):
        q, k, v, cu_seqlens, workspace, rem = ctx.saved_tensors
        if ctx.recompute:  # rebuild the carries: the forward once more, its o and rem dropped
            workspace = varlen_fwd(q, k, v, cu_seqlens, ctx.max_seqlens, ctx.logit_scale, attend_current=ctx.attend_current,
                                   fuse_remainder=ctx.fuse_remainder)[3]
        if do is None:
            do = torch.zeros_like(q)
        if drem is None:
            drem = torch.zeros(q.shape[:-1], dtype=q.dtype, device=q.device)
        dq, dk, dv = varlen_bwd(do, drem, q, k, v, cu_seqlens, ctx.max_seqlens, workspace, ctx.logit_scale,
                                attend_current=ctx.attend_current, fuse_remainder=ctx.fuse_remainder, rem=rem)
        return dq, dk, dv, None, None, None, None, None


def sb_attn_varlen(q, k, v, cu_seqlens, max_seqlens=None, inv_temp=None, zero_start=True, attend_current=False,
                   fuse_remainder=False):
    """q, k, v: [H, T, D]; cu_seqlens: cumulative sequence boundaries (with a leading 0 iff ``zero_start``).

    ``max_seqlens`` may be omitted (the reference's README calls it that way); it is then read from the device,
    which costs one synchronisation.  Returns (o, rem); callers usually form ``o + rem[..., None] * v``
    (tests/test_varlen.py:103 of the reference): with ``fuse_remainder=True`` (no counterpart in the reference) the first
    result is that sum already, computed in the kernels' epilogues, and the backward accounts for it."""
    if zero_start:
        assert cu_seqlens[0] == 0
        cu_seqlens = cu_seqlens[1:]
    if inv_temp is None:
        inv_temp = 1 / math.sqrt(q.size(-1))
    if fuse_remainder and not fusable(q, k, v):  # fp32-arithmetic kernels: the same sum, formed here
        o, rem = sb_attn_varlen_(q, k, v, inv_temp, cu_seqlens, max_seqlens, attend_current)
        return o + rem[..., None] * v, rem
    return sb_attn_varlen_(q, k, v, inv_temp, cu_seqlens, max_seqlens, attend_current, fuse_remainder)


def sb_attn_varlen_(q, k, v, inv_temp, cu_seqlens, max_seqlens, attend_current, fuse_remainder=False):
    return StickBreakingAttention.apply(q, k, v, cu_seqlens, max_seqlens, inv_temp, attend_current, fuse_remainder)

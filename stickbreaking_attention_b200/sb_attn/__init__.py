"""Batched stick-breaking attention with the reference's Python interface
(stickbreaking_attention/sb_attn/__init__.py:15-63)."""
import math

import torch

from ..ops import attn_bwd, attn_fwd, fusable, get_carry_policy


class StickBreakingAttention(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, v, inv_temp, attend_current=False, fuse_remainder=False):
        no_grad = not any(ctx.needs_input_grad[:3])
        ctx.recompute = not no_grad and get_carry_policy() == "recompute"  # see ops.set_carry_policy
        o, rem, neg_log_acc, workspace = attn_fwd(q, k, v, inv_temp, attend_current=attend_current,
                                                  no_grad=no_grad or ctx.recompute, fuse_remainder=fuse_remainder)
        ctx.save_for_backward(q, k, v, rem if ctx.recompute else workspace, rem)
        ctx.fuse_remainder = fuse_remainder
        ctx.logit_scale = inv_temp
        ctx.attend_current = attend_current
        return o, rem

    @staticmethod
    def backward(ctx, do, drem):
        q, k, v, workspace, rem = ctx.saved_tensors
        if ctx.recompute:  # rebuild the carries: the forward once more, its o and rem dropped
            workspace = attn_fwd(q, k, v, ctx.logit_scale, attend_current=ctx.attend_current,
                                 fuse_remainder=ctx.fuse_remainder)[3]
        if do is None:
            do = torch.zeros_like(q)
        if drem is None:
            drem = torch.zeros(q.shape[:-1], dtype=q.dtype, device=q.device)
        dq, dk, dv = attn_bwd(do, drem, q, k, v, workspace, ctx.logit_scale, attend_current=ctx.attend_current,
                              fuse_remainder=ctx.fuse_remainder, rem=rem)
        return dq, dk, dv, None, None, None


def sb_attn(q, k, v, inv_temp=None, zero_start=True, attend_current=False, fuse_remainder=False):
    """q, k, v: [B, H, T, D].  ``zero_start`` is accepted and ignored, as in the reference (sb_attn/__init__.py:56-59).
    ``fuse_remainder=True`` (no counterpart in the reference) returns ``o + rem[..., None] * v`` as the first result."""
    if inv_temp is None:
        inv_temp = 1 / math.sqrt(q.size(-1))
    if fuse_remainder and not fusable(q, k, v):  # fp32-arithmetic kernels: the same sum, formed here
        o, rem = sb_attn_(q, k, v, inv_temp, attend_current=attend_current)
        return o + rem[..., None] * v, rem
    return sb_attn_(q, k, v, inv_temp, attend_current=attend_current, fuse_remainder=fuse_remainder)


def sb_attn_(q, k, v, inv_temp, attend_current, fuse_remainder=False):
    return StickBreakingAttention.apply(q, k, v, inv_temp, attend_current, fuse_remainder)

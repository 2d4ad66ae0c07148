"""Packed variable-length stick-breaking attention with the reference's Python interface
(stickbreaking_attention/sb_varlen/__init__.py:23-81)."""
import math

import torch

from ..ops import varlen_bwd, varlen_fwd


class StickBreakingAttention(torch.autograd.Function):
    """Same argument order and return values as the reference's Function (sb_varlen/__init__.py:26,48)."""

    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, max_seqlens, inv_temp, attend_current):
        no_grad = not any(ctx.needs_input_grad[:3])
        o, rem, neg_log_acc, workspace = varlen_fwd(q, k, v, cu_seqlens, max_seqlens, inv_temp,
                                                    attend_current=attend_current, no_grad=no_grad)
        ctx.save_for_backward(q, k, v, cu_seqlens, workspace)
        ctx.logit_scale = inv_temp
        ctx.max_seqlens = max_seqlens
        ctx.attend_current = attend_current
        return o, rem

    @staticmethod
    def backward(ctx, do, drem):
        q, k, v, cu_seqlens, workspace = ctx.saved_tensors
        if do is None:
            do = torch.zeros_like(q)
        if drem is None:
            drem = torch.zeros(q.shape[:-1], dtype=q.dtype, device=q.device)
        dq, dk, dv = varlen_bwd(do, drem, q, k, v, cu_seqlens, ctx.max_seqlens, workspace, ctx.logit_scale,
                                attend_current=ctx.attend_current)
        return dq, dk, dv, None, None, None, None


def sb_attn_varlen(q, k, v, cu_seqlens, max_seqlens=None, inv_temp=None, zero_start=True, attend_current=False):
    """q, k, v: [H, T, D]; cu_seqlens: cumulative sequence boundaries (with a leading 0 iff ``zero_start``).

    ``max_seqlens`` may be omitted (the reference's README calls it that way); it is then read from the device,
    which costs one synchronisation.  Returns (o, rem); callers usually form ``o + rem[..., None] * v``."""
    if zero_start:
        assert cu_seqlens[0] == 0
        cu_seqlens = cu_seqlens[1:]
    if inv_temp is None:
        inv_temp = 1 / math.sqrt(q.size(-1))
    return sb_attn_varlen_(q, k, v, inv_temp, cu_seqlens, max_seqlens, attend_current)


def sb_attn_varlen_(q, k, v, inv_temp, cu_seqlens, max_seqlens, attend_current):
    return StickBreakingAttention.apply(q, k, v, cu_seqlens, max_seqlens, inv_temp, attend_current)

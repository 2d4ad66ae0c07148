"""CPU restatement of the reference's dense stick-breaking attention.  TEST INFRASTRUCTURE ONLY.

Parity status: PINNED.  ``tests/golden/make_golden.py`` imports the reference's own
``stickbreaking_attention/sb_ref.py`` (function ``stickbreaking``, lines 8-25), runs it forward and,
through autograd, backward on seeded inputs and stores the results under ``tests/golden/``;
``tests/test_oracle.py`` checks every function of this file against those fixtures.

What is restated, with the reference lines each step follows:

* forward  -- ``stickbreaking_attention/sb_ref.py:12-25``: logits = q k^T / temperature (:12), computed in
  float32 inside the reference (:16); ``log_z = logsigmoid(logits)`` masked (:17); ``log_beta =
  logsigmoid(-logits)`` masked to 0 (:19); exclusive suffix sum over the keys to the right, written there as a
  matmul with a strictly-lower-triangular ones matrix (:21-22); ``att = exp(log_z + suffix)`` (:23-24);
  ``o = att v`` and ``rem = 1 - sum(att)`` (:25).
* per-sequence driving of a packed batch -- ``tests/test_varlen.py:11-28`` (split the token axis by the lengths,
  mask ``triu(0)`` for strict causality and ``triu(1)`` when the current token may be attended).
* backward -- the closed form the reference's Triton kernel implements,
  ``stickbreaking_attention/sb_varlen/sb_varlen_bwd.py:438-452``:
  ``g = att * (do v^T - drem)`` (:438-439), inclusive prefix of g over keys (:440-445),
  ``ds = g - sigmoid(logits) * prefix`` (:446-447), ``dq = scale * ds k`` (:449,:475),
  ``dk = scale * ds^T q`` (:450-451), ``dv = att^T do`` (:452).

Everything is numpy; ``dtype`` selects float32 (what the reference computes in) or float64 (a tighter
yard-stick for the float32-input mode of the CUDA path).
"""
from __future__ import annotations

import numpy as np

__all__ = [
    "logsigmoid", "sb_dense_fwd", "sb_dense_bwd", "sb_varlen_fwd", "sb_varlen_fwd_bwd",
    "sb_batched_fwd_bwd", "sb_rows_fwd", "sb_rows_dq", "ends_from_lengths",
]


def logsigmoid(x):
    """log(sigmoid(x)) without overflow: min(x,0) - log1p(exp(-|x|)) (torch's formula for F.logsigmoid)."""
    return np.minimum(x, 0) - np.log1p(np.exp(-np.abs(x)))


def _masked(L_q, L_k, row0, attend_current):
    """Boolean [L_q, L_k] matrix, True where key j may NOT be used by query row0+i.

    ``tests/test_varlen.py:14`` builds ``triu(0)`` (j >= i masked) or ``triu(1)`` (j > i masked)."""
    i = np.arange(row0, row0 + L_q)[:, None]
    j = np.arange(L_k)[None, :]
    return (j > i) if attend_current else (j >= i)


def _suffix_exclusive(x, faithful):
    """sum over keys strictly to the right (``sb_ref.py:21-22``).

    ``faithful`` multiplies by the triangular ones matrix exactly as the reference does (O(L^3) per head);
    otherwise a reversed cumulative sum gives the same numbers in O(L^2)."""
    if faithful:
        L = x.shape[-1]
        cum_weight = np.tril(np.ones((L, L), dtype=x.dtype), -1)
        return x @ cum_weight
    rev = np.cumsum(x[..., ::-1], axis=-1)[..., ::-1]
    return rev - x


def sb_dense_fwd(q, k, v, inv_temp, attend_current=False, dtype=np.float64, row0=0, faithful=False,
                 return_att=False):
    """One sequence.  q [H, Lq, D] are query rows row0..row0+Lq-1 of the sequence, k,v [H, Lk, D] its keys 0..Lk-1.

    Returns (o [H,Lq,D], rem [H,Lq]) and, on request, the attention matrix and sigmoid(logits)."""
    q = np.asarray(q, dtype=dtype)
    k = np.asarray(k, dtype=dtype)
    v = np.asarray(v, dtype=dtype)
    logits = np.matmul(q, np.swapaxes(k, -1, -2)) * dtype(inv_temp)
    m = _masked(q.shape[-2], k.shape[-2], row0, attend_current)
    log_z = np.where(m, dtype(-1e5), logsigmoid(logits))
    log_beta = np.where(m, dtype(0), logsigmoid(-logits))
    att = np.exp(log_z + _suffix_exclusive(log_beta, faithful))
    o = np.matmul(att, v)
    rem = 1 - att.sum(-1)
    if return_att:
        beta = np.where(m, dtype(0), np.exp(logsigmoid(logits)))
        return o, rem, att, beta
    return o, rem


def sb_dense_bwd(q, k, v, do, drem, inv_temp, attend_current=False, dtype=np.float64, row0=0):
    """Gradients of one sequence (or of a slab of its query rows).

    Returns dq for the given rows and the CONTRIBUTION of those rows to dk and dv (sum over slabs = total)."""
    o, rem, att, beta = sb_dense_fwd(q, k, v, inv_temp, attend_current, dtype, row0, return_att=True)
    q = np.asarray(q, dtype=dtype)
    k = np.asarray(k, dtype=dtype)
    v = np.asarray(v, dtype=dtype)
    do = np.asarray(do, dtype=dtype)
    drem = np.asarray(drem, dtype=dtype)
    g = att * (np.matmul(do, np.swapaxes(v, -1, -2)) - drem[..., None])
    ds = g - beta * np.cumsum(g, axis=-1)
    dq = np.matmul(ds, k) * dtype(inv_temp)
    dk = np.matmul(np.swapaxes(ds, -1, -2), q) * dtype(inv_temp)
    dv = np.matmul(np.swapaxes(att, -1, -2), do)
    return o, rem, dq, dk, dv


def ends_from_lengths(lengths):
    """cumulative sequence ends without a leading zero (the layout ``varlen_fwd`` receives)."""
    return np.cumsum(np.asarray(lengths, dtype=np.int64))


def _bounds(cu_ends):
    ends = [int(e) for e in np.asarray(cu_ends).tolist()]
    starts = [0] + ends[:-1]
    return list(zip(starts, ends))


def sb_varlen_fwd(q, k, v, cu_ends, inv_temp, attend_current=False, dtype=np.float64, faithful=False):
    """Packed layout [H, T, D]; ``cu_ends`` are cumulative sequence ends (no leading 0)."""
    H, T, D = q.shape
    o = np.zeros((H, T, D), dtype=dtype)
    rem = np.ones((H, T), dtype=dtype)
    for a, b in _bounds(cu_ends):
        if b > a:
            o[:, a:b], rem[:, a:b] = sb_dense_fwd(q[:, a:b], k[:, a:b], v[:, a:b], inv_temp, attend_current,
                                                  dtype, faithful=faithful)
    return o, rem


def sb_varlen_fwd_bwd(q, k, v, do, drem, cu_ends, inv_temp, attend_current=False, dtype=np.float64):
    H, T, D = q.shape
    o = np.zeros((H, T, D), dtype=dtype)
    rem = np.ones((H, T), dtype=dtype)
    dq = np.zeros((H, T, D), dtype=dtype)
    dk = np.zeros((H, T, D), dtype=dtype)
    dv = np.zeros((H, T, D), dtype=dtype)
    for a, b in _bounds(cu_ends):
        if b > a:
            s = slice(a, b)
            o[:, s], rem[:, s], dq[:, s], dk[:, s], dv[:, s] = sb_dense_bwd(
                q[:, s], k[:, s], v[:, s], do[:, s], drem[:, s], inv_temp, attend_current, dtype)
    return o, rem, dq, dk, dv


def sb_batched_fwd_bwd(q, k, v, do, drem, inv_temp, attend_current=False, dtype=np.float64):
    """Batched layout [B, H, T, D] (``stickbreaking_attention/sb_attn/__init__.py:56``): every batch entry is one sequence."""
    outs = [sb_dense_bwd(q[b], k[b], v[b], do[b], drem[b], inv_temp, attend_current, dtype)
            for b in range(q.shape[0])]
    return tuple(np.stack([x[i] for x in outs]) for i in range(5))


def sb_rows_fwd(q, k, v, a, lo, hi, inv_temp, attend_current=False, dtype=np.float64):
    """Rows lo..hi-1 (relative to the sequence start ``a``) of one long sequence: only keys a..a+hi-1 are touched."""
    return sb_dense_fwd(q[:, a + lo:a + hi], k[:, a:a + hi], v[:, a:a + hi], inv_temp, attend_current, dtype,
                        row0=lo)


def sb_rows_dq(q, k, v, do, drem, a, lo, hi, inv_temp, attend_current=False, dtype=np.float64):
    """dq of rows lo..hi-1 of a long sequence (dq of a row needs that row's keys only)."""
    res = sb_dense_bwd(q[:, a + lo:a + hi], k[:, a:a + hi], v[:, a:a + hi], do[:, a + lo:a + hi],
                       drem[:, a + lo:a + hi], inv_temp, attend_current, dtype, row0=lo)
    return res[2]

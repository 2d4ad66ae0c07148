"""Helpers shared by the GPU parity tests: run the CUDA path through the public API and the oracle on the same data."""
import numpy as np
import torch

from oracle import sb_oracle as orc

TOL_BF16 = 2e-2   # max-abs bar for bf16 inputs against an fp32/fp64 reference of the same (rounded) inputs
TOL_F32 = 1e-5    # max-abs bar in the float32-input mode


def to_dev(x, dtype, device="cuda"):
    return torch.from_numpy(np.ascontiguousarray(x)).to(device=device, dtype=dtype)


def run_varlen(q, k, v, do, drem, lengths, inv_temp, attend_current, dtype, zero_start=False, cu_dtype=torch.int64,
               max_seqlens="given"):
    """numpy in, numpy (float64) out: o, rem, dq, dk, dv from sb_attn_varlen + autograd."""
    from stickbreaking_attention_b200 import sb_attn_varlen
    tq, tk, tv = (to_dev(x, dtype).requires_grad_() for x in (q, k, v))
    tdo, tdr = to_dev(do, dtype), to_dev(drem, dtype)
    ends = np.cumsum(np.asarray(lengths, dtype=np.int64))
    cu = np.concatenate([[0], ends]) if zero_start else ends
    cu = torch.from_numpy(cu).to(device="cuda", dtype=cu_dtype)
    ms = int(max(lengths)) if max_seqlens == "given" else max_seqlens
    o, rem = sb_attn_varlen(tq, tk, tv, cu, ms, inv_temp=inv_temp, zero_start=zero_start,
                            attend_current=attend_current)
    dq, dk, dv = torch.autograd.grad([o, rem], [tq, tk, tv], [tdo, tdr])
    torch.cuda.synchronize()
    return [x.detach().double().cpu().numpy() for x in (o, rem, dq, dk, dv)]


def run_batched(q, k, v, do, drem, inv_temp, attend_current, dtype):
    from stickbreaking_attention_b200 import sb_attn
    tq, tk, tv = (to_dev(x, dtype).requires_grad_() for x in (q, k, v))
    tdo, tdr = to_dev(do, dtype), to_dev(drem, dtype)
    o, rem = sb_attn(tq, tk, tv, inv_temp=inv_temp, attend_current=attend_current)
    dq, dk, dv = torch.autograd.grad([o, rem], [tq, tk, tv], [tdo, tdr])
    torch.cuda.synchronize()
    return [x.detach().double().cpu().numpy() for x in (o, rem, dq, dk, dv)]


def oracle_varlen(q, k, v, do, drem, lengths, inv_temp, attend_current):
    return orc.sb_varlen_fwd_bwd(q, k, v, do, drem, orc.ends_from_lengths(lengths), inv_temp, attend_current,
                                 np.float64)


MARGINS = []   # (test id, what, tensor, max-abs error, bar): printed by conftest.py at the end of the run


def note_margin(what, name, err, tol):
    """Puts a measured max-abs error on record (the terminal summary lists them all with their bars)."""
    import os
    test = os.environ.get("PYTEST_CURRENT_TEST", "").split(" ")[0]
    MARGINS.append((test, what, name, float(err), float(tol)))
    print(f"parity {what} {name}: max-abs {float(err):.3e} (bar {tol:g})")


def assert_close(names, got, want, tol, what="", out_half_ulp=0.0):
    """max-abs error of every tensor against the bar `tol`.  `out_half_ulp` (2**-8 for bfloat16 results) adds what
    storing the exact value in the output type would cost, |want| * out_half_ulp, to the bar of each element: a
    bfloat16 result of magnitude 4 ... 8 is off by up to 1.6e-2 from rounding alone, whatever computed it.  The strict
    max-abs error is what goes on record either way."""
    for n, g, w in zip(names, got, want):
        assert np.isfinite(g).all(), (what, n, "non-finite output")
        err = np.abs(g - w).max() if g.size else 0.0
        note_margin(what, n, err, tol)
        if out_half_ulp:
            excess = (np.abs(g - w) - np.abs(w) * out_half_ulp).max() if g.size else 0.0
            assert excess <= tol, (what, n, float(err), float(excess), tol)
        else:
            assert err <= tol, (what, n, float(err), tol)


def rounded(x, dtype):
    """numpy float32 array rounded to dtype and back (what the kernel sees)."""
    return torch.from_numpy(np.ascontiguousarray(x)).to(dtype).float().numpy()


def synth(H, T, D, seed, dist="normal", scale=1.0):
    g = torch.Generator().manual_seed(seed)

    def randn(*s):
        return torch.randn(*s, generator=g, dtype=torch.float32)

    if dist == "normal":
        q, k, v = randn(H, T, D) * scale, randn(H, T, D) * scale, randn(H, T, D) * scale
    else:
        v = 0.25 * randn(H, T, D)
        q = 0.25 * (randn(H, T, D) + 1)
        k = 0.25 * (randn(H, T, D) - 1)
    do, drem = randn(H, T, D), randn(H, T)
    return [x.numpy() for x in (q, k, v, do, drem)]

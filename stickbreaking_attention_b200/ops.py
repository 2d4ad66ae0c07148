"""Host launchers with the reference's names and argument meaning, on top of the C ABI.

``varlen_fwd`` / ``varlen_bwd`` mirror stickbreaking_attention/sb_varlen/sb_varlen_fwd.py:411 and
sb_varlen_bwd.py:483; ``attn_fwd`` / ``attn_bwd`` mirror sb_attn/sb_fwd.py:137 (``_fwd``) and sb_bwd.py:162
(``_bwd``).  Differences that a caller can see: the forward returns one more value, an opaque workspace that
the backward needs (the tile table and the per-tile carries), and gradients of the batched layout keep the input
dtype instead of being forced to bfloat16 (sb_bwd.py:172-173).
"""
import ctypes
import os

import torch

from . import _lib
from ._lib import SbMat, SbParams, SbVec

_DTYPES = {torch.bfloat16: _lib.SBATTN_BF16, torch.float32: _lib.SBATTN_F32, torch.float16: _lib.SBATTN_F16}
_PATHS = {"auto": _lib.PATH_AUTO, "simt": _lib.PATH_SIMT, "tensor": _lib.PATH_TENSOR}
_status_words = {}
_forced_path = os.environ.get("SBATTN_PATH", "auto")


_carry_policy = os.environ.get("SBATTN_CARRIES", "save")


def set_carry_policy(name):
    """What the autograd functions keep between forward and backward.

    'save' (default): the forward's workspace with the per-tile carries, two floats per query row and 64 keys.  That is
    H * sum(ceil(len / 128) * (ceil(len / 128) + 1)) KiB: 95 MB for the 16384-token benchmark pack of 32 heads, 2 GB for one
    65536-token sequence of 8 heads; it grows with the square of the sequence length, where the reference keeps 4 bytes per
    row (its neg_log_acc, sb_varlen/__init__.py:41).
    'recompute': nothing beyond q, k, v and rem; the backward runs the forward kernel once more to rebuild the carries
    in scratch memory that lives only for the backward call.  Costs one forward (about a fifth of forward + backward),
    keeps the memory held between the two passes linear in the sequence length.  Same gradients, bit for bit."""
    global _carry_policy
    if name not in ("save", "recompute"):
        raise ValueError(name)
    _carry_policy = name


def get_carry_policy():
    return _carry_policy


def set_path(name):
    """'auto' (default), 'simt' (fp32-arithmetic kernels) or 'tensor' (tcgen05 kernels or an error)."""
    global _forced_path
    if name not in _PATHS:
        raise ValueError(name)
    _forced_path = name


def get_path():
    return _forced_path


def status_word(device):
    """int32 device word the kernels OR their SBATTN_ST_* bits into (one per device, never reset by the library)."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _status_words:
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
    return _status_words[key]


def check_status(device=None, reset=True):
    """Synchronises and raises if a kernel reported bad sequence ends or a wait that ran out."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = status_word(device)
    val = int(w.item())
    if reset:
        w.zero_()
    if val & _lib.ST_BAD_SEQLENS:
        raise ValueError("cu_seqlens rejected on the device: ends must be non-decreasing, at most the number of "
                         "tokens, and no sequence longer than max_seqlens")
    if val & _lib.ST_TIMEOUT:
        raise RuntimeError("a stick-breaking attention kernel gave up waiting (results are invalid)")
    return val


def launch_count():
    """Kernels the library has launched in this process so far (sbattn_launch_count)."""
    return int(_lib.lib().sbattn_launch_count())


def _require_cuda(*tensors):
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("stick-breaking attention runs on CUDA tensors only (there is no CPU implementation)")


def _mat(t, batched):
    if t is None:
        return SbMat(None, 0, 0, 0)
    if batched:
        return SbMat(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))
    return SbMat(t.data_ptr(), 0, t.stride(0), t.stride(1))


def _vec(t, batched):
    if t is None:
        return SbVec(None, 0, 0, 0)
    if batched:
        return SbVec(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))
    return SbVec(t.data_ptr(), 0, t.stride(0), t.stride(1))


def _unit_inner(t):
    return t if t.stride(-1) == 1 else t.contiguous()


def _empty_like_rows(t):
    out = torch.empty_like(t)
    return out if out.stride(-1) == 1 else torch.empty(t.shape, dtype=t.dtype, device=t.device)


def _base_params(q, batched, cu_seqlens, max_seqlens, logit_scale, attend_current, save_carries, fused=False):
    if q.dtype not in _DTYPES:
        raise TypeError(f"unsupported dtype {q.dtype}")
    p = SbParams()
    p.dtype = _DTYPES[q.dtype]
    p.path = _PATHS[_forced_path]
    if batched:
        B, H, T, D = q.shape
        p.batch, p.num_seqs, p.cu_width, p.cu_seqlens, p.max_seqlen = B, 0, 4, None, T
    else:
        H, T, D = q.shape
        p.batch = 0
        p.num_seqs = cu_seqlens.numel()
        p.cu_width = cu_seqlens.element_size()
        p.cu_seqlens = cu_seqlens.data_ptr()
        p.max_seqlen = int(max_seqlens)
    p.heads, p.tokens, p.head_dim = H, T, D
    p.attend_current = int(bool(attend_current))
    p.inv_temp = float(logit_scale)
    p.save_carries = int(bool(save_carries))
    p.flags = _lib.FLAG_FUSED_REMAINDER if fused else 0
    p.status = status_word(q.device).data_ptr()
    p.stream = torch.cuda.current_stream(q.device).cuda_stream
    return p


def _workspace_sizes(p):
    fb, bb = ctypes.c_size_t(0), ctypes.c_size_t(0)
    _lib.check(_lib.lib().sbattn_workspace_bytes(ctypes.byref(p), ctypes.byref(fb), ctypes.byref(bb)),
               "sbattn_workspace_bytes")
    return fb.value, bb.value


def _check_qkv(q, k, v, ndim):
    if q.dim() != ndim or k.shape != q.shape or v.shape != q.shape:
        raise ValueError(f"q, k, v must share one {ndim}-d shape, got {tuple(q.shape)} {tuple(k.shape)} {tuple(v.shape)}")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("q, k, v must share one dtype")
    if k.device != q.device or v.device != q.device:
        raise ValueError("q, k, v must live on one device")
    if q.size(-1) > 128:
        raise ValueError("head_dim above 128 is not supported")


def _prep_cu(cu_seqlens, q, max_seqlens):
    if cu_seqlens.dtype not in (torch.int32, torch.int64):
        raise TypeError("cu_seqlens must be int32 or int64")
    if cu_seqlens.dim() != 1:
        raise ValueError("cu_seqlens must be 1-d")
    if cu_seqlens.device != q.device:
        cu_seqlens = cu_seqlens.to(q.device)
    cu_seqlens = cu_seqlens.contiguous()
    if max_seqlens is None:
        # one device-to-host read, exactly what callers of the reference do to obtain this argument
        if cu_seqlens.numel() == 0:
            max_seqlens = 0
        else:
            lens = torch.diff(cu_seqlens, prepend=cu_seqlens.new_zeros(1))
            max_seqlens = int(lens.max().item())
    return cu_seqlens, int(max_seqlens)


def workspace_bytes(batched, n_seqs, heads, tokens, max_seqlens, save_carries=True):
    """(forward, backward) workspace sizes in bytes: the formula of sbattn_workspace_bytes restated in Python, so that
    a traced program (torch.compile) can size the buffers without calling into the library."""
    tile = 128
    up = lambda x: (x + 255) // 256 * 256
    maxlen = tokens if batched else (min(max_seqlens, tokens) if max_seqlens > 0 else tokens)
    n_max = max(1, (maxlen + tile - 1) // tile)
    if batched:
        max_items = n_seqs * n_max
        slot_cap = n_seqs * n_max * (n_max + 1)
    else:
        max_items = tokens // tile + n_seqs
        slot_cap = max_items * (n_max + 1)
    off = 256                               # header
    off = up(off + 16 * n_seqs)             # sequence table
    off = up(off + 8 * max_items)           # item table
    off = up(off + 4 * 2 * (n_max + 2))     # histogram scratch
    carry = 4 * heads * 2 * slot_cap * tile  # two 32-key carries per 64-key slot
    drem = 4 * heads * tokens * (n_seqs if batched else 1)  # drem + do . v per row (fused-remainder backward)
    return off + (carry if save_carries else 0), up(carry) + up(drem)


def _forward_into(q, k, v, batched, cu_seqlens, max_seqlens, logit_scale, attend_current, no_grad, o, rem, neg_log_acc,
                  ws, fused=False):
    """The forward into buffers that exist already (what the registered operators do)."""
    with torch.cuda.device(q.device):
        p = _base_params(q, batched, cu_seqlens, max_seqlens, logit_scale, attend_current, not no_grad, fused)
        p.q, p.k, p.v, p.o = _mat(q, batched), _mat(k, batched), _mat(v, batched), _mat(o, batched)
        p.rem, p.neg_log_acc = _vec(rem, batched), _vec(neg_log_acc, batched)
        p.fwd_workspace, p.fwd_workspace_bytes = ws.data_ptr(), ws.numel()
        _lib.check(_lib.lib().sbattn_fwd(ctypes.byref(p)), "sbattn_fwd")
        if os.environ.get("SBATTN_CHECK_STATUS") == "1":
            check_status(q.device)


def _backward_into(do, dr, q, k, v, batched, cu_seqlens, max_seqlens, ws, logit_scale, attend_current, phases, dq, dk,
                   dv, bws, fused=False, rem=None):
    with torch.cuda.device(q.device):
        p = _base_params(q, batched, cu_seqlens, max_seqlens, logit_scale, attend_current, True, fused)
        if fused:
            p.rem = _vec(rem, batched)
        p.bwd_phases = phases
        fwd_bytes, bwd_bytes = _workspace_sizes(p)
        if ws.numel() < fwd_bytes:
            raise ValueError("the forward workspace does not belong to this problem (was the forward run with no_grad?)")
        if bws.numel() < bwd_bytes:
            raise ValueError("the backward workspace is too small")
        p.q, p.k, p.v = _mat(q, batched), _mat(k, batched), _mat(v, batched)
        p.d_o, p.d_rem = _mat(do, batched), _vec(dr, batched)
        p.dq, p.dk, p.dv = _mat(dq, batched), _mat(dk, batched), _mat(dv, batched)
        p.fwd_workspace, p.fwd_workspace_bytes = ws.data_ptr(), ws.numel()
        p.bwd_workspace, p.bwd_workspace_bytes = bws.data_ptr(), bws.numel()
        _lib.check(_lib.lib().sbattn_bwd(ctypes.byref(p)), "sbattn_bwd")
        if os.environ.get("SBATTN_CHECK_STATUS") == "1":
            check_status(q.device)


# ---------------------------------------------------------------------------------------------- registered operators
# The reference wraps its launchers in torch.library.custom_op so that they survive torch.compile: operators
# "stickbreaking_attention::varlen_fwd" / "varlen_bwd" / "attn_fwd" / "attn_bwd" that write into buffers allocated by the
# caller and return None (utils.py:12-40, sb_varlen_fwd.py:453, sb_varlen_bwd.py:541, sb_fwd.py:175, sb_bwd.py:207).  The
# same operators exist here, with this library's argument lists.  They take the reference's namespace unless the
# reference itself has been imported into the process, in which case they go to "stickbreaking_attention_b200".
def _register_ops():
    ns = "stickbreaking_attention"
    try:
        getattr(torch.ops, ns).varlen_fwd
        ns = "stickbreaking_attention_b200"
    except (AttributeError, RuntimeError):
        pass
    T = torch.Tensor

    @torch.library.custom_op(f"{ns}::varlen_fwd", mutates_args={"o", "rem", "neg_log_acc", "workspace"}, device_types="cuda")
    def varlen_fwd_op(q: T, k: T, v: T, cu_seqlens: T, max_seqlens: int, logit_scale: float, attend_current: bool,
                      no_grad: bool, fused: bool, o: T, rem: T, neg_log_acc: T, workspace: T) -> None:
        _forward_into(q, k, v, False, cu_seqlens, max_seqlens, logit_scale, attend_current, no_grad, o, rem, neg_log_acc,
                      workspace, fused)

    @torch.library.custom_op(f"{ns}::varlen_bwd", mutates_args={"dq", "dk", "dv", "bwd_workspace"}, device_types="cuda")
    def varlen_bwd_op(do: T, dr: T, q: T, k: T, v: T, cu_seqlens: T, max_seqlens: int, workspace: T, logit_scale: float,
                      attend_current: bool, fused: bool, rem: T, dq: T, dk: T, dv: T, bwd_workspace: T) -> None:
        _backward_into(do, dr, q, k, v, False, cu_seqlens, max_seqlens, workspace, logit_scale, attend_current, 0, dq, dk,
                       dv, bwd_workspace, fused, rem)

    @torch.library.custom_op(f"{ns}::attn_fwd", mutates_args={"o", "rem", "neg_log_acc", "workspace"}, device_types="cuda")
    def attn_fwd_op(q: T, k: T, v: T, logit_scale: float, attend_current: bool, no_grad: bool, fused: bool, o: T, rem: T,
                    neg_log_acc: T, workspace: T) -> None:
        _forward_into(q, k, v, True, None, q.size(2), logit_scale, attend_current, no_grad, o, rem, neg_log_acc, workspace,
                      fused)

    @torch.library.custom_op(f"{ns}::attn_bwd", mutates_args={"dq", "dk", "dv", "bwd_workspace"}, device_types="cuda")
    def attn_bwd_op(do: T, dr: T, q: T, k: T, v: T, workspace: T, logit_scale: float, attend_current: bool, fused: bool,
                    rem: T, dq: T, dk: T, dv: T, bwd_workspace: T) -> None:
        _backward_into(do, dr, q, k, v, True, None, q.size(2), workspace, logit_scale, attend_current, 0, dq, dk, dv,
                       bwd_workspace, fused, rem)

    return ns, {"varlen_fwd": varlen_fwd_op, "varlen_bwd": varlen_bwd_op, "attn_fwd": attn_fwd_op, "attn_bwd": attn_bwd_op}


OP_NAMESPACE, _OPS = _register_ops()


def _forward(q, k, v, batched, cu_seqlens, max_seqlens, logit_scale, attend_current, no_grad, fused=False):
    compiling = torch.compiler.is_compiling()
    if not compiling:
        _require_cuda(q, k, v)
    q, k, v = _unit_inner(q), _unit_inner(k), _unit_inner(v)
    o = _empty_like_rows(q)
    # no zero-fill: the library writes every row of rem and neg_log_acc (zeros for tokens outside every sequence, which is
    # what the reference's zero-initialised outputs hold there, sb_varlen_fwd.py:418-419)
    rem = torch.empty(q.shape[:-1], dtype=q.dtype, device=q.device)
    neg_log_acc = torch.empty(q.shape[:-1], dtype=torch.float32, device=q.device)
    if batched:
        n_seqs, heads, tokens = q.size(0), q.size(1), q.size(2)
    else:
        n_seqs, heads, tokens = cu_seqlens.numel(), q.size(0), q.size(1)
    fwd_bytes, _ = workspace_bytes(batched, n_seqs, heads, tokens, max_seqlens, not no_grad)
    ws = torch.empty(fwd_bytes, dtype=torch.uint8, device=q.device)
    if compiling:  # the traced program sees one opaque operator
        if batched:
            _OPS["attn_fwd"](q, k, v, float(logit_scale), bool(attend_current), bool(no_grad), bool(fused), o, rem,
                             neg_log_acc, ws)
        else:
            _OPS["varlen_fwd"](q, k, v, cu_seqlens, int(max_seqlens), float(logit_scale), bool(attend_current),
                               bool(no_grad), bool(fused), o, rem, neg_log_acc, ws)
    else:
        _forward_into(q, k, v, batched, cu_seqlens, max_seqlens, logit_scale, attend_current, no_grad, o, rem, neg_log_acc,
                      ws, fused)
    return o, rem, neg_log_acc, ws


def _backward(do, dr, q, k, v, batched, cu_seqlens, max_seqlens, ws, logit_scale, attend_current, phases=0,
              out=None, bwd_ws=None, fused=False, rem=None):
    if rem is None:
        rem = dr  # placeholder of the right shape: only read when fused
    compiling = torch.compiler.is_compiling()
    if not compiling:
        _require_cuda(q, k, v, do, dr, ws)
    q, k, v, do = _unit_inner(q), _unit_inner(k), _unit_inner(v), _unit_inner(do)
    if do.dtype != q.dtype:
        do = do.to(q.dtype)
    if fused and not compiling and not _tma_ok(do):
        do = do.contiguous().clone()  # the fused backward exists in the tensor-core kernels only: give them an aligned copy
    if dr.dtype != q.dtype:
        dr = dr.to(q.dtype)
    if out is not None:
        dq, dk, dv = out
    else:
        # no zero-fill: the library writes every row (rows outside all sequences are cleared by a small kernel)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        if dq.stride(-1) != 1:
            dq, dk, dv = (torch.empty(q.shape, dtype=q.dtype, device=q.device) for _ in range(3))
    if batched:
        n_seqs, heads, tokens = q.size(0), q.size(1), q.size(2)
    else:
        n_seqs, heads, tokens = cu_seqlens.numel(), q.size(0), q.size(1)
    _, bwd_bytes = workspace_bytes(batched, n_seqs, heads, tokens, max_seqlens)
    bws = bwd_ws if bwd_ws is not None else torch.empty(bwd_bytes, dtype=torch.uint8, device=q.device)
    if compiling:
        if batched:
            _OPS["attn_bwd"](do, dr, q, k, v, ws, float(logit_scale), bool(attend_current), bool(fused), rem, dq, dk, dv,
                             bws)
        else:
            _OPS["varlen_bwd"](do, dr, q, k, v, cu_seqlens, int(max_seqlens), ws, float(logit_scale), bool(attend_current),
                               bool(fused), rem, dq, dk, dv, bws)
    else:
        _backward_into(do, dr, q, k, v, batched, cu_seqlens, max_seqlens, ws, logit_scale, attend_current, phases, dq, dk,
                       dv, bws, fused, rem)
    return dq, dk, dv


def _tma_ok(t):
    """Whether the tensor-core kernels can read or write t: 16-byte aligned base, outer strides that are multiples of
    8 elements and at least one row long (a broadcast head has stride 0).  Addresses are not visible while a program is
    being traced: a misaligned tensor then fails in the operator."""
    if t.stride(-1) != 1 or not all(st % 8 == 0 and (st >= t.size(-1) or n == 1) for st, n in zip(t.stride()[:-1], t.shape[:-1])):
        return False
    return torch.compiler.is_compiling() or t.data_ptr() % 16 == 0


def fusable(q, k=None, v=None):
    """Whether the fused remainder (out = o + rem * v inside the kernels) is available for these tensors: it exists in
    the tensor-core kernels only, which need 16-bit inputs, a head_dim they take and operands TMA can read."""
    if not (q.dtype in (torch.bfloat16, torch.float16) and q.size(-1) in (32, 64, 128) and _forced_path != "simt"):
        return False
    return all(_tma_ok(t) for t in (q, k, v) if t is not None)


def attention_weights(q, k, cu_seqlens=None, logit_scale=None, attend_current=False):
    """The attention matrix in float32, for debugging: [H, T, T] for the packed layout (cu_seqlens given; row and column
    are token indices of the pack, each sequence fills its diagonal block), [B, H, T, T] for the batched one.  Entries of
    pairs that are not attended are zero.  What the reference's launchers return as ``W`` with return_attention=True
    (sb_varlen_fwd.py:420-422,447-448; sb_fwd.py:145-147,169-170)."""
    batched = cu_seqlens is None
    _check_qkv(q, k, k, 4 if batched else 3)
    _require_cuda(q, k)
    q, k = _unit_inner(q), _unit_inner(k)
    if logit_scale is None:
        logit_scale = q.size(-1) ** -0.5
    if not batched:
        cu_seqlens, _ = _prep_cu(cu_seqlens, q, q.size(1))
    tokens = q.size(-2)
    w = torch.zeros(q.shape[:-1] + (tokens,), dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        p = _base_params(q, batched, cu_seqlens, tokens, logit_scale, attend_current, False)
        p.q, p.k = _mat(q, batched), _mat(k, batched)
        _lib.check(_lib.lib().sbattn_attention_weights(ctypes.byref(p), w.data_ptr(), w.stride(0) if batched else 0,
                                                       w.stride(-3), w.stride(-2)), "sbattn_attention_weights")
    return w


def varlen_fwd(q, k, v, cu_seqlens, max_seqlens, logit_scale, attend_current=False, no_grad=False, fuse_remainder=False,
               return_attention=False):
    """Packed layout: q, k, v [H, T, D]; cu_seqlens = cumulative sequence ends without a leading zero.

    Returns (o, rem, neg_log_acc, workspace) and, with ``return_attention``, the float32 attention matrix [H, T, T] after
    them.  Mirrors varlen_fwd of the reference (sb_varlen_fwd.py:411-452)."""
    _check_qkv(q, k, v, 3)
    cu_seqlens, max_seqlens = _prep_cu(cu_seqlens, q, max_seqlens)
    out = _forward(q, k, v, False, cu_seqlens, max_seqlens, logit_scale, attend_current, no_grad, fuse_remainder)
    if return_attention:
        return out + (attention_weights(q, k, cu_seqlens, logit_scale, attend_current),)
    return out


def varlen_bwd(do, dr, q, k, v, cu_seqlens, max_seqlens, workspace, logit_scale, attend_current=False, phases=0,
               out=None, bwd_workspace=None, fuse_remainder=False, rem=None):
    """Returns (dq, dk, dv).  Mirrors varlen_bwd of the reference (sb_varlen_bwd.py:483-539); ``workspace`` takes
    the place of its ``neg_log_acc`` argument.  ``phases`` (1: dq kernel only, 2: dk/dv kernel only), ``out`` and
    ``bwd_workspace`` exist for benchmarking the two backward kernels apart; leave them at their defaults."""
    _check_qkv(q, k, v, 3)
    cu_seqlens, max_seqlens = _prep_cu(cu_seqlens, q, max_seqlens)
    return _backward(do, dr, q, k, v, False, cu_seqlens, max_seqlens, workspace, logit_scale, attend_current, phases,
                     out, bwd_workspace, fuse_remainder, rem)


def attn_fwd(q, k, v, logit_scale, attend_current=False, no_grad=False, fuse_remainder=False, return_attention=False):
    """Batched layout: q, k, v [B, H, T, D].  Mirrors _fwd of the reference (sb_attn/sb_fwd.py:137-173); with
    ``return_attention`` the float32 attention matrix [B, H, T, T] follows the other results."""
    _check_qkv(q, k, v, 4)
    out = _forward(q, k, v, True, None, q.size(2), logit_scale, attend_current, no_grad, fuse_remainder)
    if return_attention:
        return out + (attention_weights(q, k, None, logit_scale, attend_current),)
    return out


def attn_bwd(do, dr, q, k, v, workspace, logit_scale, attend_current=False, fuse_remainder=False, rem=None):
    """Mirrors _bwd of the reference (sb_attn/sb_bwd.py:162-204)."""
    _check_qkv(q, k, v, 4)
    return _backward(do, dr, q, k, v, True, None, q.size(2), workspace, logit_scale, attend_current, 0, None, None,
                     fuse_remainder, rem)

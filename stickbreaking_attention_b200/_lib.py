"""ctypes binding of libsbattn.so (see include/sbattn.h).  There is no fallback: if the library cannot be loaded
every operator raises."""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libsbattn.so")

SBATTN_BF16, SBATTN_F32, SBATTN_F16 = 0, 1, 2
PATH_AUTO, PATH_SIMT, PATH_TENSOR = 0, 1, 2
ST_BAD_SEQLENS, ST_TIMEOUT = 1, 2


class SbMat(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("stride_b", ctypes.c_int64), ("stride_h", ctypes.c_int64),
                ("stride_t", ctypes.c_int64)]


class SbVec(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("stride_b", ctypes.c_int64), ("stride_h", ctypes.c_int64),
                ("stride_t", ctypes.c_int64)]


class SbParams(ctypes.Structure):
    _fields_ = [
        ("dtype", ctypes.c_int32), ("path", ctypes.c_int32), ("batch", ctypes.c_int32), ("heads", ctypes.c_int32),
        ("tokens", ctypes.c_int32), ("head_dim", ctypes.c_int32), ("num_seqs", ctypes.c_int32),
        ("cu_width", ctypes.c_int32), ("cu_seqlens", ctypes.c_void_p), ("max_seqlen", ctypes.c_int32),
        ("attend_current", ctypes.c_int32), ("inv_temp", ctypes.c_float), ("save_carries", ctypes.c_int32),
        ("bwd_phases", ctypes.c_int32), ("flags", ctypes.c_int32),
        ("q", SbMat), ("k", SbMat), ("v", SbMat), ("o", SbMat), ("rem", SbVec), ("neg_log_acc", SbVec),
        ("d_o", SbMat), ("d_rem", SbVec), ("dq", SbMat), ("dk", SbMat), ("dv", SbMat),
        ("fwd_workspace", ctypes.c_void_p), ("fwd_workspace_bytes", ctypes.c_size_t),
        ("bwd_workspace", ctypes.c_void_p), ("bwd_workspace_bytes", ctypes.c_size_t),
        ("status", ctypes.c_void_p), ("stream", ctypes.c_void_p),
    ]


FLAG_FUSED_REMAINDER = 1

EXPORTS = ("sbattn_workspace_bytes", "sbattn_fwd", "sbattn_bwd", "sbattn_strerror", "sbattn_version",
           "sbattn_params_size", "sbattn_fwd_static", "sbattn_static_scratch_bytes", "sbattn_attention_weights",
           "sbattn_launch_count")

_lib = None


class SbAttnError(RuntimeError):
    def __init__(self, code, where):
        self.code = code
        msg = lib().sbattn_strerror(code).decode() if _lib is not None else "?"
        super().__init__(f"{where}: {msg} (code {code})")


def lib():
    """The loaded library; raises if it is missing (build it with ``python -m stickbreaking_attention_b200.build``)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: the CUDA library has not been built "
                "(python -m stickbreaking_attention_b200.build). There is no fallback implementation.")
        L = ctypes.CDLL(LIB_PATH)
        L.sbattn_workspace_bytes.argtypes = [ctypes.POINTER(SbParams), ctypes.POINTER(ctypes.c_size_t),
                                             ctypes.POINTER(ctypes.c_size_t)]
        L.sbattn_workspace_bytes.restype = ctypes.c_int
        L.sbattn_fwd.argtypes = [ctypes.POINTER(SbParams)]
        L.sbattn_fwd.restype = ctypes.c_int
        L.sbattn_bwd.argtypes = [ctypes.POINTER(SbParams)]
        L.sbattn_bwd.restype = ctypes.c_int
        L.sbattn_strerror.argtypes = [ctypes.c_int]
        L.sbattn_strerror.restype = ctypes.c_char_p
        L.sbattn_version.restype = ctypes.c_int
        L.sbattn_params_size.restype = ctypes.c_size_t
        L.sbattn_launch_count.restype = ctypes.c_ulonglong
        L.sbattn_fwd_static.argtypes = [ctypes.POINTER(SbParams)]
        L.sbattn_fwd_static.restype = ctypes.c_int
        L.sbattn_static_scratch_bytes.restype = ctypes.c_size_t
        L.sbattn_attention_weights.argtypes = [ctypes.POINTER(SbParams), ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                               ctypes.c_int64]
        L.sbattn_attention_weights.restype = ctypes.c_int
        if L.sbattn_params_size() != ctypes.sizeof(SbParams):
            raise RuntimeError("libsbattn.so and its Python binding disagree about SbParams")
        _lib = L
    return _lib


def check(code, where):
    if code != 0:
        raise SbAttnError(code, where)

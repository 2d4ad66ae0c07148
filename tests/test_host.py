"""CPU-only checks: the C-ABI library loads, exports every declared symbol, rejects bad arguments without touching
a GPU, and the Python layer refuses CPU tensors (there is no fallback)."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from stickbreaking_attention_b200 import build, _lib
    build.build()
    return _lib.lib()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "sbattn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sbattn_[a-z_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    names = declared_symbols()
    assert {"sbattn_fwd", "sbattn_bwd", "sbattn_workspace_bytes", "sbattn_strerror", "sbattn_version"} <= set(names)
    for n in names:
        assert hasattr(lib, n), n
    from stickbreaking_attention_b200 import _lib
    assert set(_lib.EXPORTS) <= set(names)


def test_struct_mirror_matches(lib):
    from stickbreaking_attention_b200._lib import SbParams
    assert lib.sbattn_params_size() == ctypes.sizeof(SbParams)
    assert lib.sbattn_version() == 100


def params(**kw):
    from stickbreaking_attention_b200._lib import SbParams
    p = SbParams()
    p.dtype, p.path, p.batch, p.heads, p.tokens, p.head_dim = 0, 0, 0, 4, 1024, 128
    p.num_seqs, p.cu_width, p.max_seqlen, p.save_carries, p.inv_temp = 3, 8, 512, 1, 0.1
    for k, v in kw.items():
        setattr(p, k, v)
    return p


def test_argument_errors_without_gpu(lib):
    assert lib.sbattn_fwd(None) == -2
    assert lib.sbattn_fwd(ctypes.byref(params(dtype=7))) == -1
    assert lib.sbattn_fwd(ctypes.byref(params(head_dim=256))) == -3
    assert lib.sbattn_fwd(ctypes.byref(params(cu_width=2))) == -1
    assert lib.sbattn_fwd(ctypes.byref(params())) == -2          # null q
    assert lib.sbattn_bwd(ctypes.byref(params())) == -2
    assert lib.sbattn_fwd(ctypes.byref(params(heads=0))) == 0    # empty problem: nothing to do
    lib.sbattn_attention_weights.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64]
    assert lib.sbattn_attention_weights(None, None, 0, 0, 0) == -2
    assert lib.sbattn_attention_weights(ctypes.byref(params()), None, 0, 0, 1024) == -2   # null q
    assert lib.sbattn_attention_weights(ctypes.byref(params(heads=0)), None, 0, 0, 0) == 0
    for code in range(0, -7, -1):
        assert lib.sbattn_strerror(code)


def test_workspace_sizes(lib):
    fb, bb = ctypes.c_size_t(), ctypes.c_size_t()
    p = params()
    assert lib.sbattn_workspace_bytes(ctypes.byref(p), ctypes.byref(fb), ctypes.byref(bb)) == 0
    # items <= T/128 + S = 11, tiles per sequence <= 4: 64-key slots <= 11*5, two 32-key carries of 128 floats each, per head
    carry = 4 * 11 * 5 * 2 * 128 * 4
    rows = 4 * 1024 * 4  # one float per (head, token): drem + do . v of the fused-remainder backward
    assert bb.value == carry + rows and fb.value > carry
    p.save_carries = 0
    small = ctypes.c_size_t()
    lib.sbattn_workspace_bytes(ctypes.byref(p), ctypes.byref(small), None)
    assert small.value == fb.value - carry


def test_no_cpu_fallback():
    from stickbreaking_attention_b200 import sb_attn, sb_attn_varlen
    q = torch.randn(2, 16, 8)
    with pytest.raises(RuntimeError, match="CUDA"):
        sb_attn_varlen(q, q, q, torch.tensor([0, 16]), 16)
    with pytest.raises(RuntimeError, match="CUDA"):
        sb_attn(q[None], q[None], q[None])


def test_shape_and_dtype_validation():
    from stickbreaking_attention_b200 import sb_attn_varlen
    q = torch.randn(2, 16, 8)
    with pytest.raises(ValueError):
        sb_attn_varlen(q, q[:, :8], q, torch.tensor([16]), 16, zero_start=False)
    with pytest.raises(TypeError):
        sb_attn_varlen(q, q.double(), q, torch.tensor([16]), 16, zero_start=False)
    with pytest.raises(TypeError):
        sb_attn_varlen(q, q, q, torch.tensor([16.0]), 16, zero_start=False)
    with pytest.raises(AssertionError):
        sb_attn_varlen(q, q, q, torch.tensor([4, 16]), 16, zero_start=True)


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "stickbreaking_attention_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                assert "oracle" not in open(os.path.join(dirpath, f)).read(), f


def test_python_workspace_formula_matches_the_library(lib):
    """The traced (torch.compile) path sizes its buffers in Python; the formula must agree with the library."""
    from stickbreaking_attention_b200 import _lib, ops
    for batched, n_seqs, heads, tokens, max_len in [(False, 3, 4, 512, 192), (False, 7, 32, 16384, 3696), (False, 1, 8, 65536, 65536),
                                                     (False, 70, 64, 131072, 16384), (False, 5, 3, 1000, 0), (False, 2, 1, 77, 500),
                                                     (True, 2, 4, 500, 500), (True, 1, 2, 128, 128), (True, 8, 16, 4096, 4096)]:
        for save in (True, False):
            p = _lib.SbParams()
            p.dtype, p.heads, p.tokens, p.head_dim = _lib.SBATTN_BF16, heads, tokens, 64
            p.batch = n_seqs if batched else 0
            p.num_seqs = 0 if batched else n_seqs
            p.cu_width = 4
            p.max_seqlen = tokens if batched else max_len
            p.save_carries = int(save)
            fb, bb = ctypes.c_size_t(0), ctypes.c_size_t(0)
            assert lib.sbattn_workspace_bytes(ctypes.byref(p), ctypes.byref(fb), ctypes.byref(bb)) == 0
            assert ops.workspace_bytes(batched, n_seqs, heads, tokens, max_len, save) == (fb.value, bb.value)


def test_operators_are_registered_under_the_reference_names():
    """stickbreaking_attention::{varlen,attn}_{fwd,bwd}: out-parameters mutated, nothing returned
    (reference: utils.py:12-40, sb_varlen_fwd.py:453, sb_varlen_bwd.py:541, sb_fwd.py:175, sb_bwd.py:207)."""
    from stickbreaking_attention_b200 import ops
    ns = getattr(torch.ops, ops.OP_NAMESPACE)
    assert ops.OP_NAMESPACE == "stickbreaking_attention"
    for name, mutated in [("varlen_fwd", {"o", "rem", "neg_log_acc", "workspace"}), ("varlen_bwd", {"dq", "dk", "dv", "bwd_workspace"}),
                          ("attn_fwd", {"o", "rem", "neg_log_acc", "workspace"}), ("attn_bwd", {"dq", "dk", "dv", "bwd_workspace"})]:
        schema = getattr(ns, name).default._schema
        assert {a.name for a in schema.arguments if a.alias_info is not None and a.alias_info.is_write} == mutated
        assert len(schema.returns) == 0

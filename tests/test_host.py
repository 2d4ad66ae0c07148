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
    for code in range(0, -7, -1):
        assert lib.sbattn_strerror(code)


def test_workspace_sizes(lib):
    fb, bb = ctypes.c_size_t(), ctypes.c_size_t()
    p = params()
    assert lib.sbattn_workspace_bytes(ctypes.byref(p), ctypes.byref(fb), ctypes.byref(bb)) == 0
    # items <= T/128 + S = 11, tiles per sequence <= 4: slots <= 11*5, 128 floats each, per head
    carry = 4 * 11 * 5 * 128 * 4
    assert bb.value == carry and fb.value > carry
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

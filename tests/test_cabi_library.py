"""CPU-side checks of the C-ABI shared library: it loads, exports every symbol
that include/ua_b200.h declares, and validates arguments without a GPU."""
import ctypes
import os
import re

import pytest

from universal_attention_triton_b200 import _lib
from universal_attention_triton_b200._lib import UaDims
from universal_attention_triton_b200.build import build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build()
    return _lib.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ua_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ua_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(lib):
    names = declared_symbols()
    assert {"ua_fwd", "ua_bwd", "ua_relayout", "ua_merge_fwd", "ua_merge_bwd"} <= set(names)
    for n in names:
        assert hasattr(lib, n), n
    assert set(names) == set(_lib.SIGNATURES), "python binding table and header disagree"


def declared_parameter_counts():
    """name -> number of parameters of every function declaration in the header."""
    text = open(os.path.join(ROOT, "include", "ua_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    counts = {}
    for name, params in re.findall(r"\b(ua_[a-z0-9_]+)\s*\(([^()]*)\)\s*;", text):
        params = params.strip()
        counts[name] = 0 if params in ("", "void") else params.count(",") + 1
    return counts


def test_binding_table_has_the_headers_parameter_counts(lib):
    counts = declared_parameter_counts()
    assert set(counts) == set(_lib.SIGNATURES)
    for name, (_, argtypes) in _lib.SIGNATURES.items():
        assert len(argtypes) == counts[name], (name, len(argtypes), counts[name])


def test_version_and_error_strings(lib):
    assert lib.ua_version() >= 1
    assert lib.ua_error_string(0) == b"ok"
    assert b"unknown" in lib.ua_error_string(12345)


def test_argument_validation_without_gpu(lib):
    good = UaDims(1, 2, 2, 4, 64, 64)
    bad_chunk = UaDims(1, 2, 2, 4, 60, 64)
    null = ctypes.c_void_p(0)
    one = ctypes.c_void_p(16)
    # bad dims are rejected before anything touches the device
    rc = lib.ua_fwd(ctypes.byref(bad_chunk), 0, 0, one, one, one, one, one, one, one, null, null, 0, 0, null)
    assert rc == 1
    rc = lib.ua_fwd(ctypes.byref(good), 7, 0, one, one, one, one, one, one, one, null, null, 0, 0, null)
    assert rc == 2
    rc = lib.ua_fwd(ctypes.byref(good), 0, 0, null, one, one, one, one, one, one, null, null, 0, 0, null)
    assert rc == 3
    rc = lib.ua_fwd(ctypes.byref(good), 0, 0, ctypes.c_void_p(8), one, one, one, one, one, one, null, null, 0, 0, null)
    assert rc == 7
    # backward without workspace
    rc = lib.ua_bwd(ctypes.byref(good), 0, 0, one, one, one, one, one, one, one, 0, one, one, one, one, one, null, 0, 0, null)
    assert rc == 4
    assert lib.ua_bwd_workspace_bytes(ctypes.byref(good), 0, 0) > 0
    assert lib.ua_bwd_workspace_bytes(ctypes.byref(bad_chunk), 0, 0) == 0


def test_scratch_plan_routes_wide_chunks_to_the_tensor_core_kernels(lib):
    """bf16 chunks of 256 / 384 keys at head_dim 64 or 128 are swept as sub-chunks of 128 keys by the tensor-core kernels:
    the plan then holds a decay-prefix table per sub-chunk and room for the sub-chunk outputs (host-side arithmetic only)."""
    b, h, r, n, d = 1, 2, 2, 4, 128
    for c, m in ((256, 2), (384, 3)):
        dims = UaDims(b, h, r, n, c, d)
        L = n * c
        assert lib.ua_carry_bytes(ctypes.byref(dims), 1, 0) == b * h * (n * m) ** 2 * 256 * 4
        sub_out = b * h * n * m * r * L * d * 2
        assert lib.ua_fwd_workspace_bytes(ctypes.byref(dims), 1, 0) >= 256 + sub_out
        assert lib.ua_bwd_workspace_bytes(ctypes.byref(dims), 1, 0) >= 2 * sub_out
        # fp32, forced generic kernels, other head dims: no sub-chunk plan
        assert lib.ua_carry_bytes(ctypes.byref(dims), 0, 0) == 0
        assert lib.ua_carry_bytes(ctypes.byref(dims), 1, 4) == 0 and lib.ua_fwd_workspace_bytes(ctypes.byref(dims), 1, 4) == 256
    assert lib.ua_fwd_workspace_bytes(ctypes.byref(UaDims(b, h, r, n, 256, 32)), 1, 0) == 256


def test_cpu_tensors_are_rejected():
    import torch
    from universal_attention_triton_b200 import UniversalAttention
    from oracle.ua_oracle import make_inputs
    kc, vc, xq, ss, sd = make_inputs(1, 1, 1, 32, 16, 8)
    with pytest.raises(RuntimeError, match="no CPU path"):
        UniversalAttention.apply(kc, vc, xq, ss, sd)
    with pytest.raises(AssertionError):
        UniversalAttention.apply(kc, vc[:, :, :1], xq, ss, sd)
    assert not torch.cuda.is_available() or True

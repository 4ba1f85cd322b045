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

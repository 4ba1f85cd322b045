"""ctypes binding of libua_b200.so (the C ABI declared in include/ua_b200.h).

There is no fallback: if the library cannot be loaded every operator raises.
"""
from __future__ import annotations

import ctypes
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libua_b200.so")

UA_F32, UA_BF16 = 0, 1
FLAG_SKIP_MASKED_GRADS = 1
FLAG_SKIP_MASKED_FILL = 2
FLAG_FORCE_SIMT = 4


class UaDims(ctypes.Structure):
    _fields_ = [("batch", ctypes.c_int32), ("kv_heads", ctypes.c_int32), ("q_per_kv", ctypes.c_int32),
                ("n_chunks", ctypes.c_int32), ("chunk", ctypes.c_int32), ("head_dim", ctypes.c_int32)]


class UaRows(ctypes.Structure):
    _fields_ = [("tile_begin", ctypes.c_int32), ("tile_end", ctypes.c_int32), ("rows_total", ctypes.c_int32),
                ("row_offset", ctypes.c_int32)]


class UaLibraryError(RuntimeError):
    pass


_vp, _i, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
_dp = ctypes.POINTER(UaDims)
_rp = ctypes.POINTER(UaRows)

# name -> (restype, argtypes); every symbol include/ua_b200.h declares
SIGNATURES = {
    "ua_version": (_i, []),
    "ua_error_string": (ctypes.c_char_p, [_i]),
    "ua_fwd_workspace_bytes": (_sz, [_dp, _i, _i]),
    "ua_bwd_workspace_bytes": (_sz, [_dp, _i, _i]),
    "ua_fwd": (_i, [_dp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _vp]),
    "ua_bwd": (_i, [_dp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _vp]),
    "ua_carry_bytes": (_sz, [_dp, _i, _i]),
    "ua_fwd_keep": (_i, [_dp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _vp]),
    "ua_bwd_kept": (_i, [_dp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _vp]),
    "ua_bwd_saved": (_i, [_dp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _vp]),
    "ua_fwd_rows": (_i, [_dp, _i, _i, _rp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _vp]),
    "ua_decay_totals_rows": (_i, [_dp, _i, _i, _rp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "ua_fwd_rows_keep": (_i, [_dp, _i, _i, _rp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _vp]),
    "ua_bwd_rows_workspace_bytes": (_sz, [_dp, _i]),
    "ua_bwd_rows_suffix_workspace_bytes": (_sz, [_dp, _i]),
    "ua_bwd_rows_kept": (_i, [_dp, _i, _i, _rp] + [_vp] * 7 + [_i] + [_vp] * 11 + [_sz, _i, _vp]),
    "ua_bwd_rows": (_i, [_dp, _i, _i, _rp] + [_vp] * 7 + [_i] + [_vp] * 9 + [_sz, _i, _vp]),
    "ua_bwd_rows_suffix": (_i, [_dp, _i, _i, _rp] + [_vp] * 9 + [_sz, _vp]),
    "ua_static_scratch_bytes": (_sz, []),
    "ua_bwd_static": (_i, [_dp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "ua_static_status": (_i, [_vp]),
    "ua_workspace_status": (_i, [_vp, _vp]),
    "ua_selftest_wait_timeout": (_i, [_vp, ctypes.c_size_t, ctypes.c_uint, _vp]),
    "ua_relayout": (_i, [_dp, _i, _i, _i, _vp, _vp, _vp]),
    "ua_merge_fwd": (_i, [_dp, _i, _vp, _vp, _vp, _vp]),
    "ua_merge_bwd": (_i, [_dp, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "ua_merge_fwd_stats": (_i, [_dp, _i, _vp, _vp, _vp, _vp, _vp]),
    "ua_row_dot": (_i, [ctypes.c_longlong, _i, _i, _vp, _vp, _vp, _vp]),
    "ua_fwd_merged_workspace_bytes": (_sz, [_dp, _i]),
    "ua_fwd_merged": (_i, [_dp, _i, _i] + [_vp] * 9 + [_sz, _vp]),
    "ua_bwd_merged": (_i, [_dp, _i, _i] + [_vp] * 15 + [_sz, _vp]),
    "ua_decode_step": (_i, [_dp, _i, _i, _i] + [_vp] * 9),
    "ua_prepare_inputs": (_i, [_i] * 7 + [_vp] * 11),
    "ua_prepare_inputs_bwd": (_i, [_i] * 7 + [_vp] * 14),
}
PREP_NORMALIZE_KEYS, PREP_SIGMOID_GATES = 1, 2

_lib = None


def load():
    """Load the shared library once; raises UaLibraryError when it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise UaLibraryError(
            f"{LIB_PATH} is missing: build it with `python -m universal_attention_triton_b200.build` "
            "(there is no CPU or PyTorch fallback for the Universal Attention kernels)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(code: int, what: str):
    if code != 0:
        msg = load().ua_error_string(code).decode()
        raise UaLibraryError(f"{what} failed: {msg} (code {code})")

"""ua_bwd_static: the backward entry point that allocates nothing.

It exists for hosts that cannot give the library a workspace (a runtime with a
frozen memory plan, a plugin interface that passes only inputs and outputs):
the scratch is a fixed 16 MiB buffer inside the library's device image.  The
test drives it through the C ABI with caller-owned inputs and outputs and
compares every gradient with the regular ua_bwd entry point, twice in a row:
the second call finds the buffer as the first one left it, so it also checks
that the call clears what has to start at zero.  The file name sorts last so
that a run that stops at the first failure has already run every other test.
"""
import ctypes

import pytest
import torch

from oracle import ua_oracle as O
from tests._util import rel_fro

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("shape,dtype", [((1, 2, 2, 512, 128, 64), torch.bfloat16),    # tensor-core kernels
                                         ((1, 2, 2, 256, 64, 64), torch.float32)])      # generic fp32 kernels
def test_static_backward_matches_regular_backward(shape, dtype):
    from universal_attention_triton_b200 import _lib, ops
    from universal_attention_triton_b200._lib import UaDims
    lib = _lib.load()
    B, H, R, L, c, D = shape
    n = L // c
    code = _lib.UA_BF16 if dtype == torch.bfloat16 else _lib.UA_F32
    dims = UaDims(B, H, R, n, c, D)
    assert lib.ua_bwd_workspace_bytes(ctypes.byref(dims), code, 0) <= lib.ua_static_scratch_bytes()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):
        ins = O.make_inputs(B, H, R, L, c, D, dtype=dtype, seed=40 + call)
        kc, vc, xq, ss, sd = [t.cuda().contiguous() for t in ins]
        gen = torch.Generator(device="cuda").manual_seed(50 + call)
        g_out = torch.randn(B, H, n, R, L, D, generator=gen, device="cuda", dtype=dtype)
        g_lse = torch.randn(B, H, n, R, L, generator=gen, device="cuda")
        want = ops.backward_cm(kc, vc, xq, ss, sd, g_out, g_lse)
        got = [torch.full_like(t, float("nan")) for t in (kc, vc, xq, ss, sd)]
        rc = lib.ua_bwd_static(ctypes.byref(dims), code, code, _ptr(kc), _ptr(vc), _ptr(xq), _ptr(ss), _ptr(sd),
                               _ptr(g_out), _ptr(g_lse), _lib.UA_F32, *[_ptr(t) for t in got], 0, stream)
        assert rc == 0, lib.ua_error_string(rc)
        assert lib.ua_static_status(stream) == 0
        for a, b, name in zip(got, want, ["dkc", "dvc", "dxq", "dsrc", "ddest"]):
            assert torch.isfinite(a.float()).all(), (call, name)
            # same kernels on both sides; only the order of the fp32 atomic additions differs
            assert rel_fro(a.float().cpu(), b.float().cpu()) <= 2e-2, (call, name)


def test_static_backward_refuses_oversized_problems():
    from universal_attention_triton_b200 import _lib
    from universal_attention_triton_b200._lib import UaDims
    lib = _lib.load()
    dims = UaDims(4, 8, 4, 32, 128, 64)                     # needs far more than 16 MiB of scratch
    assert lib.ua_bwd_workspace_bytes(ctypes.byref(dims), _lib.UA_BF16, 0) > lib.ua_static_scratch_bytes()
    one = ctypes.c_void_p(256)
    rc = lib.ua_bwd_static(ctypes.byref(dims), _lib.UA_BF16, _lib.UA_BF16, one, one, one, one, one, one, one, _lib.UA_F32,
                           one, one, one, one, one, 0, ctypes.c_void_p(0))
    assert rc == 10 and b"static" in lib.ua_error_string(rc)

"""Drop-in for the reference's kernel-backed Function
(Universal_Attention/universal_attention.py:5-46): 2-D signature, shape asserts,
last-dimension contiguity fix-ups, then the CUDA library instead of the Triton
launchers (_universal_attention_fwd / _universal_attention_bwd)."""
from __future__ import annotations

from torch.autograd import Function

from .. import universal_attention_autograd as _ua


class UniversalAttention(Function):
    @staticmethod
    def forward(ctx, kc, vc, xq, static_src, static_dest):
        b, h, r, _n, _c, d = xq.shape
        _, _, n_, c_, _ = kc.shape
        assert kc.shape == (b, h, n_, c_, d)
        assert vc.shape == (b, h, n_, c_, d)
        assert static_src.shape == (b, h, n_, c_)
        assert static_dest.shape == (b, h, _n, _c)
        return _ua._forward(ctx, kc, vc, xq, static_src, static_dest)

    @staticmethod
    def backward(ctx, dout, ddenom):
        kc, vc, xq, static_src, static_dest = ctx.saved_tensors
        b, h, r, _n, _c, d = xq.shape
        _, _, n_, c_, _ = kc.shape
        assert dout.shape == (b, h, r, n_ * c_, d, n_)
        assert ddenom.shape == (b, h, r, n_ * c_, n_)
        return _ua._backward(ctx, dout, ddenom)

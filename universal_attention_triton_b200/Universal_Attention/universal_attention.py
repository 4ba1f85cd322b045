"""Drop-in for the reference's kernel-backed Function
(Universal_Attention/universal_attention.py:5-46): 2-D signature, the same
new-style ``forward`` / ``setup_context`` / ``backward`` protocol and shape
asserts, then the CUDA library instead of the Triton launchers
(_universal_attention_fwd / _universal_attention_bwd).  Tensors of any strides
are accepted (the reference makes them last-dim contiguous, :14-23, :41-44;
here the tensor plumbing does what the kernels need)."""
from __future__ import annotations

from torch.autograd import Function

from .. import universal_attention_autograd as _ua


class UniversalAttention(Function):
    @staticmethod
    def forward(kc, vc, xq, static_src, static_dest):
        b, h, r, _n, _c, d = xq.shape
        _, _, n_, c_, _ = kc.shape
        assert kc.shape == (b, h, n_, c_, d)
        assert vc.shape == (b, h, n_, c_, d)
        assert static_src.shape == (b, h, n_, c_)
        assert static_dest.shape == (b, h, _n, _c)
        return _ua._forward(kc, vc, xq, static_src, static_dest)

    @staticmethod
    def setup_context(ctx, inputs, outputs):
        _ua._setup_context(ctx, inputs, outputs)

    @staticmethod
    def backward(ctx, dout, ddenom):
        kc, vc, xq = ctx.saved_tensors[:3]
        b, h, r, _n, _c, d = xq.shape
        _, _, n_, c_, _ = kc.shape
        assert dout.shape == (b, h, r, n_ * c_, d, n_)
        assert ddenom.shape == (b, h, r, n_ * c_, n_)
        return _ua._backward(ctx, dout, ddenom)

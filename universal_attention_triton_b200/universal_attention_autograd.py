"""Drop-in autograd entry points of the Universal Attention operator, backed by
the sm_100a CUDA library.  Same names, argument layout, output shapes/dtypes
and gradients as the reference module of the same name:

* ``UniversalAttention``   1-D signature   (universal_attention_autograd.py:7-99)
* ``UniversalAttention2``  2-D signature   (universal_attention_autograd.py:102-276)
* ``SMVecMatMul``          merge over key chunks (universal_attention_autograd.py:278-297)

    out, denom = UniversalAttention.apply(kc, vc, xq, static_src, static_dest)

``out (b,h,r,L,d,n_)`` and ``denom (b,h,r,L,n_)`` have the reference's shapes and
dtypes.  By default they are permuted views of chunk-major storage (see
``ops.py``); ``set_output_layout("reference")`` makes them contiguous in the
reference's order at the cost of one extra pass over ``out``.

The five inputs are saved for backward and everything is recomputed from them
(universal_attention_autograd.py:41-44, :166-169); the only extra is the small
fp32 decay-prefix table the forward kernel has in registers anyway (16.8 MB at
B4 H8 L4096), which spares the backward its pre-pass.  Tensors must be CUDA
tensors: there is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import torch
from torch.autograd import Function

from . import _lib, ops

_OUTPUT_LAYOUT = "chunk_major"
_STRICT_MASKED_GRADS = True


def set_output_layout(layout: str) -> None:
    """"chunk_major" (default; permuted views) or "reference" (contiguous (b,h,r,L,d,n_))."""
    global _OUTPUT_LAYOUT
    if layout not in ("chunk_major", "reference"):
        raise ValueError(layout)
    _OUTPUT_LAYOUT = layout


_MERGED_BACKWARD = "composed"


def set_merged_backward(mode: str) -> None:
    """Backward of ``UniversalAttentionMerged``.  ``"composed"`` (default): the merge backward followed by the
    operator's backward, as accurate as the drop-in pair (gradients within ~5e-3 relative-Frobenius of the fp32
    reference in bf16).  ``"fused"``: one kernel (``ua_bwd_merged``) that forms ``dS = P (dP - g.merged)`` with the
    bf16 merged output, as flash-attention backwards do with their output; about 15 % faster end to end, but the
    rounding of ``merged`` enters the decay gradient through a cumulative sum: gradients within 1-4e-2 of the
    reference at L = 1024..4096 (inside the 5e-2 bar, ten times the composed path's error)."""
    global _MERGED_BACKWARD
    assert mode in ("composed", "fused")
    _MERGED_BACKWARD = mode


def set_strict_masked_grads(on: bool) -> None:
    """When off, backward skips the gradient through fully masked blocks (rows
    before a key chunk).  That gradient is exactly zero when ``SMVecMatMul``
    consumes ``(out, denom)``; it is not for arbitrary upstream gradients."""
    global _STRICT_MASKED_GRADS
    _STRICT_MASKED_GRADS = bool(on)


def _forward(ctx, kc, vc, xq, static_src, static_dest):
    out_cm, lse_cm, denom_cm, carry = ops.forward_cm(kc, vc, xq, static_src, static_dest, keep_carry=True)
    ctx.save_for_backward(kc, vc, xq, static_src, static_dest)
    ctx.ua_carry = carry
    ctx.ua_lse = lse_cm            # fp32 log-sum-exp (33 MB at B4 H8 R4 L4096): spares the backward its row max / sum
    if _OUTPUT_LAYOUT == "reference":
        return ops.to_reference_layout(out_cm, denom_cm)
    return ops.as_reference_out(out_cm), ops.as_reference_denom(denom_cm)


def _backward(ctx, g_out, g_denom):
    kc, vc, xq, static_src, static_dest = ctx.saved_tensors
    flags = 0 if _STRICT_MASKED_GRADS else _lib.FLAG_SKIP_MASKED_GRADS
    g_out_cm = ops.out_to_chunk_major(g_out)
    g_denom_cm = ops.denom_to_chunk_major(g_denom)
    return ops.backward_cm(kc, vc, xq, static_src, static_dest, g_out_cm, g_denom_cm, flags,
                           carry=getattr(ctx, "ua_carry", None), lse=getattr(ctx, "ua_lse", None))


class UniversalAttention(Function):
    """kc, vc (b,h,n,c,d); xq (b,h,r,l,d); static_src (b,h,n,c); static_dest (b,h,l)."""

    @staticmethod
    def forward(ctx, kc, vc, xq, static_src, static_dest):
        b, h, r, l, d = xq.shape
        _, _, n, c, _ = kc.shape
        assert kc.shape == (b, h, n, c, d) and n * c == l
        assert vc.shape == (b, h, n, c, d)
        assert static_src.shape == (b, h, n, c)
        assert static_dest.shape == (b, h, l)
        return _forward(ctx, kc, vc, xq, static_src, static_dest)

    @staticmethod
    def backward(ctx, g_out, g_denom):
        return _backward(ctx, g_out, g_denom)


class UniversalAttention2(Function):
    """kc, vc (b,h,n_,c_,d); xq (b,h,r,_n,_c,d); static_src (b,h,n_,c_); static_dest (b,h,_n,_c).
    The row chunking (_n,_c) is only a view of the rows; the result does not depend on it."""

    @staticmethod
    def forward(ctx, kc, vc, xq, static_src, static_dest):
        b, h, r, _n, _c, d = xq.shape
        _, _, n_, c_, _ = kc.shape
        assert kc.shape == (b, h, n_, c_, d) and n_ * c_ == _n * _c
        assert vc.shape == (b, h, n_, c_, d)
        assert static_src.shape == (b, h, n_, c_)
        assert static_dest.shape == (b, h, _n, _c)
        return _forward(ctx, kc, vc, xq, static_src, static_dest)

    @staticmethod
    def backward(ctx, g_out, g_denom):
        return _backward(ctx, g_out, g_denom)


class SMVecMatMul(Function):
    """``mat (..., d, n)``, ``vec (..., n)`` -> ``sum_n softmax(vec)[n] * mat[..., n]``.
    Takes the 6-D ``out`` and 5-D ``denom`` of the operator (any strides)."""

    @staticmethod
    def forward(mat, vec):
        assert mat.dim() == 6 and vec.dim() == 5 and mat.shape[:4] == vec.shape[:4] and mat.shape[-1] == vec.shape[-1]
        return ops.merge_fwd_cm(ops.out_to_chunk_major(mat), ops.denom_to_chunk_major(vec))

    @staticmethod
    def setup_context(ctx, inputs, outputs):
        ctx.save_for_backward(*inputs)

    @staticmethod
    def backward(ctx, g):
        mat, vec = ctx.saved_tensors
        g_out_cm, g_lse_cm = ops.merge_bwd_cm(ops.out_to_chunk_major(mat), ops.denom_to_chunk_major(vec), g,
                                              skip_zero_weight_blocks=not _STRICT_MASKED_GRADS)
        return ops.as_reference_out(g_out_cm), ops.as_reference_denom(g_lse_cm).to(vec.dtype)


class UniversalAttentionMerged(Function):
    """``merged = SMVecMatMul.apply(*UniversalAttention.apply(kc, vc, xq, static_src, static_dest))`` as one Function:
    the flow of the reference's driver (``main.py:55-62``) for callers that only consume the merged output
    ``(b,h,r,l,d)``.  No counterpart in the reference.  The merge weights come from the fp32 log-sum-exp (the
    drop-in ``denom`` is rounded to the input dtype as in the reference, which moves bf16 weights).  Backward: see
    ``set_merged_backward``; with ``"fused"`` the (b,h,r,l,d,n) ``out`` tensor lives only inside the forward and
    nothing of its size is kept for or produced by the backward.  ``xq`` and ``static_dest`` in either the 1-D or
    the 2-D form."""

    @staticmethod
    def forward(ctx, kc, vc, xq, static_src, static_dest):
        b, h, n, c, d = kc.shape
        assert vc.shape == kc.shape and static_src.shape == (b, h, n, c)
        assert xq.shape[:2] == (b, h) and xq.shape[-1] == d and xq[0, 0, 0].numel() == n * c * d
        assert static_dest.numel() == b * h * n * c
        out_cm, lse_cm, _, carry = ops.forward_cm(kc, vc, xq, static_src, static_dest, keep_carry=True)
        merged, row_lse = ops.merge_fwd_stats_cm(out_cm, lse_cm)
        ctx.fused = _MERGED_BACKWARD == "fused" and ops.merged_backward_supported(kc, xq)
        ctx.ua_carry = carry
        if ctx.fused:
            ctx.save_for_backward(kc, vc, xq, static_src, static_dest, merged, row_lse)
        else:
            ctx.save_for_backward(kc, vc, xq, static_src, static_dest, out_cm, lse_cm)
        return merged.view(*xq.shape)

    @staticmethod
    def backward(ctx, g):
        kc, vc, xq, static_src, static_dest, x, y = ctx.saved_tensors
        if ctx.fused:
            return ops.backward_merged(kc, vc, xq, static_src, static_dest, g, x, y, carry=ctx.ua_carry)
        g_out_cm, g_lse_cm = ops.merge_bwd_cm(x, y, g.reshape(x.shape[0], x.shape[1], x.shape[3], x.shape[4], x.shape[5]),
                                              skip_zero_weight_blocks=True)
        return ops.backward_cm(kc, vc, xq, static_src, static_dest, g_out_cm, g_lse_cm, _lib.FLAG_SKIP_MASKED_GRADS,
                               carry=ctx.ua_carry, lse=y)


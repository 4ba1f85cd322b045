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

The Functions follow the reference's protocol: a ``forward`` without ``ctx``, ``setup_context``
and ``backward`` (universal_attention_autograd.py:9, :41-44, :47).  The five inputs are saved
for backward as in the reference (:41-44, :166-169); two by-products of the forward kernel are
saved with them through ``save_for_backward`` -- the fp32 log-sum-exp and the small decay-prefix
table (16.8 MB at B4 H8 L4096) -- which spare the backward a second forward pass; a backward
that finds only the inputs recomputes both.  Tensors must be CUDA
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
    bf16 merged output, as flash-attention backwards do with their output; about 18 % faster end to end, but the
    rounding of ``merged`` enters the decay gradient through a cumulative sum: gradients within 1-4e-2 of the
    reference at L = 1024..4096 (inside the 5e-2 bar, ten times the composed path's error)."""
    global _MERGED_BACKWARD
    assert mode in ("composed", "fused")
    _MERGED_BACKWARD = mode


_MERGED_FORWARD = "materialise"


def set_merged_forward(mode: str) -> None:
    """Forward of ``UniversalAttentionMerged``.  ``"materialise"`` (default): the operator's forward, then the merge over
    key chunks (the (b,h,n,r,L,d) tensor ``out`` lives inside the forward).  ``"low_memory"``: two passes of the forward
    kernel that never write ``out`` (``ua_fwd_merged``): (b,h,n,r,L) + (b,h,r,L,d) floats of scratch instead of two n-fold
    tensors, about 0.7 ms more per step at B4 H8 R4 L4096 D64; implies the fused backward (there is no ``out`` to merge
    backwards through); shapes the tensor-core kernels do not take fall back to ``"materialise"``."""
    global _MERGED_FORWARD
    assert mode in ("materialise", "low_memory")
    _MERGED_FORWARD = mode


_SAVE_OUTPUT = True


def set_save_output(on: bool) -> None:
    """When on (default), the Functions also save their own output ``out`` for backward (chunk-major layout only).  The
    tensor-core backward then takes the softmax gradient's row term ``sum_k P dP`` as ``out . g_out`` per row instead of
    summing over the keys (the backward kernel then takes 2.15 ms instead of 2.55 at B4 H8 R4 L4096 D64).  ``out`` stays alive until backward has run -- which
    it does anyway whenever ``SMVecMatMul`` (or any node that saves its input) consumes it -- and, like every saved
    tensor, must not be modified in place before backward.  Off: exactly the reference's set of saved inputs plus the two
    small by-products."""
    global _SAVE_OUTPUT
    _SAVE_OUTPUT = bool(on)


def set_strict_masked_grads(on: bool) -> None:
    """When off, backward skips the gradient through fully masked blocks (rows
    before a key chunk).  That gradient is exactly zero when ``SMVecMatMul``
    consumes ``(out, denom)``; it is not for arbitrary upstream gradients."""
    global _STRICT_MASKED_GRADS
    _STRICT_MASKED_GRADS = bool(on)


def _forward(kc, vc, xq, static_src, static_dest):
    """Shared new-style forward (no ctx): returns ``(out, denom)``.  The fp32 log-sum-exp and the decay-prefix table that
    the forward kernel produces anyway ride on the returned ``denom`` as ``_ua_extras`` so that ``_setup_context`` can
    hand them to ``ctx.save_for_backward``; a backward that does not find them recomputes them."""
    out_cm, lse_cm, denom_cm, carry = ops.forward_cm(kc, vc, xq, static_src, static_dest, keep_carry=True)
    if _OUTPUT_LAYOUT == "reference":
        out, denom = ops.to_reference_layout(out_cm, denom_cm)
    else:
        out, denom = ops.as_reference_out(out_cm), ops.as_reference_denom(denom_cm)
    denom._ua_extras = (lse_cm, carry)
    return out, denom


def _setup_context(ctx, inputs, outputs):
    """Saves the five inputs, as the reference does (universal_attention_autograd.py:41-44, :166-169), plus -- when the
    forward left them on ``denom`` -- the fp32 log-sum-exp (33 MB at B4 H8 R4 L4096) and the decay-prefix table, all
    through ``save_for_backward`` so that saved-tensor hooks and version checks apply to them too."""
    kc, vc, xq, static_src, static_dest = inputs
    extras = getattr(outputs[1], "_ua_extras", None) if isinstance(outputs, tuple) else None
    if extras is not None and isinstance(extras[0], torch.Tensor):
        lse_cm, carry = extras
        del outputs[1]._ua_extras                   # denom must not keep the two tensors alive on its own
        ctx.ua_has_carry = carry is not None
        saved = (kc, vc, xq, static_src, static_dest, lse_cm) + ((carry,) if carry is not None else ())
        ctx.ua_has_out = _SAVE_OUTPUT and _OUTPUT_LAYOUT == "chunk_major"
        if ctx.ua_has_out:
            saved = saved + (outputs[0],)
        ctx.save_for_backward(*saved)
        ctx.ua_has_extras = True
    else:
        ctx.save_for_backward(kc, vc, xq, static_src, static_dest)
        ctx.ua_has_extras = False


def _mark_masked_zero(*tensors):
    """Notes on gradient tensors that their part for the rows before each chunk is exactly zero (``SMVecMatMul.backward``
    produces such tensors: the merge weight of a fully masked block is exp(-1e12 - lse) = 0).  The note holds the tensor's
    version counter, so that an in-place change of the tensor voids it; a tensor that autograd builds from it (a sum with
    another gradient, a hook's replacement) does not carry it."""
    for t in tensors:
        t._ua_masked_zero = t._version


def _masked_zero(t) -> bool:
    v = getattr(t, "_ua_masked_zero", None)
    return v is not None and v == t._version


def _backward(ctx, g_out, g_denom):
    # Upstream gradients that are known to vanish on the rows before each chunk contribute nothing there: the kernels of
    # those rows are skipped, with the same result.  Anything else takes the full path (unless strict mode is off).
    upstream_zero = _masked_zero(g_out) and _masked_zero(g_denom)
    saved = ops.plain(*ctx.saved_tensors)
    g_out, g_denom = ops.plain(g_out, g_denom)
    kc, vc, xq, static_src, static_dest = saved[:5]
    out_cm = None
    if getattr(ctx, "ua_has_extras", False):
        lse = saved[5]
        carry = saved[6] if ctx.ua_has_carry else None
        if getattr(ctx, "ua_has_out", False):
            v = saved[-1].permute(0, 1, 5, 2, 3, 4)            # the chunk-major storage behind the reference-shaped view
            out_cm = v if v.is_contiguous() else None
    else:                      # only the inputs were saved: recompute what the forward would have handed over
        _, lse, _, carry = ops.forward_cm(kc, vc, xq, static_src, static_dest, flags=_lib.FLAG_SKIP_MASKED_FILL, keep_carry=True)
    flags = 0 if (_STRICT_MASKED_GRADS and not upstream_zero) else _lib.FLAG_SKIP_MASKED_GRADS
    g_out_cm = ops.out_to_chunk_major(g_out)
    g_denom_cm = ops.denom_to_chunk_major(g_denom)
    return ops.backward_cm(kc, vc, xq, static_src, static_dest, g_out_cm, g_denom_cm, flags, carry=carry, lse=lse, out_cm=out_cm)


class UniversalAttention(Function):
    """kc, vc (b,h,n,c,d); xq (b,h,r,l,d); static_src (b,h,n,c); static_dest (b,h,l).
    Same protocol as the reference class: new-style ``forward`` without ctx, ``setup_context``, ``backward``
    (universal_attention_autograd.py:9, :41-44, :47)."""

    @staticmethod
    def forward(kc, vc, xq, static_src, static_dest):
        b, h, r, l, d = xq.shape
        _, _, n, c, _ = kc.shape
        assert kc.shape == (b, h, n, c, d) and n * c == l
        assert vc.shape == (b, h, n, c, d)
        assert static_src.shape == (b, h, n, c)
        assert static_dest.shape == (b, h, l)
        return _forward(kc, vc, xq, static_src, static_dest)

    @staticmethod
    def setup_context(ctx, inputs, outputs):
        _setup_context(ctx, inputs, outputs)

    @staticmethod
    def backward(ctx, g_out, g_denom):
        return _backward(ctx, g_out, g_denom)


class UniversalAttention2(Function):
    """kc, vc (b,h,n_,c_,d); xq (b,h,r,_n,_c,d); static_src (b,h,n_,c_); static_dest (b,h,_n,_c).
    The row chunking (_n,_c) is only a view of the rows; the result does not depend on it
    (universal_attention_autograd.py:104, :166-169, :172)."""

    @staticmethod
    def forward(kc, vc, xq, static_src, static_dest):
        b, h, r, _n, _c, d = xq.shape
        _, _, n_, c_, _ = kc.shape
        assert kc.shape == (b, h, n_, c_, d) and n_ * c_ == _n * _c
        assert vc.shape == (b, h, n_, c_, d)
        assert static_src.shape == (b, h, n_, c_)
        assert static_dest.shape == (b, h, _n, _c)
        return _forward(kc, vc, xq, static_src, static_dest)

    @staticmethod
    def setup_context(ctx, inputs, outputs):
        _setup_context(ctx, inputs, outputs)

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
        mat, vec, g = ops.plain(*ctx.saved_tensors, g)
        g_out_cm, g_lse_cm = ops.merge_bwd_cm(ops.out_to_chunk_major(mat), ops.denom_to_chunk_major(vec), g,
                                              skip_zero_weight_blocks=not _STRICT_MASKED_GRADS)
        g_mat, g_vec = ops.as_reference_out(g_out_cm), ops.as_reference_denom(g_lse_cm).to(vec.dtype)
        _mark_masked_zero(g_mat, g_vec)
        return g_mat, g_vec


class UniversalAttentionMerged(Function):
    """``merged = SMVecMatMul.apply(*UniversalAttention.apply(kc, vc, xq, static_src, static_dest))`` as one Function:
    the flow of the reference's driver (``main.py:55-62``) for callers that only consume the merged output
    ``(b,h,r,l,d)``.  No counterpart in the reference.  The merge weights come from the fp32 log-sum-exp (the
    drop-in ``denom`` is rounded to the input dtype as in the reference, which moves bf16 weights).  Backward: see
    ``set_merged_backward``; with ``"fused"`` the (b,h,r,l,d,n) ``out`` tensor lives only inside the forward and
    nothing of its size is kept for or produced by the backward.  ``xq`` and ``static_dest`` in either the 1-D or
    the 2-D form."""

    @staticmethod
    def forward(kc, vc, xq, static_src, static_dest):
        b, h, n, c, d = kc.shape
        assert vc.shape == kc.shape and static_src.shape == (b, h, n, c)
        assert xq.shape[:2] == (b, h) and xq.shape[-1] == d and xq[0, 0, 0].numel() == n * c * d
        assert static_dest.numel() == b * h * n * c
        if _MERGED_FORWARD == "low_memory" and ops.merged_backward_supported(kc, xq):
            res = ops.forward_merged_lowmem(kc, vc, xq, static_src, static_dest)
            if res is not None:
                merged, row_lse, carry = res
                merged = merged.view(*xq.shape)
                merged._ua_extras = (True, (merged, row_lse), carry)
                return merged
        out_cm, lse_cm, _, carry = ops.forward_cm(kc, vc, xq, static_src, static_dest, keep_carry=True)
        merged, row_lse = ops.merge_fwd_stats_cm(out_cm, lse_cm)
        fused = _MERGED_BACKWARD == "fused" and ops.merged_backward_supported(kc, xq)
        merged = merged.view(*xq.shape)
        merged._ua_extras = (fused, (merged, row_lse) if fused else (out_cm, lse_cm), carry)
        return merged

    @staticmethod
    def setup_context(ctx, inputs, output):
        ctx.fused, (x, y), carry = output._ua_extras
        del output._ua_extras                       # (it holds a reference to the output itself in fused mode)
        ctx.ua_has_carry = carry is not None
        ctx.save_for_backward(*inputs, x, y, *((carry,) if carry is not None else ()))

    @staticmethod
    def backward(ctx, g):
        saved = ops.plain(*ctx.saved_tensors)
        g = ops.plain(g)
        kc, vc, xq, static_src, static_dest, x, y = saved[:7]
        carry = saved[7] if ctx.ua_has_carry else None
        if ctx.fused:
            return ops.backward_merged(kc, vc, xq, static_src, static_dest, g, x, y, carry=carry)
        g_out_cm, g_lse_cm = ops.merge_bwd_cm(x, y, g.reshape(x.shape[0], x.shape[1], x.shape[3], x.shape[4], x.shape[5]),
                                              skip_zero_weight_blocks=True)
        return ops.backward_cm(kc, vc, xq, static_src, static_dest, g_out_cm, g_lse_cm, _lib.FLAG_SKIP_MASKED_GRADS,
                               carry=carry, lse=y)


"""Tensor-level calls into the CUDA library on chunk-major storage.

Chunk-major storage keeps the key-chunk axis outside the row axis:
``out_cm (b,h,n,r,L,d)`` and ``lse_cm (b,h,n,r,L)``.  The reference's
``out (b,h,r,L,d,n)`` / ``denom (b,h,r,L,n)`` are permuted views of them
(``as_reference_out`` / ``as_reference_denom``): same shape, dtype and values,
different strides, so that every kernel reads and writes whole contiguous
``(rows, d)`` tiles.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib
from ._lib import UaDims


def _dtype_code(t: torch.dtype) -> int:
    if t == torch.float32:
        return _lib.UA_F32
    if t == torch.bfloat16:
        return _lib.UA_BF16
    raise TypeError(f"Universal Attention kernels support float32 and bfloat16, got {t}")


def plain(*tensors):
    """Strips functorch wrappers (``torch.func.grad`` hands the backward its gradients and saved tensors wrapped, alive
    or already dead) so that the kernels get tensors with storage; first-order transforms only."""
    try:
        from torch._C._functorch import get_unwrapped, maybe_get_level, unwrap_if_dead
    except ImportError:      # pragma: no cover
        return tensors if len(tensors) != 1 else tensors[0]
    out = []
    for t in tensors:
        if isinstance(t, torch.Tensor):
            for _ in range(16):
                if maybe_get_level(t) == -1:
                    break
                u = unwrap_if_dead(t)
                t = u if u is not t else get_unwrapped(t)
        out.append(t)
    return tuple(out) if len(out) != 1 else out[0]


def _ptr(t):
    return ctypes.c_void_p(plain(t).data_ptr()) if t is not None else ctypes.c_void_p(0)


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _require_cuda(*tensors):
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("Universal Attention has no CPU path: tensors must live on a CUDA device")


def _check_status(lib, ws, what):
    """With UA_CHECK_STATUS=1 every call synchronises and reads the kernels' status word
    (a bounded device-side wait that ran out) -- for tests and debugging."""
    if os.environ.get("UA_CHECK_STATUS") == "1":
        _lib.check(lib.ua_workspace_status(_ptr(ws), _stream()), what + " (device status)")


def make_dims(kc, xq):
    b, h, n, c, d = kc.shape
    r = xq.shape[2]
    return UaDims(b, h, r, n, c, d)


def _gate_cast(g, dtype):
    # kernels take gates either in the q/k/v dtype or in fp32
    if g.dtype == dtype or g.dtype == torch.float32:
        return g.contiguous()
    return g.float().contiguous()


def forward_cm(kc, vc, xq, static_src, static_dest, flags: int = 0, keep_carry: bool = False):
    """Returns (out_cm, lse_cm fp32, denom_cm).  ``denom_cm`` is ``lse_cm`` itself in fp32 mode.
    With ``keep_carry`` a fourth value is returned: the decay-prefix table for ``backward_cm(carry=...)``
    (``None`` for shapes whose backward does not use one)."""
    _require_cuda(kc, vc, xq, static_src, static_dest)
    lib = _lib.load()
    b, h, n, c, d = kc.shape
    r = xq.shape[2]
    L = n * c
    dt = xq.dtype
    code = _dtype_code(dt)
    kc, vc = kc.contiguous(), vc.contiguous()
    q = xq.reshape(b, h, r, L, d).contiguous()
    ss = _gate_cast(static_src.reshape(b, h, L), dt)
    sd = _gate_cast(static_dest.reshape(b, h, L), dt)
    if ss.dtype != sd.dtype:
        ss, sd = ss.float(), sd.float()
    dims = UaDims(b, h, r, n, c, d)
    with torch.cuda.device(kc.device):
        out_cm = torch.empty(b, h, n, r, L, d, dtype=dt, device=kc.device)
        lse_cm = torch.empty(b, h, n, r, L, dtype=torch.float32, device=kc.device)
        denom_cm = lse_cm if dt == torch.float32 else torch.empty(b, h, n, r, L, dtype=dt, device=kc.device)
        ws_bytes = lib.ua_fwd_workspace_bytes(ctypes.byref(dims), code, flags)
        ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=kc.device)
        carry = None
        if keep_carry:
            cbytes = lib.ua_carry_bytes(ctypes.byref(dims), code, flags)
            if cbytes:
                carry = torch.empty(cbytes // 4, dtype=torch.float32, device=kc.device)
        rc = lib.ua_fwd_keep(ctypes.byref(dims), code, _dtype_code(ss.dtype), _ptr(kc), _ptr(vc), _ptr(q), _ptr(ss), _ptr(sd),
                             _ptr(out_cm), _ptr(lse_cm), _ptr(None if denom_cm is lse_cm else denom_cm), _ptr(carry),
                             _ptr(ws), ws_bytes, flags, _stream())
        _lib.check(rc, "ua_fwd")
        _check_status(lib, ws, "ua_fwd")
    if keep_carry:
        return out_cm, lse_cm, denom_cm, carry
    return out_cm, lse_cm, denom_cm


def backward_cm(kc, vc, xq, static_src, static_dest, g_out_cm, g_denom_cm, flags: int = 0, carry=None, lse=None, out_cm=None):
    """Gradients (dkc, dvc, dxq, dstatic_src, dstatic_dest) shaped and typed like the inputs.
    ``carry``: the table ``forward_cm(keep_carry=True)`` returned for the same inputs (skips the pre-pass).
    ``lse``: the fp32 ``lse_cm (b,h,n,r,L)`` of the same forward (lets the tensor-core backward skip its row max / sum).
    ``out_cm``: the output tiles ``(b,h,n,r,L,d)`` of the same forward, when the caller still holds them (``ua_bwd_saved``:
    the softmax gradient's row term comes from them instead of a sum over the keys)."""
    _require_cuda(kc, vc, xq, static_src, static_dest, g_out_cm, g_denom_cm)
    lib = _lib.load()
    b, h, n, c, d = kc.shape
    r = xq.shape[2]
    L = n * c
    dt = xq.dtype
    code = _dtype_code(dt)
    kcc, vcc = kc.contiguous(), vc.contiguous()
    q = xq.reshape(b, h, r, L, d).contiguous()
    ss = _gate_cast(static_src.reshape(b, h, L), dt)
    sd = _gate_cast(static_dest.reshape(b, h, L), dt)
    if ss.dtype != sd.dtype:
        ss, sd = ss.float(), sd.float()
    g_out_cm = g_out_cm.to(dt).contiguous()
    if g_denom_cm.dtype not in (torch.float32, dt):
        g_denom_cm = g_denom_cm.float()
    g_denom_cm = g_denom_cm.contiguous()
    dims = UaDims(b, h, r, n, c, d)
    with torch.cuda.device(kc.device):
        dkc = torch.empty_like(kcc)
        dvc = torch.empty_like(vcc)
        dxq = torch.empty_like(q)
        dss = torch.empty_like(ss)
        dsd = torch.empty_like(sd)
        ws_bytes = lib.ua_bwd_workspace_bytes(ctypes.byref(dims), code, flags)
        ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=kc.device)
        if carry is not None and carry.numel() * 4 != lib.ua_carry_bytes(ctypes.byref(dims), code, flags):
            carry = None
        if lse is not None:
            if lse.dtype != torch.float32 or tuple(lse.shape) != (b, h, n, r, L) or not lse.is_cuda:
                raise ValueError("lse must be the fp32 chunk-major (b,h,n,r,L) log-sum-exp of the forward")
            lse = lse.contiguous()
        if out_cm is not None and not (out_cm.is_cuda and out_cm.dtype == dt and out_cm.is_contiguous()
                                       and tuple(out_cm.shape) == (b, h, n, r, L, d)):
            out_cm = None
        rc = lib.ua_bwd_saved(ctypes.byref(dims), code, _dtype_code(ss.dtype), _ptr(kcc), _ptr(vcc), _ptr(q), _ptr(ss), _ptr(sd),
                        _ptr(g_out_cm), _ptr(g_denom_cm), _dtype_code(g_denom_cm.dtype), _ptr(carry), _ptr(lse), _ptr(out_cm),
                        _ptr(dkc), _ptr(dvc), _ptr(dxq), _ptr(dss), _ptr(dsd), _ptr(ws), ws_bytes, flags, _stream())
        _lib.check(rc, "ua_bwd")
        _check_status(lib, ws, "ua_bwd")
    return (dkc.view(kc.shape), dvc.view(vc.shape), dxq.view(xq.shape),
            dss.to(static_src.dtype).view(static_src.shape), dsd.to(static_dest.dtype).view(static_dest.shape))


def as_reference_out(out_cm):
    """(b,h,n,r,L,d) storage viewed as the reference's out (b,h,r,L,d,n)."""
    return out_cm.permute(0, 1, 3, 4, 5, 2)


def as_reference_denom(denom_cm):
    """(b,h,n,r,L) storage viewed as the reference's denom (b,h,r,L,n)."""
    return denom_cm.permute(0, 1, 3, 4, 2)


def out_to_chunk_major(t):
    """Reference-shaped out / g_out (b,h,r,L,d,n), any strides -> contiguous (b,h,n,r,L,d)."""
    v = t.permute(0, 1, 5, 2, 3, 4)
    return v if v.is_contiguous() else _relayout(t, inner=t.shape[4], to_reference=False)


def denom_to_chunk_major(t):
    """Reference-shaped denom / g_denom (b,h,r,L,n), any strides -> contiguous (b,h,n,r,L)."""
    v = t.permute(0, 1, 4, 2, 3)
    return v if v.is_contiguous() else _relayout(t, inner=1, to_reference=False)


def _relayout(t, inner: int, to_reference: bool):
    _require_cuda(t)
    lib = _lib.load()
    if t.element_size() not in (2, 4):
        raise TypeError("relayout handles 2- and 4-byte elements")
    if to_reference:      # t is chunk-major (b,h,n,r,L[,d])
        b, h, n, r, L = t.shape[:5]
        src = t.contiguous()
        dst = torch.empty((b, h, r, L) + ((inner,) if t.dim() == 6 else ()) + (n,), dtype=t.dtype, device=t.device)
    else:                 # t is reference-shaped (b,h,r,L[,d],n)
        b, h, r, L = t.shape[:4]
        n = t.shape[-1]
        src = t.contiguous()
        dst = torch.empty((b, h, n, r, L) + ((inner,) if t.dim() == 6 else ()), dtype=t.dtype, device=t.device)
    dims = UaDims(b, h, r, n, 16, 4)      # chunk/head_dim are not used by the converter; only L = n*chunk matters
    # the converter takes L through dims: encode L as n_chunks*chunk
    if L % n:
        raise ValueError("rows must be a multiple of the number of key chunks")
    dims.chunk = L // n
    if dims.chunk % 16:
        raise ValueError("chunk must be a multiple of 16")
    with torch.cuda.device(t.device):
        rc = lib.ua_relayout(ctypes.byref(dims), inner, t.element_size(), 1 if to_reference else 0,
                             _ptr(src), _ptr(dst), _stream())
    _lib.check(rc, "ua_relayout")
    return dst


def to_reference_layout(out_cm, denom_cm):
    """Materialise the reference's contiguous (b,h,r,L,d,n) / (b,h,r,L,n) tensors."""
    return (_relayout(out_cm, inner=out_cm.shape[-1], to_reference=True),
            _relayout(denom_cm, inner=1, to_reference=True))


def merge_fwd_cm(out_cm, lse_cm):
    """SMVecMatMul forward on chunk-major storage -> merged (b,h,r,L,d)."""
    _require_cuda(out_cm, lse_cm)
    lib = _lib.load()
    b, h, n, r, L, d = out_cm.shape
    dims = UaDims(b, h, r, n, L // n, d)
    out_cm = out_cm.contiguous()
    lse_cm = lse_cm.float().contiguous()
    merged = torch.empty(b, h, r, L, d, dtype=out_cm.dtype, device=out_cm.device)
    with torch.cuda.device(out_cm.device):
        rc = lib.ua_merge_fwd(ctypes.byref(dims), _dtype_code(out_cm.dtype), _ptr(out_cm), _ptr(lse_cm), _ptr(merged), _stream())
    _lib.check(rc, "ua_merge_fwd")
    return merged


def merge_fwd_stats_cm(out_cm, lse_cm):
    """``merge_fwd_cm`` that also returns the fp32 log-sum-exp of every row over ALL key chunks, (b,h,r,L)."""
    _require_cuda(out_cm, lse_cm)
    lib = _lib.load()
    b, h, n, r, L, d = out_cm.shape
    dims = UaDims(b, h, r, n, L // n, d)
    out_cm = out_cm.contiguous()
    lse_cm = lse_cm.float().contiguous()
    merged = torch.empty(b, h, r, L, d, dtype=out_cm.dtype, device=out_cm.device)
    row_lse = torch.empty(b, h, r, L, dtype=torch.float32, device=out_cm.device)
    with torch.cuda.device(out_cm.device):
        rc = lib.ua_merge_fwd_stats(ctypes.byref(dims), _dtype_code(out_cm.dtype), _ptr(out_cm), _ptr(lse_cm), _ptr(merged),
                                    _ptr(row_lse), _stream())
    _lib.check(rc, "ua_merge_fwd_stats")
    return merged, row_lse


def forward_merged_lowmem(kc, vc, xq, static_src, static_dest):
    """``merged (b,h,r,L,d)`` and ``row_lse (b,h,r,L)`` fp32 of ``SMVecMatMul(UniversalAttention(...))`` without the
    (b,h,n,r,L,d) tensor ``out`` (``ua_fwd_merged``: two passes of the forward kernel), plus the decay-prefix table for
    ``backward_merged`` (or ``None``).  Returns ``None`` for shapes the tensor-core forward does not take."""
    _require_cuda(kc, vc, xq, static_src, static_dest)
    lib = _lib.load()
    b, h, n, c, d = kc.shape
    r = xq.shape[2]
    L = n * c
    dt = xq.dtype
    code = _dtype_code(dt)
    dims = UaDims(b, h, r, n, c, d)
    ws_bytes = lib.ua_fwd_merged_workspace_bytes(ctypes.byref(dims), code)
    if not ws_bytes:
        return None
    kcc, vcc = kc.contiguous(), vc.contiguous()
    q = xq.reshape(b, h, r, L, d).contiguous()
    ss = _gate_cast(static_src.reshape(b, h, L), dt)
    sd = _gate_cast(static_dest.reshape(b, h, L), dt)
    if ss.dtype != sd.dtype:
        ss, sd = ss.float(), sd.float()
    with torch.cuda.device(kc.device):
        merged = torch.empty(b, h, r, L, d, dtype=dt, device=kc.device)
        row_lse = torch.empty(b, h, r, L, dtype=torch.float32, device=kc.device)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=kc.device)
        cbytes = lib.ua_carry_bytes(ctypes.byref(dims), code, 0)
        carry = torch.empty(cbytes // 4, dtype=torch.float32, device=kc.device) if cbytes else None
        rc = lib.ua_fwd_merged(ctypes.byref(dims), code, _dtype_code(ss.dtype), _ptr(kcc), _ptr(vcc), _ptr(q), _ptr(ss), _ptr(sd),
                               _ptr(merged), _ptr(row_lse), _ptr(carry), _ptr(ws), ws_bytes, _stream())
        _lib.check(rc, "ua_fwd_merged")
        _check_status(lib, ws, "ua_fwd_merged")
    return merged, row_lse, carry


def row_dot(a, b):
    """fp32 ``(a * b).sum(-1)`` of two equally shaped contiguous tensors (rows of head_dim elements)."""
    _require_cuda(a, b)
    lib = _lib.load()
    a, b = a.contiguous(), b.to(a.dtype).contiguous()
    out = torch.empty(a.shape[:-1], dtype=torch.float32, device=a.device)
    with torch.cuda.device(a.device):
        rc = lib.ua_row_dot(a.numel() // a.shape[-1], a.shape[-1], _dtype_code(a.dtype), _ptr(a), _ptr(b), _ptr(out), _stream())
    _lib.check(rc, "ua_row_dot")
    return out


def merged_backward_supported(kc, xq) -> bool:
    """Shapes the one-kernel backward of the merged output takes (bf16, chunk 128, head_dim 64 or 128)."""
    return xq.dtype == torch.bfloat16 and kc.shape[3] == 128 and kc.shape[4] in (64, 128)


def backward_merged(kc, vc, xq, static_src, static_dest, g_merged, merged, row_lse, carry=None):
    """Gradients of ``merged = SMVecMatMul(UniversalAttention(...))`` with respect to the five inputs, from the gradient
    of the merged output alone (``ua_bwd_merged``): no (b,h,n,r,L,d) tensor is read or written."""
    _require_cuda(kc, vc, xq, static_src, static_dest, g_merged, merged, row_lse)
    lib = _lib.load()
    b, h, n, c, d = kc.shape
    r = xq.shape[2]
    L = n * c
    dt = xq.dtype
    code = _dtype_code(dt)
    kcc, vcc = kc.contiguous(), vc.contiguous()
    q = xq.reshape(b, h, r, L, d).contiguous()
    ss = _gate_cast(static_src.reshape(b, h, L), dt)
    sd = _gate_cast(static_dest.reshape(b, h, L), dt)
    if ss.dtype != sd.dtype:
        ss, sd = ss.float(), sd.float()
    g = g_merged.to(dt).reshape(b, h, r, L, d).contiguous()
    delta = row_dot(g, merged.reshape(b, h, r, L, d))
    row_lse = row_lse.float().contiguous()
    dims = UaDims(b, h, r, n, c, d)
    with torch.cuda.device(kc.device):
        dkc, dvc, dxq = torch.empty_like(kcc), torch.empty_like(vcc), torch.empty_like(q)
        dss, dsd = torch.empty_like(ss), torch.empty_like(sd)
        ws_bytes = lib.ua_bwd_workspace_bytes(ctypes.byref(dims), code, 0)
        ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=kc.device)
        if carry is not None and carry.numel() * 4 != lib.ua_carry_bytes(ctypes.byref(dims), code, 0):
            carry = None
        rc = lib.ua_bwd_merged(ctypes.byref(dims), code, _dtype_code(ss.dtype), _ptr(kcc), _ptr(vcc), _ptr(q), _ptr(ss), _ptr(sd),
                               _ptr(g), _ptr(row_lse), _ptr(delta), _ptr(carry), _ptr(dkc), _ptr(dvc), _ptr(dxq), _ptr(dss),
                               _ptr(dsd), _ptr(ws), ws_bytes, _stream())
        _lib.check(rc, "ua_bwd_merged")
        _check_status(lib, ws, "ua_bwd_merged")
    return (dkc.view(kc.shape), dvc.view(vc.shape), dxq.view(xq.shape),
            dss.to(static_src.dtype).view(static_src.shape), dsd.to(static_dest.dtype).view(static_dest.shape))


def merge_bwd_cm(out_cm, lse_cm, g_merged, skip_zero_weight_blocks: bool = False):
    """SMVecMatMul backward on chunk-major storage -> (g_out_cm, g_lse_cm fp32).
    ``skip_zero_weight_blocks``: leave the blocks whose merge weight is exactly zero unwritten
    (only valid when the consumer never reads them: backward with masked-block gradients skipped)."""
    _require_cuda(out_cm, lse_cm, g_merged)
    lib = _lib.load()
    b, h, n, r, L, d = out_cm.shape
    dims = UaDims(b, h, r, n, L // n, d)
    out_cm = out_cm.contiguous()
    lse_cm = lse_cm.float().contiguous()
    g_merged = g_merged.to(out_cm.dtype).contiguous()
    g_out_cm = torch.empty_like(out_cm)
    g_lse_cm = torch.empty_like(lse_cm)
    with torch.cuda.device(out_cm.device):
        rc = lib.ua_merge_bwd(ctypes.byref(dims), _dtype_code(out_cm.dtype), _ptr(out_cm), _ptr(lse_cm), _ptr(g_merged),
                              _ptr(g_out_cm), _ptr(g_lse_cm),
                              _lib.FLAG_SKIP_MASKED_FILL if skip_zero_weight_blocks else 0, _stream())
    _lib.check(rc, "ua_merge_bwd")
    return g_out_cm, g_lse_cm


# ---- sequence-chunk sharding: forward / backward over a range of row tiles ---------------------------
# Row-indexed tensors are "slabs" of Ls rows (Ls = xq_rows.shape[3]); the range [tile_begin, tile_end) sits at
# row `row_offset` of the slabs, so that several ranges (zig-zag halves) can share them.

def _rows(tile_begin, tile_end, rows_total, row_offset):
    return _lib.UaRows(tile_begin, tile_end, rows_total, row_offset)


def _gates_rows(static_src, static_dest_rows, b, h, L, dt):
    ss = _gate_cast(static_src.reshape(b, h, L), dt)
    sd = _gate_cast(static_dest_rows.reshape(b, h, -1), dt)
    if ss.dtype != sd.dtype:
        ss, sd = ss.float(), sd.float()
    return ss, sd


def decay_totals_rows(kc, static_src, static_dest_rows, tile_begin: int, tile_end: int, carry_in=None, row_offset: int = 0):
    """(b,h,n,128) fp32: for every key, ``carry_in`` (or 0) plus the sum of its log-retention over the rows of
    the row tiles [tile_begin, tile_end).  ``static_dest_rows`` (b,h,Ls) is a slab holding the range at ``row_offset``."""
    _require_cuda(kc, static_src, static_dest_rows)
    lib = _lib.load()
    b, h, n, c, d = kc.shape
    dt = kc.dtype
    code = _dtype_code(dt)
    kc = kc.contiguous()
    ss, sd = _gates_rows(static_src, static_dest_rows, b, h, n * c, dt)
    dims = UaDims(b, h, 1, n, c, d)
    rows = _rows(tile_begin, tile_end, sd.shape[-1], row_offset)
    with torch.cuda.device(kc.device):
        total = torch.empty(b, h, n, 128, dtype=torch.float32, device=kc.device)
        ws = torch.empty(256, dtype=torch.uint8, device=kc.device)
        ci = carry_in.float().contiguous() if carry_in is not None else None
        rc = lib.ua_decay_totals_rows(ctypes.byref(dims), code, _dtype_code(ss.dtype), ctypes.byref(rows), _ptr(kc), _ptr(ss),
                                      _ptr(sd), _ptr(ci), _ptr(total), _ptr(ws), 256, _stream())
        _lib.check(rc, "ua_decay_totals_rows")
        _check_status(lib, ws, "ua_decay_totals_rows")
    return total


def alloc_forward_rows(kc, xq_rows):
    """Output slabs for ``forward_rows_cm``: (out_cm (b,h,n,r,Ls,d), lse_cm fp32 (b,h,n,r,Ls), denom_cm)."""
    b, h, n, c, d = kc.shape
    r, Ls = xq_rows.shape[2], xq_rows.shape[3]
    dev, dt = kc.device, xq_rows.dtype
    return (torch.empty(b, h, n, r, Ls, d, dtype=dt, device=dev), torch.empty(b, h, n, r, Ls, dtype=torch.float32, device=dev),
            torch.empty(b, h, n, r, Ls, dtype=dt, device=dev))


def alloc_carry_table(kc):
    """The decay-prefix table that ``forward_rows_cm(carry_table=...)`` fills and ``backward_rows(carry_table=...)`` reads
    (one table serves all the row ranges of a rank), or ``None`` for shapes whose backward does not use one."""
    lib = _lib.load()
    b, h, n, c, d = kc.shape
    dims = UaDims(b, h, 1, n, c, d)
    nbytes = lib.ua_carry_bytes(ctypes.byref(dims), _dtype_code(kc.dtype), 0)
    return torch.empty(nbytes // 4, dtype=torch.float32, device=kc.device) if nbytes else None


def forward_rows_cm(kc, vc, xq_rows, static_src, static_dest_rows, tile_begin: int, tile_end: int, carry_in=None,
                    flags: int = 0, row_offset: int = 0, out=None, carry_table=None):
    """Forward for the row tiles [tile_begin, tile_end), written into the rows [row_offset, ...) of the output slabs
    ``out`` (from ``alloc_forward_rows``; allocated here when None).  ``kc``, ``vc``, ``static_src`` cover the whole
    sequence; ``xq_rows`` (b,h,r,Ls,d) / ``static_dest_rows`` (b,h,Ls) are slabs; ``carry_in`` (b,h,n,128): sum of the
    ``decay_totals_rows`` of all rows before the range."""
    _require_cuda(kc, vc, xq_rows, static_src, static_dest_rows)
    lib = _lib.load()
    b, h, n, c, d = kc.shape
    r, Ls = xq_rows.shape[2], xq_rows.shape[3]
    dt = xq_rows.dtype
    code = _dtype_code(dt)
    kc, vc = kc.contiguous(), vc.contiguous()
    q = xq_rows.contiguous()
    ss, sd = _gates_rows(static_src, static_dest_rows, b, h, n * c, dt)
    dims = UaDims(b, h, r, n, c, d)
    rows = _rows(tile_begin, tile_end, Ls, row_offset)
    with torch.cuda.device(kc.device):
        out_cm, lse_cm, denom_cm = out if out is not None else alloc_forward_rows(kc, q)
        ws = torch.empty(256, dtype=torch.uint8, device=kc.device)
        ci = carry_in.float().contiguous() if carry_in is not None else None
        rc = lib.ua_fwd_rows_keep(ctypes.byref(dims), code, _dtype_code(ss.dtype), ctypes.byref(rows), _ptr(kc), _ptr(vc), _ptr(q),
                                  _ptr(ss), _ptr(sd), _ptr(ci), _ptr(out_cm), _ptr(lse_cm), _ptr(denom_cm), _ptr(carry_table),
                                  _ptr(ws), 256, flags, _stream())
        _lib.check(rc, "ua_fwd_rows")
        _check_status(lib, ws, "ua_fwd_rows")
    return out_cm, lse_cm, denom_cm


def alloc_backward_rows(kc, xq_rows):
    """Zeroed fp32 accumulators for ``backward_rows``: (dk (b,h,L,d), dv (b,h,L,d), dxq (b,h,r,Ls,d), dsrc (b,h,L),
    ddest (b,h,Ls))."""
    b, h, n, c, d = kc.shape
    r, Ls = xq_rows.shape[2], xq_rows.shape[3]
    z = lambda *shape: torch.zeros(*shape, dtype=torch.float32, device=kc.device)
    return z(b, h, n * c, d), z(b, h, n * c, d), z(b, h, r, Ls, d), z(b, h, n * c), z(b, h, Ls)


def backward_rows(kc, vc, xq_rows, static_src, static_dest_rows, g_out_cm_rows, g_denom_cm_rows, tile_begin: int,
                  tile_end: int, carry_in=None, suffix_in=None, flags: int = 0, row_offset: int = 0, acc=None,
                  carry_table=None, lse_cm_rows=None):
    """Backward for the row tiles [tile_begin, tile_end) (sequence sharding), ADDED into the fp32 accumulators ``acc``
    (from ``alloc_backward_rows``; allocated here when None).  Returns ``(dk, dv, dxq, dsrc, ddest, dctot)``: dk, dv,
    dsrc are partial sums over ALL keys; dctot (b,h,n,128) is the per-key sum of the decay-prefix gradient over the rows.
    ``carry_table`` / ``lse_cm_rows``: what ``forward_rows_cm`` produced for the same range (table from
    ``alloc_carry_table``, the fp32 log-sum-exp slab); with both, no part of the forward is run again."""
    _require_cuda(kc, vc, xq_rows, static_src, static_dest_rows, g_out_cm_rows, g_denom_cm_rows)
    lib = _lib.load()
    b, h, n, c, d = kc.shape
    r, Ls = xq_rows.shape[2], xq_rows.shape[3]
    dt = xq_rows.dtype
    code = _dtype_code(dt)
    kc, vc = kc.contiguous(), vc.contiguous()
    q = xq_rows.contiguous()
    ss, sd = _gates_rows(static_src, static_dest_rows, b, h, n * c, dt)
    g_out_cm_rows = g_out_cm_rows.to(dt).contiguous()
    if g_denom_cm_rows.dtype not in (torch.float32, dt):
        g_denom_cm_rows = g_denom_cm_rows.float()
    g_denom_cm_rows = g_denom_cm_rows.contiguous()
    dims = UaDims(b, h, r, n, c, d)
    rows = _rows(tile_begin, tile_end, Ls, row_offset)
    dev = kc.device
    with torch.cuda.device(dev):
        dk, dv, dxq, dsrc, ddest = acc if acc is not None else alloc_backward_rows(kc, q)
        dctot = torch.empty(b, h, n, 128, dtype=torch.float32, device=dev)
        ws_bytes = lib.ua_bwd_rows_workspace_bytes(ctypes.byref(dims), code)
        ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
        ci = carry_in.float().contiguous() if carry_in is not None else None
        si = suffix_in.float().contiguous() if suffix_in is not None else None
        if lse_cm_rows is not None:
            assert lse_cm_rows.dtype == torch.float32 and lse_cm_rows.is_contiguous()
        rc = lib.ua_bwd_rows_kept(ctypes.byref(dims), code, _dtype_code(ss.dtype), ctypes.byref(rows), _ptr(kc), _ptr(vc), _ptr(q),
                                  _ptr(ss), _ptr(sd), _ptr(g_out_cm_rows), _ptr(g_denom_cm_rows),
                                  _dtype_code(g_denom_cm_rows.dtype), _ptr(ci), _ptr(si), _ptr(carry_table), _ptr(lse_cm_rows),
                                  _ptr(dk), _ptr(dv), _ptr(dxq), _ptr(dsrc), _ptr(ddest), _ptr(dctot),
                                  _ptr(ws), ws_bytes, flags, _stream())
        _lib.check(rc, "ua_bwd_rows")
        _check_status(lib, ws, "ua_bwd_rows")
    return dk, dv, dxq, dsrc, ddest, dctot


def backward_rows_suffix(kc, vc, static_src, static_dest_rows, tile_begin: int, tile_end: int, suffix, dk, dsrc, ddest,
                         row_offset: int = 0):
    """Adds to ``dk``, ``dsrc``, ``ddest`` (the fp32 accumulators of ``backward_rows``) the gradient induced by the
    reverse decay carry ``suffix`` (b,h,n,128) that enters the range from the rows after it."""
    _require_cuda(kc, vc, static_src, static_dest_rows, suffix, dk, dsrc, ddest)
    lib = _lib.load()
    b, h, n, c, d = kc.shape
    dt = kc.dtype
    code = _dtype_code(dt)
    kc, vc = kc.contiguous(), vc.contiguous()
    ss, sd = _gates_rows(static_src, static_dest_rows, b, h, n * c, dt)
    assert dk.is_contiguous() and dsrc.is_contiguous() and ddest.is_contiguous()
    dims = UaDims(b, h, 1, n, c, d)
    rows = _rows(tile_begin, tile_end, sd.shape[-1], row_offset)
    with torch.cuda.device(kc.device):
        ws_bytes = max(lib.ua_bwd_rows_suffix_workspace_bytes(ctypes.byref(dims), code), 256)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=kc.device)
        sf = suffix.float().contiguous()
        rc = lib.ua_bwd_rows_suffix(ctypes.byref(dims), code, _dtype_code(ss.dtype), ctypes.byref(rows), _ptr(kc), _ptr(vc),
                                    _ptr(ss), _ptr(sd), _ptr(sf), _ptr(dk), _ptr(dsrc), _ptr(ddest), _ptr(ws), ws_bytes, _stream())
        _lib.check(rc, "ua_bwd_rows_suffix")
        _check_status(lib, ws, "ua_bwd_rows_suffix")


def decode_step(t, k_cache, v_cache, src_cache, q_t, dest_t, decay_state, chunk):
    """One incremental step (``ua_decode_step``): row ``t`` of the forward against the caches.

    ``k_cache, v_cache (b,h,L_cap,d)``, ``src_cache (b,h,L_cap)`` hold rows ``0..t``; ``q_t (b,h,r,d)``, ``dest_t (b,h)``
    are the new row; ``decay_state (b,h,L_cap)`` fp32 is updated in place (zeros before ``t = 0``).  Returns
    ``(out_t (b,h,r,d,n_t), lse_t (b,h,r,n_t) fp32)`` as views with the key-chunk index last, i.e. row ``t`` of the
    operator's ``out`` / ``denom`` restricted to the ``n_t = t // chunk + 1`` chunks that hold keys ``<= t``."""
    _require_cuda(k_cache, v_cache, src_cache, q_t, dest_t, decay_state)
    lib = _lib.load()
    b, h, Lcap, d = k_cache.shape
    r = q_t.shape[2]
    dt = q_t.dtype
    assert decay_state.dtype == torch.float32 and decay_state.is_contiguous() and decay_state.shape == (b, h, Lcap)
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and Lcap % chunk == 0
    src = _gate_cast(src_cache, dt).contiguous()
    dst = _gate_cast(dest_t, dt).contiguous()
    if src.dtype != dst.dtype:
        src, dst = src.float(), dst.float()
    nt = t // chunk + 1
    dims = UaDims(b, h, r, Lcap // chunk, chunk, d)
    with torch.cuda.device(k_cache.device):
        out = torch.empty(b, h, nt, r, d, dtype=dt, device=k_cache.device)
        lse = torch.empty(b, h, nt, r, dtype=torch.float32, device=k_cache.device)
        rc = lib.ua_decode_step(ctypes.byref(dims), _dtype_code(dt), _dtype_code(src.dtype), int(t), _ptr(k_cache), _ptr(v_cache),
                                _ptr(src), _ptr(q_t.contiguous()), _ptr(dst), _ptr(decay_state), _ptr(out), _ptr(lse), _stream())
    _lib.check(rc, "ua_decode_step")
    return out.permute(0, 1, 3, 4, 2), lse.permute(0, 1, 3, 2)


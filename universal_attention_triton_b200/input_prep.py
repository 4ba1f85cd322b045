"""Input prologue: token-major projections -> the operator's head-major inputs, in one CUDA pass each way.

The reference's driver does it with transposes and views (``main.py:24-31``); its harness additionally normalises the
keys and passes the gates through a sigmoid (``Universal_Attention/triton/_debug.py:470-475``).  ``prepare_inputs`` does
all of it in ``ua_prepare_inputs`` and is differentiable (``ua_prepare_inputs_bwd``)."""
from __future__ import annotations

import ctypes

import torch
from torch.autograd import Function

from . import _lib
from .ops import _dtype_code, _ptr, _require_cuda, _stream


class _PrepareInputs(Function):
    @staticmethod
    def forward(ctx, query_state, key_state, value_state, gate_state, chunk, normalize_keys, sigmoid_gates):
        _require_cuda(query_state, key_state, value_state, gate_state)
        lib = _lib.load()
        b, s, n, d = query_state.shape
        n_kv = key_state.shape[2]
        assert key_state.shape == (b, s, n_kv, d) and value_state.shape == (b, s, n_kv, d)
        assert gate_state.numel() == b * s * 2 * n_kv and n % n_kv == 0 and s % chunk == 0
        dt = query_state.dtype
        qs, ks, vs = query_state.contiguous(), key_state.to(dt).contiguous(), value_state.to(dt).contiguous()
        gs = gate_state.to(dt).contiguous()
        flags = (_lib.PREP_NORMALIZE_KEYS if normalize_keys else 0) | (_lib.PREP_SIGMOID_GATES if sigmoid_gates else 0)
        dev = qs.device
        with torch.cuda.device(dev):
            xq = torch.empty(b, n_kv, n // n_kv, s, d, dtype=dt, device=dev)
            kc = torch.empty(b, n_kv, s // chunk, chunk, d, dtype=dt, device=dev)
            vc = torch.empty_like(kc)
            ssrc = torch.empty(b, n_kv, s // chunk, chunk, dtype=dt, device=dev)
            sdest = torch.empty(b, n_kv, s, dtype=dt, device=dev)
            knorm = torch.empty(b, n_kv, s, dtype=torch.float32, device=dev) if normalize_keys else None
            rc = lib.ua_prepare_inputs(b, s, n, n_kv, d, _dtype_code(dt), flags, _ptr(qs), _ptr(ks), _ptr(vs), _ptr(gs),
                                       _ptr(xq), _ptr(kc), _ptr(vc), _ptr(ssrc), _ptr(sdest), _ptr(knorm), _stream())
        _lib.check(rc, "ua_prepare_inputs")
        ctx.dims = (b, s, n, n_kv, d, flags)
        ctx.in_shapes = (query_state.shape, key_state.shape, value_state.shape, gate_state.shape)
        ctx.save_for_backward(kc, ssrc, sdest, *([knorm] if knorm is not None else []))
        return kc, vc, xq, ssrc, sdest

    @staticmethod
    def backward(ctx, g_kc, g_vc, g_xq, g_src, g_dest):
        lib = _lib.load()
        b, s, n, n_kv, d, flags = ctx.dims
        kc, ssrc, sdest, *rest = ctx.saved_tensors
        knorm = rest[0] if rest else None
        dt = kc.dtype

        def full(g, like):
            return (torch.zeros_like(like) if g is None else g.to(dt)).contiguous()

        g_kc, g_vc = full(g_kc, kc), full(g_vc, kc)
        g_xq = full(g_xq, torch.empty(b, n_kv, n // n_kv, s, d, dtype=dt, device=kc.device))
        g_src, g_dest = full(g_src, ssrc), full(g_dest, sdest)
        with torch.cuda.device(kc.device):
            d_q = torch.empty(b, s, n, d, dtype=dt, device=kc.device)
            d_k = torch.empty(b, s, n_kv, d, dtype=dt, device=kc.device)
            d_v = torch.empty_like(d_k)
            d_g = torch.empty(b, s, 2, n_kv, dtype=dt, device=kc.device)
            rc = lib.ua_prepare_inputs_bwd(b, s, n, n_kv, d, _dtype_code(dt), flags, _ptr(g_xq), _ptr(g_kc), _ptr(g_vc), _ptr(g_src),
                                           _ptr(g_dest), _ptr(kc), _ptr(knorm), _ptr(ssrc), _ptr(sdest), _ptr(d_q), _ptr(d_k), _ptr(d_v),
                                           _ptr(d_g), _stream())
        _lib.check(rc, "ua_prepare_inputs_bwd")
        qsh, ksh, vsh, gsh = ctx.in_shapes
        return d_q.view(qsh), d_k.view(ksh), d_v.view(vsh), d_g.view(gsh), None, None, None


def prepare_inputs(query_state, key_state, value_state, gate_state, chunk=128, normalize_keys=False, sigmoid_gates=False):
    """``query_state (b,s,n,d)``, ``key_state, value_state (b,s,n_kv,d)``, ``gate_state (b,s,2*n_kv)`` (source gates
    first, as ``main.py:29-31`` splits them) -> ``(kc, vc, xq, static_src, static_dest)`` in the operator's 1-D layout:
    ``kc, vc (b,n_kv,s/chunk,chunk,d)``, ``xq (b,n_kv,n/n_kv,s,d)``, ``static_src (b,n_kv,s/chunk,chunk)``,
    ``static_dest (b,n_kv,s)``.  ``normalize_keys``: keys divided by ``|k| + 1e-6``; ``sigmoid_gates``: gates =
    sigmoid(gate_state).  Differentiable with respect to the four projections."""
    return _PrepareInputs.apply(query_state, key_state, value_state, gate_state, chunk, normalize_keys, sigmoid_gates)

"""Sequence-chunk sharding of the forward for long contexts.

Every rank owns a contiguous, equally long slice of the sequence (a whole number of 128-row
tiles) of all five inputs.  What crosses ranks (NCCL over NVLink through ``torch.distributed``):

1. all-gather of the keys, values and ``static_src`` (small next to ``out``: the output of one
   (b, h) is n times larger than its keys);
2. the decay carry: every rank sums, for every key of the sequence, the log-retention over its
   own rows (``decay_totals_rows``, a decay-only pass), the (b,h,n,128) totals are all-gathered,
   and a rank's carry is the sum of the totals of the ranks before it.

The per-(row, key-chunk) softmax statistics need no exchange with the reference's output format:
``denom[row, chunk]`` is complete on the rank that owns the row (it is itself the partial
log-sum-exp that a later merge over chunks consumes).

The prefix a row sees is then  carry(ranks before) + prefix inside the rank's own rows, which is
the single-GPU value up to the association of the fp32 sums.

Backward (``sp_backward``, bf16 / head_dim 64): the reverse decay carry runs from later rows to
earlier ones, but every gradient is LINEAR in it, so no rank waits for another:

3. every rank runs the backward of its own rows with a zero reverse carry and also returns, per
   key, the sum of the decay-prefix gradient over its rows (``dctot``);
4. the (b,h,n,128) ``dctot`` tables are all-gathered; a rank's reverse carry is the sum over the
   ranks AFTER it, and a decay-only correction pass adds the gradient that this carry induces;
5. the key-side gradients (dK, dV, d static_src: partial sums over the rank's rows for all keys)
   are summed over the ranks (all-reduce) and every rank keeps the slice of its own keys; dQ and
   d static_dest are row-local.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import ops


class CudaBackend:
    """The CUDA library (default)."""
    decay_totals_rows = staticmethod(ops.decay_totals_rows)
    forward_rows_cm = staticmethod(ops.forward_rows_cm)
    backward_rows = staticmethod(ops.backward_rows)
    backward_rows_suffix = staticmethod(ops.backward_rows_suffix)


def _all_gather_cat(t, dim, group):
    world = dist.get_world_size(group)
    parts = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(parts, t.contiguous(), group=group)
    return torch.cat(parts, dim=dim)


def sp_forward(kc_local, vc_local, xq_local, static_src_local, static_dest_local, group=None, backend=CudaBackend):
    """kc/vc_local (b,h,n_l,128,d), xq_local (b,h,r,L_l,d), static_src_local (b,h,n_l,128),
    static_dest_local (b,h,L_l): this rank's slice of the sequence, ``L_l = n_l * 128``, same on every rank.
    Returns ``(out, denom, lse)`` for the rank's rows against ALL key chunks, in the reference's shapes
    ``(b,h,r,L_l,d,n)`` / ``(b,h,r,L_l,n)`` (permuted views; ``lse`` is the fp32 denom)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    n_l = kc_local.shape[2]
    kc = _all_gather_cat(kc_local, 2, group)
    vc = _all_gather_cat(vc_local, 2, group)
    ss = _all_gather_cat(static_src_local, 2, group)
    begin, end = rank * n_l, (rank + 1) * n_l
    totals = backend.decay_totals_rows(kc, ss, static_dest_local, begin, end)
    parts = [torch.empty_like(totals) for _ in range(world)]
    dist.all_gather(parts, totals, group=group)
    carry = torch.zeros_like(totals)
    for g in range(rank):                     # fixed order: every rank forms the same partial sums
        carry = carry + parts[g]
    out_cm, lse_cm, denom_cm = backend.forward_rows_cm(kc, vc, xq_local, ss, static_dest_local, begin, end, carry)
    return ops.as_reference_out(out_cm), ops.as_reference_denom(denom_cm), ops.as_reference_denom(lse_cm)


def _carry_before(totals, rank, group):
    world = dist.get_world_size(group)
    parts = [torch.empty_like(totals) for _ in range(world)]
    dist.all_gather(parts, totals, group=group)
    carry = torch.zeros_like(totals)
    for g in range(rank):
        carry = carry + parts[g]
    return carry


def sp_backward(kc_local, vc_local, xq_local, static_src_local, static_dest_local, g_out_local, g_denom_local,
                group=None, backend=CudaBackend, skip_masked_grads: bool = False):
    """Gradients of the sequence-sharded operator.  Inputs as for ``sp_forward``; ``g_out_local (b,h,r,L_l,d,n)`` and
    ``g_denom_local (b,h,r,L_l,n)`` are the upstream gradients of the rank's rows (any strides).  Returns
    ``(dkc, dvc, dxq, dstatic_src, dstatic_dest)`` for the rank's own slice, shaped and typed like the local inputs."""
    from . import _lib
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    n_l = kc_local.shape[2]
    kc = _all_gather_cat(kc_local, 2, group)
    vc = _all_gather_cat(vc_local, 2, group)
    ss = _all_gather_cat(static_src_local, 2, group)
    begin, end = rank * n_l, (rank + 1) * n_l
    carry = _carry_before(backend.decay_totals_rows(kc, ss, static_dest_local, begin, end), rank, group)
    flags = _lib.FLAG_SKIP_MASKED_GRADS if skip_masked_grads else 0
    dk, dv, dxq, dsrc, ddest, dctot = backend.backward_rows(
        kc, vc, xq_local, ss, static_dest_local, ops.out_to_chunk_major(g_out_local), ops.denom_to_chunk_major(g_denom_local),
        begin, end, carry_in=carry, flags=flags)
    parts = [torch.empty_like(dctot) for _ in range(world)]
    dist.all_gather(parts, dctot, group=group)
    if rank + 1 < world:
        suffix = torch.zeros_like(dctot)
        for g in range(rank + 1, world):
            suffix = suffix + parts[g]
        backend.backward_rows_suffix(kc, vc, ss, static_dest_local, begin, end, suffix, dk, dsrc, ddest)
    for t in (dk, dv, dsrc):
        dist.all_reduce(t, group=group)
    b, h, n, c, d = kc.shape
    keys = slice(begin * c, end * c)
    return (dk[:, :, keys].reshape(kc_local.shape).to(kc_local.dtype), dv[:, :, keys].reshape(vc_local.shape).to(vc_local.dtype),
            dxq, dsrc[:, :, keys].reshape(static_src_local.shape).to(static_src_local.dtype),
            ddest.reshape(static_dest_local.shape).to(static_dest_local.dtype))

"""Sequence-chunk sharding of the operator for long contexts (one process per GPU, NCCL through
``torch.distributed``).

The sequence is cut into P equal blocks of whole 128-row tiles.  With the contiguous assignment P = G
and rank g owns block g; with the zig-zag assignment P = 2G and rank g owns blocks g and 2G-1-g, which
balances the causal work (a row sees all earlier keys, so late blocks are the expensive ones).  A rank's
local tensors are its blocks concatenated along the sequence, for all five inputs.

What crosses ranks:

1. all-gather of the keys, values and ``static_src`` (small next to ``out``: the output of one (b, h)
   is n times larger than its keys);
2. the decay carry: for every block, its owner sums every key's log-retention over the block's rows
   (``decay_totals_rows``, a decay-only pass); the (b,h,n,128) totals are all-gathered and a block's
   carry-in is the sum of the totals of the blocks before it;
3. (backward) the reverse decay carry runs from later rows to earlier ones, but every gradient is
   LINEAR in it, so nobody waits: each block's backward runs with a zero reverse carry and also returns
   the per-key sum of the decay-prefix gradient over its rows (``dctot``); these are all-gathered, a
   block's reverse carry is the sum over the blocks AFTER it, and a decay-only correction pass adds the
   gradient it induces;
4. (backward) dK, dV, d static_src -- fp32 partial sums over a rank's rows for ALL keys -- are
   all-reduced and every rank keeps the slice of its own keys.  dQ and d static_dest are row-local.

The per-(row, key-chunk) softmax statistics need no exchange with the reference's output format:
``denom[row, chunk]`` is complete on the rank that owns the row (it is itself the partial log-sum-exp
that a later merge over chunks consumes).  Results equal the single-GPU ones up to the association of
the fp32 carry sums.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import ops


class CudaBackend:
    """The CUDA library (default)."""
    decay_totals_rows = staticmethod(ops.decay_totals_rows)
    forward_rows_cm = staticmethod(ops.forward_rows_cm)
    alloc_forward_rows = staticmethod(ops.alloc_forward_rows)
    backward_rows = staticmethod(ops.backward_rows)
    backward_rows_suffix = staticmethod(ops.backward_rows_suffix)
    alloc_backward_rows = staticmethod(ops.alloc_backward_rows)


def owned_blocks(world: int, rank: int, zigzag: bool):
    """(P, [blocks of this rank in local order])."""
    if zigzag:
        return 2 * world, [rank, 2 * world - 1 - rank]
    return world, [rank]


def _gather_sequence(t_local, dim, group, zigzag):
    """All-gather a tensor whose axis `dim` holds this rank's blocks, and put the blocks in sequence order."""
    world = dist.get_world_size(group)
    parts = [torch.empty_like(t_local) for _ in range(world)]
    dist.all_gather(parts, t_local.contiguous(), group=group)
    if not zigzag:
        return torch.cat(parts, dim=dim)
    P = 2 * world
    blocks = [None] * P
    for g, t in enumerate(parts):
        first, second = t.chunk(2, dim=dim)
        blocks[g], blocks[P - 1 - g] = first, second
    return torch.cat(blocks, dim=dim)


def _gather_block_tables(tables, world, rank, zigzag, group):
    """tables: list (one per owned block, local order) of (b,h,n,128) tensors -> list of P tensors in block order."""
    stacked = torch.stack(tables)
    parts = [torch.empty_like(stacked) for _ in range(world)]
    dist.all_gather(parts, stacked, group=group)
    P, _ = owned_blocks(world, rank, zigzag)
    out = [None] * P
    for g in range(world):
        _, blks = owned_blocks(world, g, zigzag)
        for li, p in enumerate(blks):
            out[p] = parts[g][li]
    return out


def _setup(kc_local, vc_local, static_src_local, static_dest_local, group, backend, zigzag):
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    P, mine = owned_blocks(world, rank, zigzag)
    nb = kc_local.shape[2] // len(mine)                      # tiles (= key chunks of 128) per block
    kc = _gather_sequence(kc_local, 2, group, zigzag)
    vc = _gather_sequence(vc_local, 2, group, zigzag)
    ss = _gather_sequence(static_src_local, 2, group, zigzag)
    sd = static_dest_local.reshape(static_dest_local.shape[0], static_dest_local.shape[1], -1)
    rows_b = nb * kc.shape[3]                               # rows per block (row tile = key chunk = 128 rows on the GPU)
    totals = [backend.decay_totals_rows(kc, ss, sd, p * nb, (p + 1) * nb, row_offset=li * rows_b) for li, p in enumerate(mine)]
    all_tot = _gather_block_tables(totals, world, rank, zigzag, group)
    carries = []
    run = torch.zeros_like(all_tot[0])
    for p in range(P):                                       # fixed order: every rank forms the same partial sums
        carries.append(run)
        run = run + all_tot[p]
    return world, rank, P, mine, nb, kc, vc, ss, sd, carries


def sp_forward(kc_local, vc_local, xq_local, static_src_local, static_dest_local, group=None, backend=CudaBackend,
               zigzag: bool = False, return_ctx: bool = False):
    """kc/vc_local (b,h,n_l,128,d), xq_local (b,h,r,L_l,d), static_src_local (b,h,n_l,128), static_dest_local (b,h,L_l):
    this rank's blocks of the sequence (``L_l = n_l * 128``, same on every rank; two blocks when ``zigzag``).
    Returns ``(out, denom, lse)`` for the rank's rows against ALL key chunks, in the reference's shapes
    ``(b,h,r,L_l,d,n)`` / ``(b,h,r,L_l,n)`` (permuted views; ``lse`` is the fp32 denom).  With ``return_ctx`` a
    fourth value: the gathered keys / values / gates and the decay carries, which ``sp_backward(ctx=...)`` reuses
    instead of gathering and summing them again."""
    setup = _setup(kc_local, vc_local, static_src_local, static_dest_local, group, backend, zigzag)
    world, rank, P, mine, nb, kc, vc, ss, sd, carries = setup
    xq = xq_local.contiguous()
    out = backend.alloc_forward_rows(kc, xq)
    for li, p in enumerate(mine):
        backend.forward_rows_cm(kc, vc, xq, ss, sd, p * nb, (p + 1) * nb, carries[p], row_offset=li * nb * kc.shape[3], out=out)
    out_cm, lse_cm, denom_cm = out
    res = (ops.as_reference_out(out_cm), ops.as_reference_denom(denom_cm), ops.as_reference_denom(lse_cm))
    return res + (setup,) if return_ctx else res


def sp_backward(kc_local, vc_local, xq_local, static_src_local, static_dest_local, g_out_local, g_denom_local,
                group=None, backend=CudaBackend, zigzag: bool = False, skip_masked_grads: bool = False, ctx=None):
    """Gradients of the sequence-sharded operator.  Inputs as for ``sp_forward``; ``g_out_local (b,h,r,L_l,d,n)`` and
    ``g_denom_local (b,h,r,L_l,n)`` are the upstream gradients of the rank's rows (any strides).  Returns
    ``(dkc, dvc, dxq, dstatic_src, dstatic_dest)`` for the rank's own blocks, shaped and typed like the local inputs."""
    from . import _lib
    if ctx is None:         # ``ctx``: what ``sp_forward(return_ctx=True)`` returned for the same inputs and assignment
        ctx = _setup(kc_local, vc_local, static_src_local, static_dest_local, group, backend, zigzag)
    world, rank, P, mine, nb, kc, vc, ss, sd, carries = ctx
    flags = _lib.FLAG_SKIP_MASKED_GRADS if skip_masked_grads else 0
    xq = xq_local.contiguous()
    g_out_cm = ops.out_to_chunk_major(g_out_local)
    g_den_cm = ops.denom_to_chunk_major(g_denom_local)
    acc = backend.alloc_backward_rows(kc, xq)
    dctots = []
    for li, p in enumerate(mine):
        res = backend.backward_rows(kc, vc, xq, ss, sd, g_out_cm, g_den_cm, p * nb, (p + 1) * nb, carry_in=carries[p],
                                    flags=flags, row_offset=li * nb * kc.shape[3], acc=acc)
        dctots.append(res[5])
    dk, dv, dxq, dsrc, ddest = acc
    all_dct = _gather_block_tables(dctots, world, rank, zigzag, group)
    for li, p in enumerate(mine):
        if p + 1 < P:
            suffix = torch.zeros_like(all_dct[0])
            for q in range(p + 1, P):
                suffix = suffix + all_dct[q]
            backend.backward_rows_suffix(kc, vc, ss, sd, p * nb, (p + 1) * nb, suffix, dk, dsrc, ddest, row_offset=li * nb * kc.shape[3])
    for t in (dk, dv, dsrc):
        dist.all_reduce(t, group=group)
    c = kc.shape[3]
    pick = lambda t: torch.cat([t[:, :, p * nb * c:(p + 1) * nb * c] for p in mine], dim=2)
    return (pick(dk).reshape(kc_local.shape).to(kc_local.dtype), pick(dv).reshape(vc_local.shape).to(vc_local.dtype),
            dxq.reshape(xq_local.shape).to(xq_local.dtype), pick(dsrc).reshape(static_src_local.shape).to(static_src_local.dtype),
            ddest.reshape(static_dest_local.shape).to(static_dest_local.dtype))

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
4. (backward) dK, dV, d static_src -- fp32 partial sums over a rank's rows for ALL keys -- are packed
   destination-rank-major and reduce-scattered in ONE collective: every rank receives only the sums for
   its own keys.  dQ and d static_dest are row-local.

Collectives per step: forward 1 all-gather (K | V | src, byte-packed) + 1 all-gather of the decay totals;
backward 1 all-gather of the dC totals + 1 reduce-scatter (dK | dV | dsrc, fp32).

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
    alloc_carry_table = staticmethod(ops.alloc_carry_table)     # (backends without it: the backward recomputes)


def owned_blocks(world: int, rank: int, zigzag: bool):
    """(P, [blocks of this rank in local order])."""
    if zigzag:
        return 2 * world, [rank, 2 * world - 1 - rank]
    return world, [rank]


def _block_order(world: int, zigzag: bool):
    """Block ids in the order (rank 0's blocks, rank 1's blocks, ...)."""
    return [p for g in range(world) for p in owned_blocks(world, g, zigzag)[1]]


def _gather_sequence(locals_, group, zigzag):
    """ONE all-gather for several local tensors whose axis 2 holds this rank's blocks (keys, values, static_src:
    byte-packed into one send buffer, received into one preallocated buffer), then the blocks of each tensor are put
    in sequence order with a single copy."""
    world = dist.get_world_size(group)
    flat = [t.contiguous().view(torch.uint8).reshape(-1) for t in locals_]
    sizes = [f.numel() for f in flat]
    assert all(sz % 4 == 0 for sz in sizes)
    send = torch.cat(flat)
    recv = torch.empty(world * send.numel(), dtype=torch.uint8, device=send.device)
    dist.all_gather_into_tensor(recv, send, group=group)
    recv = recv.view(world, -1)
    outs, off = [], 0
    for t, sz in zip(locals_, sizes):
        parts = recv[:, off:off + sz].view(t.dtype).reshape((world,) + tuple(t.shape))      # (G, b, h, n_l, ...)
        off += sz
        nd = parts.dim()
        tail = list(range(4, nd))
        if not zigzag:
            full = parts.permute(1, 2, 0, 3, *tail)                                              # (b, h, G, n_l, ...)
        else:
            nb = t.shape[2] // 2
            halves = parts.reshape((world, t.shape[0], t.shape[1], 2, nb) + tuple(t.shape[3:]))    # (G, b, h, 2, nb, ...)
            tail2 = list(range(5, halves.dim()))
            first = halves[:, :, :, 0].permute(1, 2, 0, 3, *[x - 1 for x in tail2])               # blocks 0 .. G-1
            second = halves[:, :, :, 1].flip(0).permute(1, 2, 0, 3, *[x - 1 for x in tail2])      # blocks G .. 2G-1
            full = torch.cat([first, second], dim=2)
        outs.append(full.reshape((t.shape[0], t.shape[1], -1) + tuple(t.shape[3:])))
    return outs


def _gather_block_tables(tables, world, rank, zigzag, group):
    """tables: list (one per owned block, local order) of (b,h,n,128) tensors -> (P, b,h,n,128) stacked in block order."""
    stacked = torch.stack(tables).contiguous()
    recv = torch.empty(world * stacked.numel(), dtype=stacked.dtype, device=stacked.device)
    dist.all_gather_into_tensor(recv, stacked.reshape(-1), group=group)
    recv = recv.reshape((-1,) + tuple(stacked.shape[1:]))                # (rank-major, local block) = _block_order
    order = torch.tensor(_block_order(world, zigzag), device=recv.device)
    out = torch.empty_like(recv)
    out[order] = recv
    return out


def _reduce_scatter_keys(parts, kc_local_shape, world, zigzag, group):
    """``parts``: fp32 partial sums over this rank's rows for ALL keys, each (b,h,L[,d]).  Every rank needs only the sum for
    its OWN keys: the tensors are packed destination-rank-major and ONE reduce-scatter returns this rank's segment
    (1/G of the bytes an all-reduce would bring back).  Returns the tensors restricted to the rank's blocks, (b,h,L_l[,d])."""
    order = _block_order(world, zigzag)
    P = len(order)
    idx = torch.tensor(order, device=parts[0].device)
    packed, shapes = [], []
    for t in parts:
        b, h, L = t.shape[:3]
        blk = t.reshape((b, h, P, L // P) + tuple(t.shape[3:]))
        perm = blk.permute(2, 0, 1, 3, *range(4, blk.dim()))[idx]         # (P in destination order, b, h, rows, ...)
        shapes.append(tuple(perm.shape[1:]))
        packed.append(perm.reshape(world, -1))
    send = torch.cat(packed, dim=1).contiguous()
    recv = torch.empty(send.shape[1], dtype=send.dtype, device=send.device)
    if dist.get_backend(group) == "gloo":      # no reduce-scatter on the CPU backend of the tests
        dist.all_reduce(send, group=group)
        recv = send[dist.get_rank(group)].clone()
    else:
        dist.reduce_scatter_tensor(recv, send, group=group)
    outs, off = [], 0
    per = P // world
    for shp in shapes:
        nel = per * int(torch.tensor(shp).prod())
        mine = recv[off:off + nel].reshape((per,) + shp)                 # (own blocks, b, h, rows, ...)
        off += nel
        mine = mine.permute(1, 2, 0, 3, *range(4, mine.dim()))
        outs.append(mine.reshape((shp[0], shp[1], -1) + shp[3:]))
    return outs


def _setup(kc_local, vc_local, static_src_local, static_dest_local, group, backend, zigzag):
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    P, mine = owned_blocks(world, rank, zigzag)
    nb = kc_local.shape[2] // len(mine)                      # tiles (= key chunks of 128) per block
    kc, vc, ss = _gather_sequence([kc_local, vc_local, static_src_local], group, zigzag)
    sd = static_dest_local.reshape(static_dest_local.shape[0], static_dest_local.shape[1], -1)
    rows_b = nb * kc.shape[3]                               # rows per block (row tile = key chunk = 128 rows on the GPU)
    totals = [backend.decay_totals_rows(kc, ss, sd, p * nb, (p + 1) * nb, row_offset=li * rows_b) for li, p in enumerate(mine)]
    all_tot = _gather_block_tables(totals, world, rank, zigzag, group)
    carries = all_tot.cumsum(0) - all_tot                    # exclusive prefix over the blocks (same order on every rank)
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
    # with return_ctx the forward also hands its decay-prefix table and log-sum-exp to the backward
    table = backend.alloc_carry_table(kc) if (return_ctx and hasattr(backend, "alloc_carry_table")) else None
    extra = {"carry_table": table} if table is not None else {}
    for li, p in enumerate(mine):
        backend.forward_rows_cm(kc, vc, xq, ss, sd, p * nb, (p + 1) * nb, carries[p], row_offset=li * nb * kc.shape[3], out=out,
                                **extra)
    out_cm, lse_cm, denom_cm = out
    res = (ops.as_reference_out(out_cm), ops.as_reference_denom(denom_cm), ops.as_reference_denom(lse_cm))
    return res + (setup + ((table, lse_cm) if table is not None else ()),) if return_ctx else res


def sp_backward(kc_local, vc_local, xq_local, static_src_local, static_dest_local, g_out_local, g_denom_local,
                group=None, backend=CudaBackend, zigzag: bool = False, skip_masked_grads: bool = False, ctx=None):
    """Gradients of the sequence-sharded operator.  Inputs as for ``sp_forward``; ``g_out_local (b,h,r,L_l,d,n)`` and
    ``g_denom_local (b,h,r,L_l,n)`` are the upstream gradients of the rank's rows (any strides).  Returns
    ``(dkc, dvc, dxq, dstatic_src, dstatic_dest)`` for the rank's own blocks, shaped and typed like the local inputs."""
    from . import _lib
    if ctx is None:         # ``ctx``: what ``sp_forward(return_ctx=True)`` returned for the same inputs and assignment
        ctx = _setup(kc_local, vc_local, static_src_local, static_dest_local, group, backend, zigzag)
    world, rank, P, mine, nb, kc, vc, ss, sd, carries = ctx[:10]
    kept = {"carry_table": ctx[10], "lse_cm_rows": ctx[11]} if len(ctx) > 10 else {}
    flags = _lib.FLAG_SKIP_MASKED_GRADS if skip_masked_grads else 0
    xq = xq_local.contiguous()
    g_out_cm = ops.out_to_chunk_major(g_out_local)
    g_den_cm = ops.denom_to_chunk_major(g_denom_local)
    acc = backend.alloc_backward_rows(kc, xq)
    dctots = []
    for li, p in enumerate(mine):
        res = backend.backward_rows(kc, vc, xq, ss, sd, g_out_cm, g_den_cm, p * nb, (p + 1) * nb, carry_in=carries[p],
                                    flags=flags, row_offset=li * nb * kc.shape[3], acc=acc, **kept)
        dctots.append(res[5])
    dk, dv, dxq, dsrc, ddest = acc
    all_dct = _gather_block_tables(dctots, world, rank, zigzag, group)
    suffixes = all_dct.flip(0).cumsum(0).flip(0) - all_dct   # sum over the blocks AFTER each block
    for li, p in enumerate(mine):
        if p + 1 < P:
            backend.backward_rows_suffix(kc, vc, ss, sd, p * nb, (p + 1) * nb, suffixes[p], dk, dsrc, ddest,
                                         row_offset=li * nb * kc.shape[3])
    dk_l, dv_l, dsrc_l = _reduce_scatter_keys([dk, dv, dsrc], kc_local.shape, world, zigzag, group)
    return (dk_l.reshape(kc_local.shape).to(kc_local.dtype), dv_l.reshape(vc_local.shape).to(vc_local.dtype),
            dxq.reshape(xq_local.shape).to(xq_local.dtype), dsrc_l.reshape(static_src_local.shape).to(static_src_local.dtype),
            ddest.reshape(static_dest_local.shape).to(static_dest_local.dtype))

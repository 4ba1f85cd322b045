"""(batch, kv-head) sharding of the operator over the GPUs of one box.

The units `(b, h)` of the operator are independent (no term couples two kv
heads or two batch rows), so N ranks each take a contiguous range of the
flattened `b*h` list and run the single-GPU operator on it: no collective on
the data path.  One process per GPU; `torch.distributed` is only used by the
callers for rendezvous, timing barriers and (in tests) to gather results.
"""
from __future__ import annotations

from typing import Callable, Sequence, Tuple

import torch


def unit_range(n_units: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced range [lo, hi) of units for `rank`; the first `n_units % world` ranks get one more."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    base, extra = divmod(n_units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_inputs(tensors: Sequence[torch.Tensor], world: int, rank: int):
    """Slice (kc, vc, xq, static_src, static_dest), all shaped (b, h, ...), to this rank's units.
    Returns tensors shaped (1, units, ...) and the unit range."""
    b, h = tensors[0].shape[:2]
    lo, hi = unit_range(b * h, world, rank)
    out = []
    for t in tensors:
        flat = t.reshape((b * h,) + tuple(t.shape[2:]))
        out.append(flat[lo:hi].unsqueeze(0).contiguous())
    return out, (lo, hi)


def run_sharded(op: Callable, tensors: Sequence[torch.Tensor], world: int, rank: int):
    """Run `op(kc, vc, xq, static_src, static_dest)` on this rank's shard; returns its outputs
    (shaped (1, units, ...)) and the unit range they cover."""
    shard, rng = shard_inputs(tensors, world, rank)
    if rng[0] == rng[1]:
        return None, rng
    return op(*shard), rng

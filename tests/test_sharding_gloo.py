"""(batch, kv-head) sharding across ranks: world-size-2 gloo processes on CPU.
The CPU oracle stands in for the operator (no GPU here); the test checks that the
shards cover every unit exactly once and that gathered shard results equal the
unsharded result bit for bit (units are independent: no collective is needed)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from universal_attention_triton_b200.sharding import run_sharded, unit_range


def test_unit_ranges_partition():
    for n in (1, 5, 32, 128):
        for world in (1, 2, 3, 4, 8):
            covered = []
            for r in range(world):
                lo, hi = unit_range(n, world, r)
                covered += list(range(lo, hi))
            assert covered == list(range(n))
    with pytest.raises(ValueError):
        unit_range(4, 2, 2)


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import ua_oracle as O
    torch.set_num_threads(1)
    ins = O.make_inputs(3, 1, 2, 64, 16, 8, seed=4)          # 3 units over 2 ranks: uneven split

    def op(kc, vc, xq, ss, sd):
        out, denom, _ = O.ua_forward(kc, vc, xq, ss, sd)
        return out, denom

    (out, denom), (lo, hi) = run_sharded(op, ins, world, rank)
    full_out, full_denom, _ = O.ua_forward(*ins)
    flat = full_out.reshape((3,) + tuple(full_out.shape[2:]))
    ok = torch.equal(out[0], flat[lo:hi]) and torch.equal(denom[0], full_denom.reshape((3,) + tuple(full_denom.shape[2:]))[lo:hi])
    counts = torch.tensor([hi - lo], dtype=torch.int64)
    dist.all_reduce(counts)
    flag = torch.tensor([1 if ok else 0], dtype=torch.int64)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        ret["units"] = int(counts.item())
        ret["ok"] = int(flag.item())
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_matches_unsharded():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret["units"] == 3 and ret["ok"] == 1

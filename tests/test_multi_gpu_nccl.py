"""Multi-GPU tests over NCCL (skipped on a single-GPU box): the sequence-sharded forward and backward on 2 (and, where
the box has them, 4) GPUs against the CPU oracle restricted to each rank's rows and keys, and (batch, kv-head) sharding
of forward + backward."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _sp_worker(rank, world, port, ret, zigzag):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from oracle import ua_oracle as O
    from universal_attention_triton_b200 import ops
    from universal_attention_triton_b200.sequence_parallel import sp_forward
    B, H, R, L, c, D = 1, 2, 2, 2048, 128, 64
    ins = [t.cuda() for t in O.make_inputs(B, H, R, L, c, D, dtype=torch.bfloat16, seed=61)]
    kc, vc, xq, ss, sd = ins
    from universal_attention_triton_b200.sequence_parallel import owned_blocks
    n = L // c
    P, mine = owned_blocks(world, rank, zigzag)
    nb = n // P
    sc = torch.cat([torch.arange(p * nb, (p + 1) * nb) for p in mine]).cuda()
    sr = torch.cat([torch.arange(p * nb * c, (p + 1) * nb * c) for p in mine]).cuda()
    out, denom, lse, ctx = sp_forward(kc[:, :, sc].contiguous(), vc[:, :, sc].contiguous(), xq[:, :, :, sr].contiguous(),
                                      ss[:, :, sc].contiguous(), sd[:, :, sr].contiguous(), zigzag=zigzag, return_ctx=True)
    # the oracle (CPU, fp32, fed the same bf16 values) on the whole sequence, restricted to this rank's rows / keys
    ins32 = [t.float().cpu() for t in ins]
    ref_out, _, ref_lse = O.ua_forward(*ins32)
    src_, srr = sc.cpu(), sr.cpu()
    valid = (torch.arange(L).view(L, 1) >= torch.arange(n).view(1, n) * c)[srr]
    e_lse = ((lse.cpu() - ref_lse[:, :, :, srr]).abs() * valid).max().item()
    e_out = ((out.float().cpu() - ref_out[:, :, :, srr]).abs() * valid.view(-1, 1, n)).max().item()
    ok = e_lse <= 2e-2 and e_out <= 2e-2 + 2.0 ** -9 * ref_out.abs().max().item()      # (+ half a bf16 ulp of the largest output)
    # backward: random upstream gradients of the rank's rows
    from universal_attention_triton_b200.sequence_parallel import sp_backward
    gen = torch.Generator().manual_seed(63)
    g_out = torch.randn(B, H, R, L, D, n, generator=gen).bfloat16()
    g_den = torch.randn(B, H, R, L, n, generator=gen)
    want = O.ua_backward(*ins32, g_out.float(), g_den)
    got = sp_backward(kc[:, :, sc].contiguous(), vc[:, :, sc].contiguous(), xq[:, :, :, sr].contiguous(),
                      ss[:, :, sc].contiguous(), sd[:, :, sr].contiguous(),
                      g_out.cuda()[:, :, :, sr], g_den.cuda()[:, :, :, sr], zigzag=zigzag,
                      ctx=ctx if zigzag else None)       # one assignment reuses the forward's gathers and carries, the other redoes them
    want_local = (want[0][:, :, src_], want[1][:, :, src_], want[2][:, :, :, srr], want[3][:, :, src_], want[4][:, :, srr])
    worst = 0.0
    for a, b_ in zip(got, want_local):
        rel = ((a.float().cpu() - b_).norm() / b_.norm().clamp_min(1e-20)).item()
        worst = max(worst, rel)
        ok = ok and a.shape == b_.shape and rel <= 5e-2
    print(f"[sp world={world} zigzag={zigzag} rank={rank}] lse {e_lse:.3e} out {e_out:.3e} worst grad rel-Frobenius {worst:.3e}", flush=True)
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        ret["ok"] = int(flag.item())
    dist.barrier()
    dist.destroy_process_group()


def _bh_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from oracle import ua_oracle as O
    from universal_attention_triton_b200 import UniversalAttention
    from universal_attention_triton_b200.sharding import run_sharded
    B, H, R, L, c, D = 3, 1, 2, 512, 128, 64             # 3 units over 2 ranks
    ins = [t.cuda() for t in O.make_inputs(B, H, R, L, c, D, dtype=torch.bfloat16, seed=62)]
    (out, denom), (lo, hi) = run_sharded(UniversalAttention.apply, ins, world, rank)
    full_out, full_denom = UniversalAttention.apply(*ins)
    flat = full_out.reshape((B * H,) + tuple(full_out.shape[2:]))
    ok = torch.equal(out[0], flat[lo:hi])
    cnt = torch.tensor([hi - lo], device="cuda")
    dist.all_reduce(cnt)
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        ret["ok"] = int(flag.item())
        ret["units"] = int(cnt.item())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,zigzag", [(2, False), (2, True), (4, True)])
def test_sequence_sharded_forward_and_backward_against_the_oracle(world, zigzag):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ret = mp.Manager().dict()
    mp.spawn(_sp_worker, args=(world, _free_port(), ret, zigzag), nprocs=world, join=True)
    assert ret["ok"] == 1


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_batch_head_sharding_two_gpus():
    ret = mp.Manager().dict()
    mp.spawn(_bh_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert ret["ok"] == 1 and ret["units"] == 3

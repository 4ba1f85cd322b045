"""Two-GPU tests over NCCL (skipped on a single-GPU box): the sequence-sharded forward against the
single-GPU forward of the same library, and (batch, kv-head) sharding of forward + backward."""
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
    B, H, R, L, c, D = 1, 2, 2, 1024, 128, 64
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
    out_cm, lse_cm, _ = ops.forward_cm(kc, vc, xq, ss, sd)
    ref_out = ops.as_reference_out(out_cm)[:, :, :, sr]
    ref_lse = ops.as_reference_denom(lse_cm)[:, :, :, sr]
    valid = (torch.arange(L).view(L, 1) >= torch.arange(n).view(1, n) * c).cuda()[sr]
    ok = bool((((lse - ref_lse).abs() <= 1e-3 + 1e-6 * ref_lse.abs()) | ~valid).all().item())
    ok = ok and bool(((out.float() - ref_out.float()).abs() <= 2e-2 + ref_out.float().abs() * 2.0 ** -7).all().item())
    # backward: random upstream gradients of the rank's rows, against the single-GPU backward
    from universal_attention_triton_b200.sequence_parallel import sp_backward
    gen = torch.Generator(device="cuda").manual_seed(63)
    g_out = torch.randn(B, H, n, R, L, D, generator=gen, device="cuda", dtype=torch.bfloat16)
    g_lse = torch.randn(B, H, n, R, L, generator=gen, device="cuda")
    want = ops.backward_cm(kc, vc, xq, ss, sd, g_out, g_lse)
    got = sp_backward(kc[:, :, sc].contiguous(), vc[:, :, sc].contiguous(), xq[:, :, :, sr].contiguous(),
                      ss[:, :, sc].contiguous(), sd[:, :, sr].contiguous(),
                      ops.as_reference_out(g_out)[:, :, :, sr], ops.as_reference_denom(g_lse)[:, :, :, sr], zigzag=zigzag,
                      ctx=ctx if zigzag else None)       # one assignment reuses the forward's gathers and carries, the other redoes them
    want_local = (want[0][:, :, sc], want[1][:, :, sc], want[2][:, :, :, sr], want[3][:, :, sc], want[4][:, :, sr])
    for a, b_ in zip(got, want_local):
        rel = ((a.float() - b_.float()).norm() / b_.float().norm().clamp_min(1e-20)).item()
        ok = ok and a.shape == b_.shape and rel <= 1e-2
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


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("zigzag", [False, True])
def test_sequence_sharded_forward_and_backward_two_gpus(zigzag):
    ret = mp.Manager().dict()
    mp.spawn(_sp_worker, args=(2, _free_port(), ret, zigzag), nprocs=2, join=True)
    assert ret["ok"] == 1


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_batch_head_sharding_two_gpus():
    ret = mp.Manager().dict()
    mp.spawn(_bh_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert ret["ok"] == 1 and ret["units"] == 3

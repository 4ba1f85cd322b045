"""Sequence-chunk sharded forward (sequence_parallel.sp_forward) on two gloo ranks, CPU.
The exchange logic (all-gather of keys/values/src gates, all-gather of per-rank decay totals, carry =
sum of the totals of the earlier ranks) runs for real; a CPU stand-in built on the oracle's arithmetic
takes the place of the two CUDA entry points.  The gathered result must equal the unsharded oracle."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


class OracleBackend:
    """CPU stand-ins for ops.decay_totals_rows / ops.forward_rows_cm (row tiles = key chunks here)."""

    @staticmethod
    def _ell_rows(kc, ss, sd_rows, begin, end):
        from oracle import ua_oracle as O
        b, h, n, c, d = kc.shape
        L = n * c
        k = kc.reshape(b, h, L, d).float()
        rows = k[:, :, begin * c:end * c]
        gram = k @ rows.transpose(-1, -2)                                   # (b,h,L keys, Lr rows)
        aff = gram.clamp_min(0).pow(2.0 / 3.0) * ss.reshape(b, h, L, 1).float().pow(1.0 / 3.0) * \
            sd_rows.reshape(b, h, 1, -1).float().pow(1.0 / 3.0)
        ell = torch.log1p(-aff.clamp(0, torch.tensor(O.CLAMP_MAX, dtype=torch.float32).item()))
        kidx = torch.arange(L).view(L, 1)
        qidx = torch.arange(begin * c, end * c).view(1, -1)
        return torch.where(qidx > kidx, ell, torch.zeros(())), kidx, qidx

    @staticmethod
    def decay_totals_rows(kc, ss, sd_slab, begin, end, carry_in=None, row_offset=0):
        b, h, n, c, d = kc.shape
        sd_rows = sd_slab[:, :, row_offset:row_offset + (end - begin) * c]
        ell, _, _ = OracleBackend._ell_rows(kc, ss, sd_rows, begin, end)
        tot = ell.sum(-1).view(b, h, n, c)
        return tot if carry_in is None else tot + carry_in

    @staticmethod
    def alloc_forward_rows(kc, xq_slab):
        b, h, n, c, d = kc.shape
        r, Ls = xq_slab.shape[2], xq_slab.shape[3]
        return (torch.zeros(b, h, n, r, Ls, d), torch.zeros(b, h, n, r, Ls), torch.zeros(b, h, n, r, Ls))

    @staticmethod
    def forward_rows_cm(kc, vc, xq_slab, ss, sd_slab, begin, end, carry, flags=0, row_offset=0, out=None):
        from oracle import ua_oracle as O
        b, h, n, c, d = kc.shape
        L = n * c
        r = xq_slab.shape[2]
        nrows = (end - begin) * c
        xq_rows = xq_slab[:, :, :, row_offset:row_offset + nrows]
        sd_rows = sd_slab[:, :, row_offset:row_offset + nrows]
        ell, kidx, qidx = OracleBackend._ell_rows(kc, ss, sd_rows, begin, end)
        decay = ell.cumsum(-1) + carry.reshape(b, h, L, 1)
        decay = torch.where(qidx < kidx, torch.full((), O.MASK_VALUE), decay)
        k = kc.reshape(b, h, L, d).float()
        score = (k.unsqueeze(2) @ xq_rows.float().transpose(-1, -2) + decay.unsqueeze(2)).view(b, h, r, n, c, -1)
        lse = score.logsumexp(dim=-2)                                       # (b,h,r,n,Lr)
        prob = score.softmax(dim=-2)
        res = prob.transpose(-1, -2) @ vc.float().view(b, h, 1, n, c, d)   # (b,h,r,n,Lr,d)
        out[0][:, :, :, :, row_offset:row_offset + nrows] = res.permute(0, 1, 3, 2, 4, 5)
        out[1][:, :, :, :, row_offset:row_offset + nrows] = lse.permute(0, 1, 3, 2, 4)
        out[2][:, :, :, :, row_offset:row_offset + nrows] = lse.permute(0, 1, 3, 2, 4)
        return out


def _worker(rank, world, port, ret, zigzag):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    from oracle import ua_oracle as O
    from universal_attention_triton_b200.sequence_parallel import sp_forward
    B, H, R, L, c, D = 1, 2, 2, 128, 16, 8
    kc, vc, xq, ss, sd = O.make_inputs(B, H, R, L, c, D, seed=6)
    from universal_attention_triton_b200.sequence_parallel import owned_blocks
    n = L // c
    P, mine = owned_blocks(world, rank, zigzag)
    nb = n // P
    sl_c = torch.cat([torch.arange(p * nb, (p + 1) * nb) for p in mine])
    sl_r = torch.cat([torch.arange(p * nb * c, (p + 1) * nb * c) for p in mine])
    out, denom, lse = sp_forward(kc[:, :, sl_c], vc[:, :, sl_c], xq[:, :, :, sl_r], ss[:, :, sl_c], sd[:, :, sl_r],
                                 backend=OracleBackend, zigzag=zigzag)
    ref_out, ref_denom, _ = O.ua_forward(kc, vc, xq, ss, sd)
    ok = (out.shape == ref_out[:, :, :, sl_r].shape and
          (out - ref_out[:, :, :, sl_r]).abs().max().item() < 1e-4 and
          ((denom - ref_denom[:, :, :, sl_r]).abs() / ref_denom[:, :, :, sl_r].abs().clamp_min(1)).max().item() < 1e-5)
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        ret["ok"] = int(flag.item())
    dist.barrier()
    dist.destroy_process_group()


import pytest


@pytest.mark.parametrize("zigzag", [False, True])
def test_two_rank_sequence_sharded_forward_matches_unsharded(zigzag):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, ret, zigzag), nprocs=2, join=True)
    assert ret["ok"] == 1

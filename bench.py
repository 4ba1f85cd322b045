#!/usr/bin/env python
"""Benchmark of the Universal Attention hot path (operator forward + backward).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2]

Prints ONE JSON line on rank 0.  A step is one forward + one backward of the
operator over one batch of seeded synthetic inputs of the named workload:

* ``value``  tokens/s (tokens = batch * L per step, summed over ranks) with all
  inputs and upstream gradients resident in HBM, timed with CUDA events.
* ``e2e``    the same metric through the public autograd entry points with HOST
  (pinned) inputs: host->device copies, operator, SMVecMatMul, loss, backward,
  and the device->host read of the loss and the five gradients are all timed.
* ``roofline``      the dominant kernel's algorithmic FLOPs / measured time against
  the measured bf16 tensor peak (MEASURED_PEAKS.json) or the stated fallback.
* ``cpu_baseline``  the CPU oracle (a port of the reference's PyTorch path) on a
  bounded sample of the same workload, on this host's cores.

``--impl reference`` times that CPU path alone and prints the same line shape.
For N > 1 launch with ``python -m torch.distributed.run --nproc-per-node N``;
every rank processes its own batch shard (weak scaling, no collective on the
data path).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: B, H, R, L, chunk, D, dtype, qkv_std, gate_mean, gate_std, fwd_only
    "c1": dict(B=1, H=2, R=2, L=256, c=64, D=64, dtype="f32", std=1.0, gm=0.0, gs=1.0, fwd_only=False),
    "c2": dict(B=4, H=8, R=4, L=4096, c=128, D=64, dtype="bf16", std=1.0, gm=0.0, gs=1.0, fwd_only=False),
    # a (batch, kv-head) slice of c2 for profiler captures: small on the device, out tensor still larger than L2
    "c2s": dict(B=1, H=2, R=4, L=4096, c=128, D=64, dtype="bf16", std=1.0, gm=0.0, gs=1.0, fwd_only=False),
    # long context for sequence-chunk sharding (--mode sp): config 4's sequence regime at the chunk / head_dim the
    # tensor-core backward supports; L is the TOTAL sequence, split over the ranks
    "long": dict(B=1, H=8, R=4, L=32768, c=128, D=64, dtype="bf16", std=1.0, gm=0.0, gs=1.0, fwd_only=False),
    "c3": dict(B=16, H=8, R=4, L=8192, c=128, D=128, dtype="bf16", std=0.5, gm=0.0, gs=1.0, fwd_only=True),
    "c5": dict(B=8, H=16, R=1, L=16384, c=128, D=128, dtype="bf16", std=1.0, gm=-4.0, gs=2.0, fwd_only=False),
}
METRIC = "fwd+bwd tokens/sec"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


# DRAM bytes per backward call at workload c2, from one ncu capture of a slice of 2 of the 32 (batch, kv-head) units: the
# keys-on-lanes kernel (163.69 MB read, of which 67 MB are the forward's output tiles, + 7.74 MB written), the sweep over
# the rows before each chunk (80.87 + 2.04 MB) and the row-side finish (5.30 MB); the small per-chunk kernels and the
# fp32 -> bf16 conversions are not in the figure.  The traffic grows in proportion to
# the units.  No figure is given for the forward: a capture of that slice ends with part of the 134 MB it writes still in
# the 126 MB L2, so its DRAM write count understates a full launch.
NCU_DRAM_BYTES = {"c2": {"fwd": None, "bwd": 16 * (163.686400e6 + 7.741696e6 + 80.872704e6 + 2.036992e6 + 5.299456e6)}}


def flops(w):
    n = w["L"] // w["c"]
    base = 2.0 * w["B"] * w["H"] * w["L"] ** 2 * w["D"] * (n + 1) / (2 * n)
    f_fwd = base * (1 + 2 * w["R"])
    f_bwd = 0.0 if w["fwd_only"] else base * (3 + 5 * w["R"])
    return f_fwd, f_bwd


def hbm_bytes(w):
    e = 2 if w["dtype"] == "bf16" else 4
    bh = w["B"] * w["H"]
    n = w["L"] // w["c"]
    inputs = (2 * w["L"] * w["D"] + w["R"] * w["L"] * w["D"] + 2 * w["L"]) * bh * e
    out = bh * w["R"] * w["L"] * w["D"] * n * e
    den = bh * w["R"] * w["L"] * n
    return inputs + out + den * e, (0 if w["fwd_only"] else 2 * inputs + out + den * 4)


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            text, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            text = ""
        sm, mx, reasons = [], [], set()
        for line in text.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def make_device_inputs(w, seed, device):
    from universal_attention_triton_b200 import ops  # noqa: F401  (import check: fails loudly without the library)
    dt = torch.bfloat16 if w["dtype"] == "bf16" else torch.float32
    g = torch.Generator(device="cpu").manual_seed(seed)
    B, H, R, L, c, D = w["B"], w["H"], w["R"], w["L"], w["c"], w["D"]
    n = L // c
    xq = (torch.randn(B, H, R, L, D, generator=g) * w["std"]).to(dt)
    kc = (torch.randn(B, H, n, c, D, generator=g) * w["std"]).to(dt)
    vc = (torch.randn(B, H, n, c, D, generator=g) * w["std"]).to(dt)
    ss = (torch.randn(B, H, n, c, generator=g) * w["gs"] + w["gm"]).sigmoid().to(dt)
    sd = (torch.randn(B, H, L, generator=g) * w["gs"] + w["gm"]).sigmoid().to(dt)
    host = [t.pin_memory() for t in (kc, vc, xq, ss, sd)]
    dev = [t.to(device) for t in host]
    return host, dev


def _load_reference_module():
    """The reference's own ``universal_attention_autograd`` module when a checkout is named by the environment variable
    UA_REF_PATH (the GPU box has none: the port is timed there), loaded by file path so that it cannot be confused with
    this repository's module of the same name."""
    ref = os.environ.get("UA_REF_PATH")
    path = os.path.join(ref, "universal_attention_autograd.py") if ref else None
    if not path or not os.path.exists(path):
        return None
    import importlib.util
    spec = importlib.util.spec_from_file_location("_reference_universal_attention_autograd", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def cpu_reference_step_time(w, steps, warmup, unit_budget_s=25.0):
    """Times the reference's CPU path (fp32) on ONE (batch, kv-head) unit of the workload, driver flow of main.py:55-62:
    the reference module itself when a checkout is available (kind "reference"), else the oracle port (kind "port").
    Returns (tokens/s, seconds per unit, sample description, kind)."""
    from oracle import ua_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    ref = _load_reference_module()
    L = w["L"]
    scale = 1.0
    while L > 4096:          # keep the L x L plane in host memory; extrapolate with L^2
        L //= 2
        scale *= 4.0
    ins = O.make_inputs(1, 1, w["R"], L, w["c"], w["D"], dtype=torch.float32, seed=0, qkv_std=w["std"],
                        gate_mean=w["gm"], gate_std=w["gs"])
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        if ref is not None:
            xs = [t.clone().requires_grad_(not w["fwd_only"]) for t in ins]
            out, denom = ref.UniversalAttention.apply(*xs)
            merged = ref.SMVecMatMul.apply(out, denom)
            if not w["fwd_only"]:
                merged.pow(2).sum().backward()
        elif w["fwd_only"]:
            O.ua_forward(*ins)
        else:
            O.driver_step(*ins)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
        if sum(times) > unit_budget_s and len(times) >= 1:
            break
    t_unit = statistics.median(times) * scale
    tokens_per_unit = w["L"] / w["H"]            # one (b,h) unit is 1/H of a batch row
    sample = (f"1 of {w['B'] * w['H']} (batch, kv-head) units, R={w['R']} L={L} chunk={w['c']} D={w['D']} fp32, "
              f"op+merge+loss fwd+bwd, median of {len(times)}" + (f", time scaled x{scale:g} to L={w['L']}" if scale > 1 else ""))
    return tokens_per_unit / t_unit, t_unit, sample, ("reference" if ref is not None else "port")


def run_reference(args, w, rank):
    if rank != 0:
        return
    val, t_unit, sample, kind = cpu_reference_step_time(w, max(1, args.steps), max(0, min(args.warmup, 1)))
    cores = os.cpu_count() or 1
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_unit * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, **{k: w[k] for k in ("B", "H", "R", "L", "c", "D")}},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def sp_leg(w, device, rank, world, group, W, K, zigzag):
    """One long sequence, rows sharded over the ranks of ``group`` (strong scaling): sp_forward + sp_backward, K timed
    steps after W warm-up steps; returns ms per step (max over the ranks).  Contiguous blocks, or zig-zag (rank g owns
    blocks g and 2G-1-g, which balances the causal work)."""
    import torch.distributed as dist
    from universal_attention_triton_b200 import ops
    from universal_attention_triton_b200.sequence_parallel import owned_blocks, sp_backward, sp_forward
    B, H, R, L, c, D = w["B"], w["H"], w["R"], w["L"], w["c"], w["D"]
    n = L // c
    L_l = L // world
    _, dev = make_device_inputs(w, seed=0, device=device)          # same full inputs on every rank, then sliced
    kc, vc, xq, ss, sd = dev
    P, mine = owned_blocks(world, rank, zigzag)
    nb = n // P                                                   # key chunks per block
    cat_n = lambda t: torch.cat([t[:, :, p * nb:(p + 1) * nb] for p in mine], dim=2).contiguous()
    loc = [cat_n(kc), cat_n(vc), torch.cat([xq[:, :, :, p * nb * c:(p + 1) * nb * c] for p in mine], dim=3).contiguous(),
           cat_n(ss), torch.cat([sd[:, :, p * nb * c:(p + 1) * nb * c] for p in mine], dim=2).contiguous()]
    del dev, kc, vc, xq, ss, sd
    gen = torch.Generator(device=device).manual_seed(99 + rank)
    g_out_cm = torch.randn(B, H, n, R, L_l, D, generator=gen, device=device, dtype=torch.bfloat16)
    g_lse_cm = torch.randn(B, H, n, R, L_l, generator=gen, device=device)
    g_out, g_den = ops.as_reference_out(g_out_cm), ops.as_reference_denom(g_lse_cm)

    def step():
        out, denom, lse, ctx = sp_forward(*loc, group=group, zigzag=zigzag, return_ctx=True)
        return sp_backward(*loc, g_out, g_den, group=group, zigzag=zigzag, ctx=ctx)

    for _ in range(W):
        step()
    dist.barrier(group=group); torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(K):
        step()
    b.record()
    dist.barrier(group=group); torch.cuda.synchronize()
    tt = torch.tensor([a.elapsed_time(b)], device=device, dtype=torch.float64)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX, group=group)
    del loc, g_out_cm, g_lse_cm, g_out, g_den
    torch.cuda.empty_cache()
    return tt.item() / K


SP_COLLECTIVES = ("forward: 1 all-gather (K | V | src, byte-packed) + 1 all-gather of the per-key decay totals; backward: 1 all-gather "
                  "of the per-key dC totals + 1 reduce-scatter (dK | dV | dsrc, fp32); NCCL")


def sequence_parallel_report(w, device, rank, world, W, K, zigzag):
    """The sequence-sharded leg at ``world`` ranks plus, for the ratio, the same sequence on rank 0 alone."""
    import torch.distributed as dist
    solo = dist.new_group([0])                                     # every rank takes part in creating it
    ms = sp_leg(w, device, rank, world, None, W, K, zigzag)
    ms_1 = None
    if world > 1:
        if rank == 0:
            ms_1 = sp_leg(w, device, 0, 1, solo, 1, max(1, min(K, 2)), False)
        dist.barrier()
    B, L = w["B"], w["L"]
    rep = {"workload": f"one sequence B={B} H_kv={w['H']} R={w['R']} L={L} chunk={w['c']} D={w['D']} bf16 fwd+bwd, rows sharded "
                       f"{'zig-zag' if zigzag else 'contiguously'} over {world} rank(s), random upstream grads, masked-block grads included",
           "scaling": "strong", "ms_per_step": ms, "tokens_per_s": B * L / (ms * 1e-3), "collectives": SP_COLLECTIVES}
    if ms_1 is not None:
        rep["ms_per_step_1gpu"] = ms_1
        rep["speedup_vs_1gpu"] = ms_1 / ms
    return rep


def run_sequence_parallel(args, w, rank, world, device, W, K):
    """``--mode sp``: only the sequence-sharded leg, printed as a line of its own."""
    import torch.distributed as dist
    if world == 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=device)
    sampler = ClockSampler(device.index)
    if rank == 0:
        sampler.start()
    rep = sequence_parallel_report(w, device, rank, world, W, K, args.zigzag)
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        B, L = w["B"], w["L"]
        ms = rep["ms_per_step"]
        f_fwd, f_bwd = flops(w)
        peaks, src = load_peaks()
        line = {"metric": METRIC, "value": B * L / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": w["dtype"],
                "data": "synthetic",
                "config": {"workload": f"{args.workload}: " + rep["workload"], "global_batch": B, "seq_len": L,
                           "parallelism": f"sequence-chunk x{world}: " + SP_COLLECTIVES, "l2_policy": "working set exceeds L2"},
                "tflops": (f_fwd + f_bwd) / (ms * 1e-3) / 1e12,
                "frac_of_bf16_peak": (f_fwd + f_bwd) / (ms * 1e-3) / 1e12 / (peaks["bf16_tflops_sustained"] * world),
                "sequence_parallel": rep, "clocks": clocks, "peak_source": src}
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--zigzag", action="store_true", help="with --mode sp: balanced block assignment")
    ap.add_argument("--e2e-loss-only", action="store_true",
                    help="end-to-end leg: return only the loss to the host (default: the loss and the five gradients); "
                         "the default run reports both variants")
    ap.add_argument("--merged-entry", default=None, choices=["composed", "fused", "low_memory"],
                    help="end-to-end leg through UniversalAttentionMerged (the additional one-call entry point, with the "
                         "given backward) instead of the drop-in pair UniversalAttention + SMVecMatMul")
    ap.add_argument("--skip-masked-grads", action="store_true",
                    help="device-resident step without the gradient through fully masked blocks (valid when SMVecMatMul is upstream)")
    ap.add_argument("--mode", default="bh", choices=["bh", "sp"],
                    help="bh: every rank runs its own batch shard (default); sp: ONE long sequence sharded by rows over "
                         "the ranks with NCCL exchange of keys and decay carries (use --workload long)")
    ap.add_argument("--no-scaling-legs", action="store_true",
                    help="N > 1: skip the strong-scaling and sequence-sharded legs that follow the headline")
    ap.add_argument("--profile", action="store_true",
                    help="profiler capture run: honour --warmup below 3; the printed numbers are not bench values")
    args = ap.parse_args()
    w = dict(WORKLOADS[args.workload])

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world == 1:
        # convenience: re-launch under torchrun
        port = os.environ.get("MASTER_PORT", "29531")
        os.execvp(sys.executable, [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                                   f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1", "--master-port", port,
                                   os.path.abspath(__file__)] + sys.argv[1:])

    if args.impl == "reference":
        run_reference(args, w, rank)
        return

    import torch.distributed as dist
    from universal_attention_triton_b200 import (SMVecMatMul, UniversalAttention, UniversalAttentionMerged, _lib, ops,
                                                set_merged_backward, set_strict_masked_grads)
    if args.merged_entry:
        # "low_memory": the two-pass forward that never writes `out`, with the one-kernel backward
        set_merged_backward("fused" if args.merged_entry == "low_memory" else args.merged_entry)
        if args.merged_entry == "low_memory":
            from universal_attention_triton_b200 import set_merged_forward
            set_merged_forward("low_memory")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path for the operator)")
    _lib.load()
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    W, K = (args.warmup if args.profile else max(args.warmup, 3)), max(args.steps, 1)
    if args.mode == "sp":
        run_sequence_parallel(args, w, rank, world, device, W, K)
        return
    host, dev = make_device_inputs(w, seed=rank, device=device)
    kc, vc, xq, ss, sd = dev
    B, H, R, L, c, D = w["B"], w["H"], w["R"], w["L"], w["c"], w["D"]
    n = L // c
    dt = xq.dtype
    f_fwd, f_bwd = flops(w)
    b_fwd, b_bwd = hbm_bytes(w)

    # resident upstream gradients in the library's chunk-major layout
    gen = torch.Generator(device=device).manual_seed(1234 + rank)
    g_out_cm = None if w["fwd_only"] else torch.randn(B, H, n, R, L, D, generator=gen, device=device, dtype=dt)
    g_lse_cm = None if w["fwd_only"] else torch.randn(B, H, n, R, L, generator=gen, device=device, dtype=torch.float32)

    bwd_flags = _lib.FLAG_SKIP_MASKED_GRADS if args.skip_masked_grads else 0
    ev = lambda: torch.cuda.Event(enable_timing=True)
    fwd_ms, bwd_ms = [], []

    def step(record):
        e0, e1, e2 = ev(), ev(), ev()
        e0.record()
        res = ops.forward_cm(kc, vc, xq, ss, sd, keep_carry=not w["fwd_only"])
        out_cm, lse_cm, denom_cm = res[:3]
        carry = res[3] if len(res) > 3 else None
        e1.record()
        if not w["fwd_only"]:
            # (the step holds the forward's output tiles, as an autograd graph does: the backward takes its row term from them)
            grads = ops.backward_cm(kc, vc, xq, ss, sd, g_out_cm, g_lse_cm, flags=bwd_flags, carry=carry, lse=lse_cm, out_cm=out_cm)
        e2.record()
        if record:
            fwd_ms.append((e0, e1)); bwd_ms.append((e1, e2))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(W):
        step(False)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    t_start, t_end = ev(), ev()
    t_start.record()
    for _ in range(K):
        step(True)
    t_end.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = t_start.elapsed_time(t_end)
    if world > 1:
        tt = torch.tensor([total_ms], device=device, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        total_ms = tt.item()
    ms_per_step = total_ms / K
    tokens = B * L * world
    value = tokens / (ms_per_step * 1e-3)
    fwd_avg = statistics.mean(a.elapsed_time(b) for a, b in fwd_ms)
    bwd_avg = statistics.mean(a.elapsed_time(b) for a, b in bwd_ms) if not w["fwd_only"] else 0.0
    # A kernel whose bounded waits ran out returns after seconds with its status word set: such a step is no measurement.
    per_step = [a.elapsed_time(b) + (c_.elapsed_time(d) if not w["fwd_only"] else 0.0) for (a, b), (c_, d) in zip(fwd_ms, bwd_ms)]
    if max(per_step) > 20 * statistics.median(per_step):
        raise RuntimeError(f"a timed step took {max(per_step):.1f} ms against a median of {statistics.median(per_step):.2f} ms")
    os.environ["UA_CHECK_STATUS"] = "1"      # one more, untimed, step that synchronises and reads the status words
    try:
        step(False)
    finally:
        os.environ.pop("UA_CHECK_STATUS", None)

    # ---- end to end through the autograd entry points, host buffers -----------------
    e2e = None
    if not args.no_e2e:
        h2d = sum(t.numel() * t.element_size() for t in host)
        # (default settings: the backward recognises SMVecMatMul's gradients, whose part for the rows before each chunk is
        # exactly zero, and leaves out the kernels of those rows)
        host_grads = [torch.empty_like(t).pin_memory() for t in host]
        host_loss = torch.empty((), dtype=torch.float32).pin_memory()

        # Steps are pipelined over three streams, as a training loop with a prefetching loader runs them: while step k
        # computes, the inputs of step k+1 travel to the device and the results of step k-1 travel back.  Every step's
        # copies (pinned host memory both ways) lie inside the timed region; two sets of device input buffers.
        s_in, s_out, s_cmp = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
        dev_in = [[torch.empty_like(t, device=device) for t in host] for _ in range(2)]
        in_ready = [None, None]
        cmp_done = [None, None]

        grads_to_host = False      # set per variant below

        def upload(k):
            b = k & 1
            with torch.cuda.stream(s_in):
                if cmp_done[b] is not None:
                    s_in.wait_event(cmp_done[b])          # the step that used this buffer set has finished its backward
                for d, h in zip(dev_in[b], host):
                    d.copy_(h, non_blocking=True)
                in_ready[b] = s_in.record_event()

        def e2e_step(k, last):
            b = k & 1
            s_cmp.wait_event(in_ready[b])
            if not last:
                upload(k + 1)
            if w["fwd_only"]:
                with torch.no_grad():
                    out, denom = UniversalAttention.apply(*dev_in[b])
                    merged = SMVecMatMul.apply(out, denom)
                    loss = merged.pow(2).sum()
                grads = []
            else:
                xs = [t.detach().requires_grad_() for t in dev_in[b]]
                if args.merged_entry:
                    merged = UniversalAttentionMerged.apply(*xs)
                else:
                    out, denom = UniversalAttention.apply(*xs)
                    merged = SMVecMatMul.apply(out, denom)
                loss = merged.pow(2).sum()
                loss.backward()
                grads = [x.grad for x in xs]
                loss = loss.detach()
            cmp_done[b] = s_cmp.record_event()
            with torch.cuda.stream(s_out):
                s_out.wait_event(cmp_done[b])
                host_loss.copy_(loss, non_blocking=True)
                loss.record_stream(s_out)
                for hg, g in zip(host_grads, grads if grads_to_host else []):
                    hg.copy_(g, non_blocking=True)
                    g.record_stream(s_out)

        def e2e_run(nsteps):
            upload(0)
            for k in range(nsteps):
                e2e_step(k, k == nsteps - 1)
            s_cmp.wait_stream(s_out)
            s_cmp.wait_stream(s_in)

        def e2e_timed():
            nonlocal cmp_done
            # warm-up: as many steps as the device-resident leg, and at least four: the pipelined pattern (buffers held
            # across streams until their copies have run) needs a few steps before the caching allocator stops growing,
            # and a cudaMalloc inside the timed region would be timed as a step
            e2e_run(max(W, 4))
            cmp_done = [None, None]
            barrier()
            a, b = ev(), ev()
            a.record()
            e2e_run(K)
            b.record()
            barrier()
            ms = a.elapsed_time(b)
            if world > 1:
                tt = torch.tensor([ms], device=device, dtype=torch.float64)
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                ms = tt.item()
            return ms

        # The step's result is the loss AND the five gradients (what the CPU arm leaves in host memory): both come back
        # by default.  The loss-only variant (gradients stay on the device, as a fused optimizer would use them) is timed
        # beside it.
        loss_only_ms = e2e_timed()
        grads_to_host = not w["fwd_only"] and not args.e2e_loss_only
        e_ms = e2e_timed() if grads_to_host else loss_only_ms
        d2h = 4 + (h2d if grads_to_host else 0)

        # The host link of this box, measured alone on the largest buffer (pinned memory both ways, nothing else running):
        # on some hosts of the pool device-to-host copies run far below the link's rate, and the figure with the gradients
        # returned is then bound by them -- the loss-only figure beside it is not.
        def link_gbs(dst, src):
            for _ in range(2):
                dst.copy_(src, non_blocking=True)
            torch.cuda.synchronize()
            a, b = ev(), ev()
            a.record()
            for _ in range(3):
                dst.copy_(src, non_blocking=True)
            b.record()
            torch.cuda.synchronize()
            return 3 * src.numel() * src.element_size() / (a.elapsed_time(b) * 1e-3) / 1e9
        big = max(range(len(host)), key=lambda i: host[i].numel())
        host_link = {"h2d_gbs": link_gbs(dev_in[0][big], host[big]), "d2h_gbs": link_gbs(host_grads[big], dev_in[0][big]),
                     "buffer_bytes": host[big].numel() * host[big].element_size()}
        e2e = {"value": tokens / (e_ms / K * 1e-3), "unit": "tokens/s", "ms_per_step": e_ms / K,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "host_link": host_link,
               "returns": "loss + five gradients" if grads_to_host else "loss",
               "loss_only": {"value": tokens / (loss_only_ms / K * 1e-3), "ms_per_step": loss_only_ms / K, "d2h_bytes_per_step": 4},
               "path": (f"UniversalAttentionMerged.apply ({args.merged_entry} backward)" if args.merged_entry else "UniversalAttention.apply -> SMVecMatMul.apply") +
                       " -> pow(2).sum() -> backward (main.py:55-62 flow); "
                       "copies of neighbouring steps overlap the compute (three streams)"}

    # ---- multi-GPU legs beside the (unchanged) headline: the SAME 32 (batch, kv-head) units of the workload split over the
    # ranks (strong scaling, no collective), and one long sequence sharded by rows (NCCL exchange of keys and decay carries)
    strong = None
    seqpar = None
    if world > 1 and not args.no_scaling_legs and not w["fwd_only"]:
        BH = B * H
        if BH % world == 0:
            per = BH // world
            lo = rank * per
            flat = lambda t: t.reshape((1, BH) + tuple(t.shape[2:]))[:, lo:lo + per].contiguous()
            skc, svc, sxq, sss, ssd = (flat(t) for t in (kc, vc, xq, ss, sd))
            sgo, sgl = flat(g_out_cm), flat(g_lse_cm)

            def strong_step():
                res = ops.forward_cm(skc, svc, sxq, sss, ssd, keep_carry=True)
                ops.backward_cm(skc, svc, sxq, sss, ssd, sgo, sgl, flags=bwd_flags, carry=res[3], lse=res[1], out_cm=res[0])

            for _ in range(3):
                strong_step()
            barrier()
            a, b = ev(), ev()
            a.record()
            for _ in range(K):
                strong_step()
            b.record()
            barrier()
            tt = torch.tensor([a.elapsed_time(b)], device=device, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            s_ms = tt.item() / K
            strong = {"workload": f"{args.workload}: the {BH} (batch, kv-head) units of ONE batch B={B} split over {world} ranks "
                                  f"({per} units each), no collective", "scaling": "strong", "ms_per_step": s_ms,
                      "tokens_per_s": B * L / (s_ms * 1e-3), "ms_per_step_1gpu": ms_per_step,
                      "speedup_vs_1gpu": ms_per_step / s_ms}
            del skc, svc, sxq, sss, ssd, sgo, sgl
        del kc, vc, xq, ss, sd, dev, g_out_cm, g_lse_cm
        torch.cuda.empty_cache()
        seqpar = sequence_parallel_report(dict(WORKLOADS["long"]), device, rank, world, 1, 3, True)

    if rank == 0:
        peaks, peak_src = load_peaks()
        dom_is_bwd = bwd_avg >= fwd_avg
        dom_f, dom_ms = (f_bwd, bwd_avg) if dom_is_bwd else (f_fwd, fwd_avg)
        achieved = dom_f / (dom_ms * 1e-3) / 1e12
        # The denominator is the burst figure unless this run itself was in the power-limited regime the sustained figure
        # was measured in: a timed region of seconds, or SM clocks sampled well below their maximum.
        sustained_regime = total_ms >= 2000.0 or bool(clocks and clocks.get("sm_mhz") and clocks.get("sm_max_mhz")
                                                     and clocks["sm_mhz"] < 0.9 * clocks["sm_max_mhz"])
        peak_key = "bf16_tflops_sustained" if sustained_regime else "bf16_tflops"
        peak = peaks[peak_key]
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": w["dtype"], "data": "synthetic",
            "config": {"workload": f"{args.workload}: B={B} (per GPU) H_kv={H} R={R} L={L} chunk={c} D={D} {w['dtype']} "
                                   f"fwd{'' if w['fwd_only'] else '+bwd'}, random upstream grads, masked-block grads {'skipped' if args.skip_masked_grads else 'included'}",
                       "global_batch": B * world, "seq_len": L, "parallelism": f"batch-shard x{world}, no collective",
                       "l2_policy": "working set (out + g_out > 4 GB) exceeds the 126 MB L2; no explicit flush"},
            "tflops": (f_fwd + f_bwd) * world / (ms_per_step * 1e-3) / 1e12,
            "frac_of_bf16_peak": (f_fwd + f_bwd) / (ms_per_step * 1e-3) / 1e12 / peak,
            "fwd_ms": fwd_avg, "bwd_ms": bwd_avg,
            # forward kernel; backward: keys-on-lanes kernel, its row-side finish, three fp32 -> dtype conversions, and with the
            # gradient through the rows before each chunk three more (per-chunk constants, sweep, per-chunk finish)
            "gpu_launches": K * (1 + (0 if w["fwd_only"] else (5 if args.skip_masked_grads else 8))),
            "clocks": clocks,
            "roofline": {"kernel": "ua backward" if dom_is_bwd else "ua forward", "bound": "tensor",
                         "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "traffic": NCU_DRAM_BYTES.get(args.workload, {}).get("bwd" if dom_is_bwd else "fwd"),
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of a 2-of-32 (batch, kv-head) slice, "
                                           "scaled by the units of a full launch",
                         "peak_source": f"{peak_src} ({peak_key}: timed region {total_ms / 1e3:.2f} s, median SM clock "
                                        f"{clocks.get('sm_mhz') if clocks else None} MHz)",
                         "algorithmic_flops_per_launch": dom_f,
                         "hbm_view": {"bytes": b_bwd if dom_is_bwd else b_fwd,
                                      "achieved_gbs": (b_bwd if dom_is_bwd else b_fwd) / (dom_ms * 1e-3) / 1e9,
                                      "peak_gbs": peaks["hbm_gbs"]}},
            "e2e": e2e,
        }
        if strong is not None:
            line["strong"] = strong
        if seqpar is not None:
            line["sequence_parallel"] = seqpar
        if not w["fwd_only"]:       # the other kernel of the step, same arithmetic
            o_f, o_ms = (f_fwd, fwd_avg) if dom_is_bwd else (f_bwd, bwd_avg)
            line["roofline_other_kernel"] = {"kernel": "ua forward" if dom_is_bwd else "ua backward", "bound": "tensor",
                                             "achieved": o_f / (o_ms * 1e-3) / 1e12, "peak": peak, "unit": "TFLOP/s",
                                             "frac": o_f / (o_ms * 1e-3) / 1e12 / peak,
                                             "traffic": NCU_DRAM_BYTES.get(args.workload, {}).get("fwd" if dom_is_bwd else "bwd")}
        if not args.no_cpu_baseline and world == 1:
            val, t_unit, sample, kind = cpu_reference_step_time(w, 2, 1)
            line["cpu_baseline"] = {"value": val, "unit": "tokens/s", "cores": os.cpu_count() or 1, "kind": kind,
                                    "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""Generate the golden vectors under tests/golden/ by running the UNMODIFIED
reference implementation (pure-PyTorch, CPU, fp32).

Usage (only where a checkout of the reference is available):

    UA_REF_PATH=/path/to/Universal_Attention_triton python tests/golden/make_golden.py

The reference is imported, never copied.  Each ``.npz`` stores the inputs next
to the reference's outputs so that the tests need neither the reference nor a
particular random-number generator.  Functions exercised:

* ``universal_attention_autograd.UniversalAttention``   (1-D signature)
* ``universal_attention_autograd.UniversalAttention2``  (2-D signature, c_ != _c too)
* ``universal_attention_autograd.SMVecMatMul`` and the driver loss of ``main.py:55-62``
"""
import os
import sys

import numpy as np
import torch

REF = os.environ.get("UA_REF_PATH") or (sys.argv[1] if len(sys.argv) > 1 else None)
if not REF or not os.path.isdir(REF):
    sys.exit("set UA_REF_PATH (or pass as first argument) to a checkout of the reference implementation")
sys.path.insert(0, REF)
from universal_attention_autograd import SMVecMatMul, UniversalAttention, UniversalAttention2  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def draw(B, H, R, L, c, D, seed, gate_mean=0.0, gate_std=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    n = L // c
    xq = torch.randn(B, H, R, L, D, generator=g)
    kc = torch.randn(B, H, n, c, D, generator=g)
    vc = torch.randn(B, H, n, c, D, generator=g)
    ss = (torch.randn(B, H, n, c, generator=g) * gate_std + gate_mean).sigmoid()
    sd = (torch.randn(B, H, L, generator=g) * gate_std + gate_mean).sigmoid()
    return kc, vc, xq, ss, sd


def run_random_upstream(name, fn, ins, seed):
    """Forward + backward with random upstream gradients (as the reference's own
    kernel test does, universal_attention_kernel.py:1261-1262): exercises the
    gradient that flows through fully masked blocks."""
    ins = [t.clone().requires_grad_() for t in ins]
    out, denom = fn(*ins)
    g = torch.Generator(device="cpu").manual_seed(seed + 1000)
    g_out = torch.randn(out.shape, generator=g)
    g_denom = torch.randn(denom.shape, generator=g)
    torch.autograd.backward([out, denom], [g_out, g_denom])
    d = dict(kc=ins[0], vc=ins[1], xq=ins[2], static_src=ins[3], static_dest=ins[4],
             out=out, denom=denom, g_out=g_out, g_denom=g_denom,
             dkc=ins[0].grad, dvc=ins[1].grad, dxq=ins[2].grad, dsrc=ins[3].grad, ddest=ins[4].grad)
    np.savez_compressed(os.path.join(HERE, name + ".npz"),
                        **{k: v.detach().numpy() for k, v in d.items()})
    print(name, "out", tuple(out.shape), "saved")


def run_driver(name, fn, ins, row_stride):
    """The driver flow of main.py:55-62: op -> SMVecMatMul -> pow(2).sum() -> backward."""
    ins = [t.clone().requires_grad_() for t in ins]
    out, denom = fn(*ins)
    merged = SMVecMatMul.apply(out, denom)
    out.retain_grad()
    denom.retain_grad()
    loss = merged.pow(2).sum()
    loss.backward()
    d = dict(kc=ins[0], vc=ins[1], xq=ins[2], static_src=ins[3], static_dest=ins[4],
             out_rows=out[:, :, :, ::row_stride], denom=denom, merged=merged, loss=loss,
             g_out_rows=out.grad[:, :, :, ::row_stride], g_denom=denom.grad,
             dkc=ins[0].grad, dvc=ins[1].grad, dxq=ins[2].grad, dsrc=ins[3].grad, ddest=ins[4].grad,
             row_stride=torch.tensor(row_stride))
    np.savez_compressed(os.path.join(HERE, name + ".npz"),
                        **{k: v.detach().numpy() for k, v in d.items()})
    print(name, "loss", loss.item(), "saved")


def main():
    torch.set_num_threads(os.cpu_count())
    # 1-D signature, tiny, random upstream gradients
    kc, vc, xq, ss, sd = draw(1, 2, 2, 64, 16, 16, seed=11)
    run_random_upstream("tiny_1d_random_upstream", UniversalAttention.apply, (kc, vc, xq, ss, sd), 11)
    # 2-D signature with key chunk 16 and row chunk 32 (c_ != _c)
    kc, vc, xq, ss, sd = draw(2, 1, 3, 64, 16, 8, seed=12)
    xq2 = xq.view(2, 1, 3, 2, 32, 8)
    sd2 = sd.view(2, 1, 2, 32)
    run_random_upstream("tiny_2d_random_upstream", UniversalAttention2.apply, (kc, vc, xq2, ss, sd2), 12)
    # strongly pruning gates (logit mean -4, std 2), 2-D signature
    kc, vc, xq, ss, sd = draw(1, 1, 1, 128, 32, 16, seed=13, gate_mean=-4.0, gate_std=2.0)
    run_random_upstream("tiny_2d_pruning_gates", UniversalAttention2.apply,
                        (kc, vc, xq.view(1, 1, 1, 4, 32, 16), ss, sd.view(1, 1, 4, 32)), 13)
    # config "CPU plumbing": fp32, B=1, H_kv=2, R=2, L=256, chunk=64, D=64, seed 0, driver flow
    kc, vc, xq, ss, sd = draw(1, 2, 2, 256, 64, 64, seed=0)
    run_driver("plumbing_1d_driver", UniversalAttention.apply, (kc, vc, xq, ss, sd), 8)
    run_driver("plumbing_2d_driver", UniversalAttention2.apply,
               (kc, vc, xq.view(1, 2, 2, 4, 64, 64), ss, sd.view(1, 2, 4, 64)), 8)


if __name__ == "__main__":
    main()

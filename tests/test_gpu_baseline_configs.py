"""Parity at the shapes and input distributions of the BASELINE configurations, one (batch, kv-head) unit each,
against the CPU oracle (never against another kernel of this library).

Bars as the task states them: bf16 forward max-abs <= 2e-2, gradients <= 5e-2 relative-Frobenius, both against the
fp32 oracle fed the same bf16-rounded values.  At these lengths the fp32 oracle carries rounding noise of its own
(its fp32 cumulative sum reaches -2e4 at L = 4096 where fp32 spacing is 2e-3; the derivative of log1p(-a) reaches
1e6 next to the clamp): every test measures that noise ON THE SAME INPUTS AND METRIC as the difference between the
oracle in fp32 and in fp64, and the bound that is asserted is

    kernel_error <= max(stated bar, K_NOISE * oracle_noise)          with K_NOISE = 2,

so a bound above the stated bar is only ever granted where the reference arithmetic itself is that uncertain, and
the figures are printed (run pytest with -s to see them).  The checks live in ``tests/_util.py``.
"""
import pytest
import torch

from oracle import ua_oracle as O
from tests._util import check_backward as _bwd_check, check_forward as _fwd_check, rel_fro

pytestmark = pytest.mark.gpu

GRADS = ["dkc", "dvc", "dxq", "dsrc", "ddest"]


def _case(shape, seed, **kw):
    ins = O.make_inputs(*shape, dtype=torch.bfloat16, seed=seed, **kw)
    return ins, [t.float() for t in ins]


def _upstream(shape, seed):
    B, H, R, L, c, D = shape
    n = L // c
    gen = torch.Generator().manual_seed(seed)
    g_out = torch.randn(B, H, R, L, D, n, generator=gen).bfloat16()
    g_den = torch.randn(B, H, R, L, n, generator=gen)
    return g_out, g_den


def _run(shape, ins, g_out, g_den):
    """forward + backward through the chunk-major entry points (what the autograd Functions call)."""
    from universal_attention_triton_b200 import ops
    cu = [t.cuda() for t in ins]
    out_cm, lse_cm, _, carry = ops.forward_cm(*cu, keep_carry=True)
    out = ops.as_reference_out(out_cm).float().cpu()
    lse = ops.as_reference_denom(lse_cm).cpu()
    grads = None
    if g_out is not None:
        grads = ops.backward_cm(*cu, ops.out_to_chunk_major(g_out.cuda()), ops.denom_to_chunk_major(g_den.cuda()),
                                carry=carry, lse=lse_cm)
    return out, lse, grads


def test_config2_unit_forward_and_backward_r4():
    """BASELINE config 2: bf16, R = 4, L = 4096, chunk 128, D = 64, q/k/v and gate logits N(0,1); random upstream
    gradients, masked-block gradients included."""
    shape = (1, 1, 4, 4096, 128, 64)
    ins, ins32 = _case(shape, seed=0)
    g_out, g_den = _upstream(shape, seed=4)
    out, lse, grads = _run(shape, ins, g_out, g_den)
    _fwd_check("C2", out, lse, ins32, 128)
    _bwd_check("C2", grads, ins32, g_out.float(), g_den)


def test_config3_unit_forward():
    """BASELINE config 3 (prefill, forward only): bf16, R = 4, L = 8192, chunk 128, D = 128, q/k/v N(0, std 0.5)."""
    shape = (1, 1, 4, 8192, 128, 128)
    ins, ins32 = _case(shape, seed=0, qkv_std=0.5)
    out, lse, _ = _run(shape, ins, None, None)
    _fwd_check("C3", out, lse, ins32, 128)


@pytest.mark.parametrize("L", [4096])
def test_config5_unit_forward_and_backward(L):
    """BASELINE config 5 (numerics stress): bf16, R = 1, chunk 128, D = 128, gate logits N(-4, std 2)."""
    shape = (1, 1, 1, L, 128, 128)
    ins, ins32 = _case(shape, seed=0, gate_mean=-4.0, gate_std=2.0)
    g_out, g_den = _upstream(shape, seed=6)
    out, lse, grads = _run(shape, ins, g_out, g_den)
    _fwd_check("C5", out, lse, ins32, 128)
    _bwd_check("C5", grads, ins32, g_out.float(), g_den)


def test_config4_tile_shape_forward_and_backward():
    """BASELINE config 4's tile: chunk 256, D = 128, R = 2 at L = 2048."""
    shape = (1, 1, 2, 2048, 256, 128)
    ins, ins32 = _case(shape, seed=0)
    g_out, g_den = _upstream(shape, seed=8)
    out, lse, grads = _run(shape, ins, g_out, g_den)
    _fwd_check("C4-tile", out, lse, ins32, 256)
    _bwd_check("C4-tile", grads, ins32, g_out.float(), g_den)


def test_kernel_backed_function_in_the_driver_flow_bf16():
    """Universal_Attention.universal_attention.UniversalAttention (2-D signature) in the reference driver's flow
    (main.py:55-62): the merged output within 2e-2 and all five gradients within 5e-2 of the fp32 oracle, in both
    masked-gradient modes (they must agree: those gradients are exactly zero under SMVecMatMul).  In strict mode the backward
    recognises SMVecMatMul's gradients (a note on the tensors) and leaves out the kernels of the rows before each chunk; a
    third run hides the note behind tensor hooks, so that those kernels do run, on the zeros: same result."""
    import universal_attention_triton_b200 as ua
    from Universal_Attention.universal_attention import UniversalAttention as KUA
    B, H, R, L, c, D = 1, 2, 2, 1024, 128, 64
    ins, ins32 = _case((B, H, R, L, c, D), seed=9)
    ins2d = [ins[0], ins[1], ins[2].view(B, H, R, L // c, c, D), ins[3], ins[4].view(B, H, L // c, c)]
    # the reference's flow merges with the bf16 denom; the oracle is given the same rounding of denom
    out_ref, _, lse_ref = O.ua_forward(*ins32)
    den_bf = lse_ref.bfloat16().float()
    merged_ref = O.merge_forward(out_ref.float(), den_bf)
    d_mat, d_vec = O.merge_backward(out_ref.float(), den_bf, 2 * merged_ref)
    grads_ref = O.ua_backward(*ins32, d_mat.bfloat16().float(), d_vec)
    results = []
    try:
        for strict, hide_note in ((True, False), (False, False), (True, True)):
            ua.set_strict_masked_grads(strict)
            xs = [t.cuda().clone().requires_grad_() for t in ins2d]
            out, denom = KUA.apply(*xs)
            assert out.shape == (B, H, R, L, D, L // c) and denom.shape == (B, H, R, L, L // c)
            assert out.dtype == torch.bfloat16 and denom.dtype == torch.bfloat16
            if hide_note:
                out.register_hook(lambda g: g.clone())
                denom.register_hook(lambda g: g.clone())
            merged = ua.SMVecMatMul.apply(out, denom)
            merged.float().pow(2).sum().backward()
            results.append((merged.float().cpu(), [t.grad.float().cpu() for t in xs]))
    finally:
        ua.set_strict_masked_grads(True)
    for (m, grads) in results:
        assert (m - merged_ref).abs().max().item() <= 2e-2
        for got, ref, key in zip(grads, grads_ref, GRADS):
            e = rel_fro(got.reshape(-1), ref.reshape(-1))
            assert e <= 5e-2, (key, e)
    for other in (1, 2):
        for a, b in zip(results[0][1], results[other][1]):
            assert torch.equal(a, b) or rel_fro(a, b) < 1e-3

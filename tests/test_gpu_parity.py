"""GPU parity tests: the CUDA library (through its C ABI) against the golden
vectors of the reference and against the CPU oracle on seeded inputs.

Tolerances (stated by the task): fp32 mode forward max-abs <= 1e-4 and grads
<= 1e-4 relative-Frobenius; bf16 mode forward max-abs <= 2e-2 and grads <= 5e-2
relative-Frobenius, both against the fp32 reference fed the same (bf16-rounded)
values."""
import pytest
import torch

from oracle import ua_oracle as O
from tests._util import check_backward, check_forward, fwd_errors, load_golden, rel_fro

pytestmark = pytest.mark.gpu

GRADS = ["dkc", "dvc", "dxq", "dsrc", "ddest"]


def _ua():
    import universal_attention_triton_b200 as ua
    return ua


def _cuda(*ts):
    return [t.cuda() for t in ts]


def _run_op(fn, ins, g_out, g_denom):
    ins = [t.clone().requires_grad_() for t in ins]
    out, denom = fn(*ins)
    torch.autograd.backward([out, denom], [g_out, g_denom])
    return out, denom, [t.grad for t in ins]


@pytest.mark.parametrize("name,fn", [("tiny_1d_random_upstream", "UniversalAttention"),
                                     ("tiny_2d_random_upstream", "UniversalAttention2"),
                                     ("tiny_2d_pruning_gates", "UniversalAttention2")])
def test_fp32_golden_random_upstream(name, fn):
    g = load_golden(name)
    ua = _ua()
    ins = _cuda(g["kc"], g["vc"], g["xq"], g["static_src"], g["static_dest"])
    out, denom, grads = _run_op(getattr(ua, fn).apply, ins, g["g_out"].cuda(), g["g_denom"].cuda())
    assert out.shape == g["out"].shape and denom.shape == g["denom"].shape
    assert out.dtype == torch.float32 and denom.dtype == torch.float32
    e = fwd_errors(out.cpu(), denom.cpu(), g["out"], g["denom"], g["kc"].shape[3])
    assert e["out_valid"] <= 1e-4 and e["out_masked"] <= 1e-6 and e["masked_denom_ok"], e
    assert e["denom_valid"] <= 1e-3, e          # |denom| reaches 1e3 here: 1e-3 is ~4 fp32 ulp
    for got, key in zip(grads, GRADS):
        assert got.shape == g[key].shape and got.dtype == g[key].dtype
        assert rel_fro(got.cpu(), g[key]) <= 1e-4, (key, rel_fro(got.cpu(), g[key]))


@pytest.mark.parametrize("name,fn", [("plumbing_1d_driver", "UniversalAttention"),
                                     ("plumbing_2d_driver", "UniversalAttention2")])
def test_fp32_golden_driver_flow(name, fn):
    """BASELINE config 1 (fp32 B1 H2 R2 L256 c64 D64) through op -> SMVecMatMul -> pow(2).sum()."""
    g = load_golden(name)
    ua = _ua()
    ins = [t.clone().requires_grad_() for t in _cuda(g["kc"], g["vc"], g["xq"], g["static_src"], g["static_dest"])]
    out, denom = getattr(ua, fn).apply(*ins)
    merged = ua.SMVecMatMul.apply(out, denom)
    loss = merged.pow(2).sum()
    loss.backward()
    rs = int(g["row_stride"])
    assert (merged.cpu() - g["merged"]).abs().max() <= 1e-4
    assert abs(loss.item() - g["loss"].item()) / g["loss"].item() <= 1e-5
    assert (out.cpu()[:, :, :, ::rs] - g["out_rows"]).abs().max() <= 2e-3   # far chunks: oracle 1-D vs 2-D differ by 2.5e-4
    for t, key in zip(ins, GRADS):
        assert rel_fro(t.grad.cpu(), g[key]) <= 1e-4, (key, rel_fro(t.grad.cpu(), g[key]))


def _bf16_case(B, H, R, L, c, D, seed, **kw):
    ins = O.make_inputs(B, H, R, L, c, D, dtype=torch.bfloat16, seed=seed, **kw)
    ins32 = [t.float() for t in ins]
    return ins, ins32


@pytest.mark.parametrize("shape", [(1, 2, 2, 512, 128, 64), (2, 1, 4, 256, 64, 64), (1, 1, 1, 512, 128, 128),
                                   (1, 1, 2, 512, 256, 128),       # the chunk-256 / head-dim-128 tile of the long-context config
                                   (1, 2, 2, 1024, 256, 64), (1, 1, 3, 768, 384, 64)])      # chunks of 2 and 3 sub-chunks of 128 keys
def test_bf16_against_oracle(shape):
    B, H, R, L, c, D = shape
    ua = _ua()
    ins, ins32 = _bf16_case(*shape, seed=3)
    gen = torch.Generator().manual_seed(5)
    n = L // c
    g_out = torch.randn(B, H, R, L, D, n, generator=gen).bfloat16()
    g_denom = torch.randn(B, H, R, L, n, generator=gen)
    ref_out, ref_denom, ref_lse = O.ua_forward(*ins32)
    ref_grads = O.ua_backward(*ins32, g_out.float(), g_denom)
    out, denom, grads = _run_op(ua.UniversalAttention.apply, _cuda(*ins), g_out.cuda(), g_denom.cuda())
    assert out.dtype == torch.bfloat16 and denom.dtype == torch.bfloat16
    e = fwd_errors(out.float().cpu(), denom.float().cpu(), ref_out, ref_denom, c)
    assert e["out_masked"] <= 2e-2 and e["masked_denom_ok"], e
    from universal_attention_triton_b200 import ops
    lse32 = ops.as_reference_denom(ops.forward_cm(*_cuda(*ins))[1]).cpu()
    check_forward(f"bf16 {shape}", out.float().cpu(), lse32, ins32, c)      # out <= 2e-2 (noise-pinned), fp32 lse <= 2e-2
    # denom is the fp32 log-sum-exp rounded to bf16: within one bf16 ulp of the reference value
    ulp = ref_denom.abs().clamp_min(1.0) * 2.0 ** -7
    from tests._util import valid_row_mask
    valid = valid_row_mask(L, n, c)
    assert (((denom.float().cpu() - ref_denom).abs() <= ulp) | ~valid).all()
    for got, ref, key in zip(grads, ref_grads, GRADS):
        assert got.dtype == torch.bfloat16
        assert rel_fro(got.float().cpu(), ref) <= 5e-2, (key, rel_fro(got.float().cpu(), ref))


def test_fp32_lse_is_returned_by_the_library():
    from universal_attention_triton_b200 import ops
    ins, ins32 = _bf16_case(1, 1, 2, 256, 64, 64, seed=7)
    _, _, ref_lse = O.ua_forward(*ins32)
    out_cm, lse_cm, denom_cm = ops.forward_cm(*_cuda(*ins))
    lse = ops.as_reference_denom(lse_cm).cpu()
    from tests._util import valid_row_mask
    valid = valid_row_mask(256, 4, 64)
    assert ((lse - ref_lse).abs() * valid).max() <= 2e-2
    assert lse_cm.dtype == torch.float32 and denom_cm.dtype == torch.bfloat16


def test_reference_layout_mode_and_relayout_roundtrip():
    ua = _ua()
    from universal_attention_triton_b200 import ops
    ins, _ = _bf16_case(1, 2, 2, 128, 32, 16, seed=2)
    cu = _cuda(*ins)
    out_v, denom_v = ua.UniversalAttention.apply(*cu)
    ua.set_output_layout("reference")
    try:
        out_c, denom_c = ua.UniversalAttention.apply(*cu)
    finally:
        ua.set_output_layout("chunk_major")
    assert out_c.is_contiguous() and denom_c.is_contiguous()
    assert torch.equal(out_c, out_v) and torch.equal(denom_c, denom_v)
    back = ops.out_to_chunk_major(out_c)
    assert torch.equal(back, out_v.permute(0, 1, 5, 2, 3, 4))


def test_merge_kernels_against_oracle():
    ua = _ua()
    gen = torch.Generator().manual_seed(1)
    mat = torch.randn(1, 2, 2, 64, 16, 4, generator=gen)
    vec = torch.randn(1, 2, 2, 64, 4, generator=gen) * 3
    g = torch.randn(1, 2, 2, 64, 16, generator=gen)
    m = mat.cuda().requires_grad_()
    v = vec.cuda().requires_grad_()
    merged = ua.SMVecMatMul.apply(m, v)
    merged.backward(g.cuda())
    assert (merged.cpu() - O.merge_forward(mat, vec)).abs().max() <= 1e-5
    d_mat, d_vec = O.merge_backward(mat, vec, g)
    assert (m.grad.cpu() - d_mat).abs().max() <= 1e-5
    assert (v.grad.cpu() - d_vec).abs().max() <= 1e-5


@pytest.mark.parametrize("shape", [(1, 2, 4, 1024, 128, 64), (2, 1, 1, 768, 128, 64), (1, 1, 3, 512, 128, 128),
                                   (1, 2, 1, 384, 128, 128)])
def test_tensor_core_forward_matches_simt_forward(shape):
    """The tcgen05 forward against the generic fp32 SIMT forward of the same library, on the device."""
    from universal_attention_triton_b200 import _lib, ops
    B, H, R, L, c, D = shape
    ins, _ = _bf16_case(*shape, seed=21)
    cu = _cuda(*ins)
    out_tc, lse_tc, den_tc = ops.forward_cm(*cu)
    out_sm, lse_sm, den_sm = ops.forward_cm(*cu, flags=_lib.FLAG_FORCE_SIMT)
    n = L // c
    valid = (torch.arange(L).view(1, L) >= torch.arange(n).view(n, 1) * c).cuda()      # (n, L)
    v5 = valid.view(1, 1, n, 1, L)
    assert ((lse_tc - lse_sm).abs() * v5).max().item() <= 2e-2
    assert torch.equal(lse_tc[~v5.expand_as(lse_tc)], lse_sm[~v5.expand_as(lse_sm)])
    err = (out_tc.float() - out_sm.float()).abs()
    bound = 2e-2 + out_sm.float().abs() * 2.0 ** -7
    assert (err <= bound).all(), (err - bound).max().item()


@pytest.mark.parametrize("L", [4096, 8192])
def test_tensor_core_backward_config2_length_against_oracle(L):
    """Backward at the sequence length of BASELINE config 2 (L=4096, chunk 128, D=64; one (b, h) unit, R=2) and at twice
    that against the CPU oracle with random upstream gradients (masked-block gradients included): 5e-2
    relative-Frobenius as the task states, through the plain backward, the one that takes the forward's table and
    log-sum-exp, and the one that also takes the forward's output tiles (row term of the softmax gradient from
    out . g_out); the forward's log-sum-exp along the way."""
    from universal_attention_triton_b200 import ops
    from tests._util import valid_row_mask
    shape = (1, 1, 2, L, 128, 64)
    B, H, R, L, c, D = shape
    n = L // c
    ins, ins32 = _bf16_case(*shape, seed=2)
    gen = torch.Generator().manual_seed(4)
    g_out = torch.randn(B, H, R, L, D, n, generator=gen).bfloat16()
    g_den = torch.randn(B, H, R, L, n, generator=gen)
    cu = _cuda(*ins)
    g_out_cm = ops.out_to_chunk_major(g_out.cuda())
    g_den_cm = ops.denom_to_chunk_major(g_den.cuda())
    out_cm, lse_cm, _, carry = ops.forward_cm(*cu, keep_carry=True)
    _, _, ref_lse = O.ua_forward(*ins32)
    dl = (ops.as_reference_denom(lse_cm).cpu() - ref_lse).abs()
    assert ((dl <= 2e-2 + 1e-5 * ref_lse.abs()) | ~valid_row_mask(L, n, c)).all()
    del ref_lse, dl
    for kwargs in ({}, {"carry": carry, "lse": lse_cm}, {"carry": carry, "lse": lse_cm, "out_cm": out_cm}):
        got = ops.backward_cm(*cu, g_out_cm, g_den_cm, **kwargs)
        check_backward(f"L={L} {sorted(kwargs)}", got, ins32, g_out.float(), g_den)      # 5e-2, noise-pinned


@pytest.mark.parametrize("shape,skip", [((1, 2, 4, 1024, 128, 64), False), ((2, 1, 1, 768, 128, 64), False),
                                         ((1, 1, 2, 1024, 128, 64), True)])
def test_tensor_core_backward_matches_simt_backward(shape, skip):
    """The tcgen05 backward against the generic fp32 SIMT backward of the same library, on the device,
    with random upstream gradients (masked-block gradients included unless skipped)."""
    from universal_attention_triton_b200 import _lib, ops
    B, H, R, L, c, D = shape
    n = L // c
    ins, _ = _bf16_case(*shape, seed=31)
    cu = _cuda(*ins)
    gen = torch.Generator(device="cuda").manual_seed(7)
    g_out = torch.randn(B, H, n, R, L, D, generator=gen, device="cuda", dtype=torch.bfloat16)
    g_lse = torch.randn(B, H, n, R, L, generator=gen, device="cuda")
    if skip:        # zero the masked-block upstream gradient so that both modes must agree with the full computation
        valid = (torch.arange(L).view(1, L) >= torch.arange(n).view(n, 1) * c).cuda().view(1, 1, n, 1, L)
        g_out = g_out * valid.unsqueeze(-1)
        g_lse = g_lse * valid
    flags = _lib.FLAG_SKIP_MASKED_GRADS if skip else 0
    tc = ops.backward_cm(*cu, g_out, g_lse, flags=flags)
    out_cm = ops.forward_cm(*cu)[0]
    tc_out = ops.backward_cm(*cu, g_out, g_lse, flags=flags, out_cm=out_cm)      # row term from the forward's output tiles
    sm = ops.backward_cm(*cu, g_out, g_lse, flags=_lib.FLAG_FORCE_SIMT)
    for got in (tc, tc_out):
        for a, b, key in zip(got, sm, GRADS):
            assert torch.isfinite(a.float()).all(), key
            assert rel_fro(a.float().cpu(), b.float().cpu()) <= 2e-2, (key, rel_fro(a.float().cpu(), b.float().cpu()))


@pytest.mark.parametrize("skip", [False, True])
def test_backward_is_repeatable_at_full_occupancy(skip):
    """A grid that fills every SM several times over (B2 H8 L4096: 512 blocks), run repeatedly: the gradients
    of all runs agree up to the order of the fp32 atomic sums, and no bounded wait ran out.  Guards the
    hand-offs between the kernel's roles, whose faults show only under load and at many tiles per block."""
    from universal_attention_triton_b200 import _lib, ops
    shape = (2, 8, 4, 4096, 128, 64)
    B, H, R, L, c, D = shape
    n = L // c
    ins, _ = _bf16_case(*shape, seed=57)
    cu = _cuda(*ins)
    gen = torch.Generator(device="cuda").manual_seed(9)
    g_out = torch.randn(B, H, n, R, L, D, generator=gen, device="cuda", dtype=torch.bfloat16)
    g_lse = torch.randn(B, H, n, R, L, generator=gen, device="cuda")
    flags = _lib.FLAG_SKIP_MASKED_GRADS if skip else 0
    first = None
    for _ in range(4):
        grads = ops.backward_cm(*cu, g_out, g_lse, flags=flags)      # the status word is checked inside (UA_CHECK_STATUS=1)
        if first is None:
            first = [g.float() for g in grads]
            for g, key in zip(first, GRADS):
                assert torch.isfinite(g).all(), key
        else:
            for a, b, key in zip(first, grads, GRADS):
                assert rel_fro(b.float(), a) <= 1e-3, (key, rel_fro(b.float(), a))


def test_backward_with_kept_decay_table_matches_prepass():
    """ua_fwd_keep / ua_bwd_kept: the decay-prefix table handed over by the forward gives the same
    gradients as the backward's own pre-pass (same kernels; only fp32 atomic order differs)."""
    from universal_attention_triton_b200 import ops
    shape = (1, 2, 2, 768, 128, 64)
    B, H, R, L, c, D = shape
    n = L // c
    ins, _ = _bf16_case(*shape, seed=41)
    cu = _cuda(*ins)
    gen = torch.Generator(device="cuda").manual_seed(8)
    g_out = torch.randn(B, H, n, R, L, D, generator=gen, device="cuda", dtype=torch.bfloat16)
    g_lse = torch.randn(B, H, n, R, L, generator=gen, device="cuda")
    out_cm, lse_cm, den_cm, carry = ops.forward_cm(*cu, keep_carry=True)
    assert carry is not None and carry.numel() == B * H * n * n * 256
    out2, lse2, _ = ops.forward_cm(*cu)
    assert torch.equal(out_cm, out2) and torch.equal(lse_cm, lse2)
    a = ops.backward_cm(*cu, g_out, g_lse, carry=carry)
    b = ops.backward_cm(*cu, g_out, g_lse)
    for x, y, key in zip(a, b, GRADS):
        assert rel_fro(x.float().cpu(), y.float().cpu()) <= 1e-3, key
    # with the forward's fp32 log-sum-exp as well: probabilities formed as exp(s - lse) instead of through the
    # backward's own row max / sum (differences: rounding of P and dS to bf16 on slightly different fp32 values)
    c = ops.backward_cm(*cu, g_out, g_lse, carry=carry, lse=lse_cm)
    for x, y, key in zip(c, b, GRADS):
        assert torch.isfinite(x.float()).all(), key
        assert rel_fro(x.float().cpu(), y.float().cpu()) <= 5e-3, (key, rel_fro(x.float().cpu(), y.float().cpu()))


@pytest.mark.parametrize("shape,ranges", [((1, 2, 2, 1024, 128, 64), [(0, 3), (3, 8)]),
                                           ((1, 1, 1, 768, 128, 128), [(0, 2), (2, 4), (4, 6)])])
def test_forward_over_row_ranges_matches_whole_forward(shape, ranges):
    """ua_decay_totals_rows + ua_fwd_rows (the sequence-sharded forward), the ranks emulated one after the
    other on one GPU: the concatenated rows equal the whole-sequence forward up to fp32 association of the carry."""
    from universal_attention_triton_b200 import ops
    B, H, R, L, c, D = shape
    n = L // c
    ins, _ = _bf16_case(*shape, seed=51)
    kc, vc, xq, ss, sd = _cuda(*ins)
    out_full, lse_full, _ = ops.forward_cm(kc, vc, xq, ss, sd)
    totals = [ops.decay_totals_rows(kc, ss, sd[:, :, b * 128:e * 128], b, e) for b, e in ranges]
    outs, lses = [], []
    carry = torch.zeros_like(totals[0])
    for (b, e), tot in zip(ranges, totals):
        o, l, _ = ops.forward_rows_cm(kc, vc, xq[:, :, :, b * 128:e * 128], ss, sd[:, :, b * 128:e * 128], b, e, carry)
        outs.append(o); lses.append(l)
        carry = carry + tot
    out_sp = torch.cat(outs, dim=4)
    lse_sp = torch.cat(lses, dim=4)
    valid = (torch.arange(L).view(1, L) >= torch.arange(n).view(n, 1) * c).cuda().view(1, 1, n, 1, L)
    assert torch.equal(lse_sp[~valid.expand_as(lse_sp)], lse_full[~valid.expand_as(lse_full)])
    dl = (lse_sp - lse_full).abs()
    assert ((dl <= 1e-3 + 1e-6 * lse_full.abs()) | ~valid).all(), (dl * valid).max().item()
    err = (out_sp.float() - out_full.float()).abs()
    assert (err <= 2e-2 + out_full.float().abs() * 2.0 ** -7).all(), err.max().item()
    # chained totals: passing the running carry through carry_in gives the same table as summing per-range totals
    chained = ops.decay_totals_rows(kc, ss, sd[:, :, ranges[1][0] * 128:ranges[1][1] * 128], *ranges[1], carry_in=totals[0])
    assert (chained - (totals[0] + totals[1])).abs().max() <= 1e-2 + 1e-6 * chained.abs().max()


@pytest.mark.parametrize("ranges,skip", [([(0, 3), (3, 8)], False), ([(0, 2), (2, 5), (5, 8)], True)])
def test_backward_over_row_ranges_matches_whole_backward(ranges, skip):
    """ua_bwd_rows + ua_bwd_rows_suffix (the sequence-sharded backward), ranks emulated one after the other on one
    GPU: partial key-side gradients summed over the ranges, row-side gradients concatenated, against the
    whole-sequence backward of the same library."""
    from universal_attention_triton_b200 import _lib, ops
    shape = (1, 2, 2, 1024, 128, 64)
    B, H, R, L, c, D = shape
    n = L // c
    ins, _ = _bf16_case(*shape, seed=71)
    kc, vc, xq, ss, sd = _cuda(*ins)
    gen = torch.Generator(device="cuda").manual_seed(9)
    g_out = torch.randn(B, H, n, R, L, D, generator=gen, device="cuda", dtype=torch.bfloat16)
    g_lse = torch.randn(B, H, n, R, L, generator=gen, device="cuda")
    flags = _lib.FLAG_SKIP_MASKED_GRADS if skip else 0
    if skip:
        valid = (torch.arange(L).view(1, L) >= torch.arange(n).view(n, 1) * c).cuda().view(1, 1, n, 1, L)
        g_out = g_out * valid.unsqueeze(-1)
        g_lse = g_lse * valid
    ref = ops.backward_cm(kc, vc, xq, ss, sd, g_out, g_lse, flags=flags)
    totals = [ops.decay_totals_rows(kc, ss, sd[:, :, b * 128:e * 128], b, e) for b, e in ranges]
    carries = [sum(totals[:g], torch.zeros_like(totals[0])) for g in range(len(ranges))]
    parts = []
    for (b, e), carry in zip(ranges, carries):
        rows = slice(b * 128, e * 128)
        parts.append(ops.backward_rows(kc, vc, xq[:, :, :, rows], ss, sd[:, :, rows], g_out[:, :, :, :, rows].contiguous(),
                                       g_lse[:, :, :, :, rows].contiguous(), b, e, carry_in=carry, flags=flags))
    # second step: reverse carry from the later ranges
    for g, ((b, e), part) in enumerate(zip(ranges, parts)):
        if g + 1 < len(ranges):
            suffix = sum([p[5] for p in parts[g + 1:]], torch.zeros_like(parts[0][5]))
            ops.backward_rows_suffix(kc, vc, ss, sd[:, :, b * 128:e * 128], b, e, suffix, part[0], part[3], part[4])
    dk = sum(p[0] for p in parts).view(kc.shape)
    dv = sum(p[1] for p in parts).view(vc.shape)
    dxq = torch.cat([p[2] for p in parts], dim=3).to(torch.bfloat16)
    dsrc = sum(p[3] for p in parts).view(ss.shape)
    ddest = torch.cat([p[4] for p in parts], dim=2)
    for got, want, key in zip((dk, dv, dxq, dsrc, ddest), ref, GRADS):
        assert torch.isfinite(got.float()).all(), key
        assert rel_fro(got.float().cpu(), want.float().cpu()) <= 1e-2, (key, rel_fro(got.float().cpu(), want.float().cpu()))


@pytest.mark.parametrize("D,skip", [(64, False), (128, False), (128, True)])
def test_two_row_ranges_sharing_slabs_zigzag_style(D, skip):
    """One owner of the row-tile blocks {0, 3} and another of {1, 2} (the zig-zag assignment of two ranks), every owner
    with its two blocks in shared slabs (row_offset): forward and backward against the whole-sequence kernels.  The first
    owner hands the forward's decay-prefix table and log-sum-exp to its backward, the second lets the backward recompute
    them."""
    from universal_attention_triton_b200 import _lib, ops
    shape = (1, 1, 2, 1024, 128, D)
    B, H, R, L, c, D = shape
    n, nb = L // c, 2                                       # 4 blocks of 2 tiles
    ins, _ = _bf16_case(*shape, seed=81)
    kc, vc, xq, ss, sd = _cuda(*ins)
    gen = torch.Generator(device="cuda").manual_seed(10)
    g_out = torch.randn(B, H, n, R, L, D, generator=gen, device="cuda", dtype=torch.bfloat16)
    g_lse = torch.randn(B, H, n, R, L, generator=gen, device="cuda")
    flags = _lib.FLAG_SKIP_MASKED_GRADS if skip else 0
    if skip:
        valid = (torch.arange(L).view(1, L) >= torch.arange(n).view(n, 1) * c).cuda().view(1, 1, n, 1, L)
        g_out = g_out * valid.unsqueeze(-1)
        g_lse = g_lse * valid
    out_full, lse_full, _ = ops.forward_cm(kc, vc, xq, ss, sd)
    ref = ops.backward_cm(kc, vc, xq, ss, sd, g_out, g_lse, flags=flags)
    owners = [[0, 3], [1, 2]]
    rows_of = lambda blks: torch.cat([torch.arange(p * nb * 128, (p + 1) * nb * 128) for p in blks]).cuda()
    # decay totals of every block, carries in block order
    totals = {}
    for blks in owners:
        sd_l = sd[:, :, rows_of(blks)]
        for li, p in enumerate(blks):
            totals[p] = ops.decay_totals_rows(kc, ss, sd_l, p * nb, (p + 1) * nb, row_offset=li * nb * 128)
    carries, run = {}, torch.zeros_like(totals[0])
    for p in range(4):
        carries[p] = run
        run = run + totals[p]
    results = []
    for oi, blks in enumerate(owners):
        idx = rows_of(blks)
        xq_l, sd_l = xq[:, :, :, idx].contiguous(), sd[:, :, idx].contiguous()
        out = ops.alloc_forward_rows(kc, xq_l)
        table = ops.alloc_carry_table(kc) if oi == 0 else None
        assert oi == 1 or table is not None
        for li, p in enumerate(blks):
            ops.forward_rows_cm(kc, vc, xq_l, ss, sd_l, p * nb, (p + 1) * nb, carries[p], row_offset=li * nb * 128, out=out,
                                carry_table=table)
        assert ((out[1] - lse_full[:, :, :, :, idx]).abs() <= 1e-3 + 1e-6 * lse_full[:, :, :, :, idx].abs()).all()
        err = (out[0].float() - out_full[:, :, :, :, idx].float()).abs()
        assert (err <= 2e-2 + out_full[:, :, :, :, idx].float().abs() * 2.0 ** -7).all()
        acc = ops.alloc_backward_rows(kc, xq_l)
        go, gl = g_out[:, :, :, :, idx].contiguous(), g_lse[:, :, :, :, idx].contiguous()
        dct = {}
        for li, p in enumerate(blks):
            kept = {"carry_table": table, "lse_cm_rows": out[1]} if table is not None else {}
            dct[p] = ops.backward_rows(kc, vc, xq_l, ss, sd_l, go, gl, p * nb, (p + 1) * nb, carry_in=carries[p],
                                       row_offset=li * nb * 128, acc=acc, flags=flags, **kept)[5]
        results.append((blks, idx, sd_l, acc, dct))
    all_dct = {}
    for r_ in results:
        all_dct.update(r_[4])
    for blks, idx, sd_l, acc, _ in results:
        for li, p in enumerate(blks):
            if p < 3:
                suffix = sum([all_dct[q] for q in range(p + 1, 4)], torch.zeros_like(all_dct[0]))
                ops.backward_rows_suffix(kc, vc, ss, sd_l, p * nb, (p + 1) * nb, suffix, acc[0], acc[3], acc[4],
                                         row_offset=li * nb * 128)
    dk = sum(r_[3][0] for r_ in results).view(kc.shape)
    dv = sum(r_[3][1] for r_ in results).view(vc.shape)
    dsrc = sum(r_[3][3] for r_ in results).view(ss.shape)
    dxq = torch.empty_like(xq, dtype=torch.float32)
    ddest = torch.empty_like(sd, dtype=torch.float32)
    for blks, idx, sd_l, acc, _ in results:
        dxq[:, :, :, idx] = acc[2]
        ddest[:, :, idx] = acc[4]
    for got, want, key in zip((dk, dv, dxq, dsrc, ddest), ref, GRADS):
        assert rel_fro(got.float().cpu(), want.float().cpu()) <= 1e-2, (key, rel_fro(got.float().cpu(), want.float().cpu()))


@pytest.mark.parametrize("shape,mode", [((1, 2, 4, 1024, 128, 64), "fused"), ((2, 1, 1, 512, 128, 64), "fused"),
                                        ((1, 2, 4, 1024, 128, 64), "composed"), ((1, 1, 2, 256, 64, 64), "fused")])
def test_merged_entry_point_matches_composition_and_oracle(shape, mode):
    """UniversalAttentionMerged against the same composition through the library's separate kernels and against the
    oracle's driver flow (main.py:55-62).  "fused": the one-kernel backward (bf16 / chunk 128 / head_dim 64; other
    shapes fall back to the composed backward), whose delta = g . merged uses the bf16 merged output: 5e-2 against
    the oracle as the task states, a few e-2 against the composed path.  "composed": 1e-2 against the oracle."""
    ua = _ua()
    ua.set_merged_backward(mode)
    B, H, R, L, c, D = shape
    ins, ins32 = _bf16_case(*shape, seed=23)
    cu = _cuda(*ins)
    gen = torch.Generator(device="cuda").manual_seed(11)
    g = torch.randn(B, H, R, L, D, generator=gen, device="cuda").bfloat16()

    xs = [t.clone().requires_grad_() for t in cu]
    try:
        merged = ua.UniversalAttentionMerged.apply(*xs)
        merged.backward(g)
    finally:
        ua.set_merged_backward("composed")
    fused = [x.grad for x in xs]

    # the same composition through the library's separate kernels, with the fp32 log-sum-exp as merge weights (the
    # drop-in `denom` is rounded to bf16 as in the reference, which moves the weights: not the thing to compare with)
    from universal_attention_triton_b200 import _lib, ops
    out_cm, lse_cm, _ = ops.forward_cm(*cu)
    merged2 = ops.merge_fwd_cm(out_cm, lse_cm)
    assert torch.equal(merged.detach().reshape(merged2.shape), merged2)
    g_out_cm, g_lse_cm = ops.merge_bwd_cm(out_cm, lse_cm, g, skip_zero_weight_blocks=True)
    comp = ops.backward_cm(*cu, g_out_cm, g_lse_cm, flags=_lib.FLAG_SKIP_MASKED_GRADS)
    for a, b2, key in zip(fused, comp, GRADS):
        assert torch.isfinite(a.float()).all(), key
        assert rel_fro(a.float().cpu(), b2.float().cpu()) <= (5e-2 if mode == "fused" else 2e-3), (key, rel_fro(a.float().cpu(), b2.float().cpu()))

    # oracle: fp32 composition on the same bf16-rounded inputs
    zs = [t.clone().requires_grad_() for t in ins32]
    o_out, o_den, o_lse = O.ua_forward(*[z.detach() for z in zs])
    o_merged = O.merge_forward(o_out.float(), o_lse)
    assert (merged.float().cpu() - o_merged).abs().max() <= 2e-2 + 2.0 ** -8 * o_merged.abs().max()
    d_mat, d_vec = O.merge_backward(o_out.float(), o_lse, g.float().cpu())
    ref = O.ua_backward(*[z.detach() for z in zs], d_mat, d_vec)
    for a, b2, key in zip(fused, ref, GRADS):
        assert rel_fro(a.float().cpu(), b2.float()) <= (5e-2 if mode == "fused" else 1e-2), (key, rel_fro(a.float().cpu(), b2.float()))


@pytest.mark.parametrize("shape", [(1, 2, 4, 2048, 128, 64), (1, 1, 2, 4096, 128, 128)])
def test_merged_entry_point_low_memory_forward(shape):
    """UniversalAttentionMerged with the two-pass forward that never writes ``out`` (``ua_fwd_merged``) and the one-kernel
    backward: merged output within 2e-2 of the oracle's driver flow (main.py:55-56), gradients within 5e-2, and no tensor
    of the size of ``out`` (b,h,n,r,L,d) is ever allocated: the peak of the caching allocator stays below half of it."""
    ua = _ua()
    B, H, R, L, c, D = shape
    n = L // c
    ins, ins32 = _bf16_case(*shape, seed=29)
    cu = _cuda(*ins)
    gen = torch.Generator(device="cuda").manual_seed(12)
    g = torch.randn(B, H, R, L, D, generator=gen, device="cuda").bfloat16()
    xs = [t.clone().requires_grad_() for t in cu]
    out_bytes = B * H * n * R * L * D * 2
    ua.set_merged_forward("low_memory")
    ua.set_merged_backward("fused")
    try:
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        base = torch.cuda.memory_allocated()
        merged = ua.UniversalAttentionMerged.apply(*xs)
        merged.backward(g)
        torch.cuda.synchronize()
        peak = torch.cuda.max_memory_allocated() - base
    finally:
        ua.set_merged_forward("materialise")
        ua.set_merged_backward("composed")
    assert peak < out_bytes // 2, (peak, out_bytes)
    grads = [x.grad for x in xs]
    o_out, o_den, o_lse = O.ua_forward(*ins32)
    o_merged = O.merge_forward(o_out.float(), o_lse)
    assert (merged.float().cpu() - o_merged).abs().max() <= 2e-2 + 2.0 ** -8 * o_merged.abs().max()
    d_mat, d_vec = O.merge_backward(o_out.float(), o_lse, g.float().cpu())
    ref = O.ua_backward(*ins32, d_mat, d_vec)
    for a, b2, key in zip(grads, ref, GRADS):
        assert torch.isfinite(a.float()).all(), key
        assert rel_fro(a.float().cpu(), b2.float()) <= 5e-2, (key, rel_fro(a.float().cpu(), b2.float()))
    # the materialising forward gives the same merged output up to the rounding of the per-chunk outputs
    merged2 = ua.UniversalAttentionMerged.apply(*cu)
    assert (merged.float() - merged2.float()).abs().max().item() <= 2e-2


@pytest.mark.parametrize("dtype,shape", [(torch.float32, (1, 2, 2, 192, 64, 32)), (torch.bfloat16, (2, 1, 4, 384, 128, 64))])
def test_decode_steps_reproduce_the_rows_of_the_forward(dtype, shape):
    """ua_decode_step issued for t = 0, 1, 2, ... against growing caches gives row t of the whole-sequence forward
    (out and log-sum-exp of every key chunk that holds keys <= t), and its decay state is the forward's decay prefix.
    fp32: 1e-4 as for the fp32 kernels; bf16: the forward's own tolerance against the oracle."""
    from universal_attention_triton_b200 import ops
    B, H, R, L, c, D = shape
    n = L // c
    kc, vc, xq, ss, sd = O.make_inputs(B, H, R, L, c, D, dtype=dtype, seed=13)
    ref_out, _, ref_lse = O.ua_forward(*[t.float() for t in (kc, vc, xq, ss, sd)])     # (b,h,r,L,d,n), (b,h,r,L,n)
    k_cache = kc.reshape(B, H, L, D).cuda().contiguous()
    v_cache = vc.reshape(B, H, L, D).cuda().contiguous()
    src = ss.reshape(B, H, L).cuda().contiguous()
    q, dest = xq.cuda(), sd.cuda()
    state = torch.zeros(B, H, L, dtype=torch.float32, device="cuda")
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    worst_out = worst_lse = 0.0
    for t in range(L):
        out_t, lse_t = ops.decode_step(t, k_cache, v_cache, src, q[:, :, :, t].contiguous(), dest[:, :, t].contiguous(), state, c)
        nt = t // c + 1
        assert out_t.shape == (B, H, R, D, nt) and lse_t.shape == (B, H, R, nt)
        ro, rl = ref_out[:, :, :, t, :, :nt], ref_lse[:, :, :, t, :nt]
        eo = (out_t.float().cpu() - ro).abs() - 2.0 ** -8 * ro.abs() * (dtype != torch.float32)
        worst_out = max(worst_out, eo.max().item())
        worst_lse = max(worst_lse, ((lse_t.cpu() - rl).abs() - 1e-5 * rl.abs()).max().item())
    assert worst_out <= tol, worst_out
    assert worst_lse <= tol, worst_lse
    assert torch.isfinite(state).all()


@pytest.mark.parametrize("shape,gate_mean,gate_fp32", [
    ((1, 1, 1, 128, 128, 64), 0.0, False),      # a single key chunk: only the diagonal tile exists
    ((1, 3, 3, 256, 128, 64), 0.0, False),      # odd head counts
    ((1, 1, 8, 384, 128, 64), 0.0, False),      # eight query heads per kv head
    ((1, 2, 2, 512, 128, 64), -4.0, False),     # weak gates: almost no decay (the numerics-stress distribution)
    ((1, 2, 2, 512, 128, 64), 4.0, False),      # strong gates: most pairs saturate the clamp
    ((1, 2, 2, 384, 128, 64), 0.0, True),       # fp32 gates with bf16 keys / values / queries
])
def test_tensor_core_kernels_on_edge_shapes_and_gates(shape, gate_mean, gate_fp32):
    """Forward and backward of the tcgen05 kernels against the generic fp32 SIMT kernels of the same library on shapes
    and gate distributions at the edges of what the tensor-core path takes (strict masked-block gradients, and the
    backward both with and without the forward's log-sum-exp)."""
    from universal_attention_triton_b200 import _lib, ops
    B, H, R, L, c, D = shape
    n = L // c
    ins = list(O.make_inputs(B, H, R, L, c, D, dtype=torch.bfloat16, seed=77, gate_mean=gate_mean, gate_std=1.0))
    if gate_fp32:
        ins[3], ins[4] = ins[3].float(), ins[4].float()
    cu = _cuda(*ins)
    out_tc, lse_tc, den_tc, carry = ops.forward_cm(*cu, keep_carry=True)
    out_sm, lse_sm, _ = ops.forward_cm(*cu, flags=_lib.FLAG_FORCE_SIMT)
    valid = (torch.arange(L).view(1, L) >= torch.arange(n).view(n, 1) * c).cuda().view(1, 1, n, 1, L)
    assert ((out_tc.float() - out_sm.float()).abs() * valid.unsqueeze(-1)).max() <= 2e-2 + 2.0 ** -8 * out_sm.float().abs().max()
    assert (((lse_tc - lse_sm).abs() - 1e-5 * lse_sm.abs()) * valid).max() <= 2e-2
    assert (lse_tc[~valid.expand_as(lse_tc)] <= -1e11).all()
    gen = torch.Generator(device="cuda").manual_seed(78)
    g_out = torch.randn(B, H, n, R, L, D, generator=gen, device="cuda", dtype=torch.bfloat16)
    g_lse = torch.randn(B, H, n, R, L, generator=gen, device="cuda")
    sm = ops.backward_cm(*cu, g_out, g_lse, flags=_lib.FLAG_FORCE_SIMT)
    for kwargs in ({}, {"carry": carry, "lse": lse_tc}):
        tc = ops.backward_cm(*cu, g_out, g_lse, **kwargs)
        for a, b, key in zip(tc, sm, GRADS):
            assert torch.isfinite(a.float()).all(), key
            assert a.dtype == b.dtype
            assert rel_fro(a.float().cpu(), b.float().cpu()) <= 2e-2, (key, kwargs.keys(), rel_fro(a.float().cpu(), b.float().cpu()))


@pytest.mark.parametrize("shape", [(2, 2, 2, 256, 64), (1, 4, 1, 384, 48)])      # (b, n_kv, rep, s, d); d = 48 is zero-padded
def test_attention_wrapper_against_global_softmax(shape):
    """attention(q, k, v, ...) with the signature and head mapping of the reference's flash-style entry point
    (universal_attention_kernel_opt.py:433-583): output and gradients against a direct fp32 evaluation of
    softmax_k(q.k + decay) v over all keys, query head h reading kv head h % n_kv."""
    from universal_attention_triton_b200.Universal_Attention.attention_opt import attention
    b, n_kv, rep, s, d = shape
    gen = torch.Generator().manual_seed(5)
    q = torch.randn(b, n_kv * rep, s, d, generator=gen).bfloat16()
    k = torch.randn(b, n_kv, s, d, generator=gen).bfloat16()
    v = torch.randn(b, n_kv, s, d, generator=gen).bfloat16()
    src = torch.randn(b, n_kv, s, generator=gen).sigmoid().bfloat16()
    dst = torch.randn(b, n_kv, s, generator=gen).sigmoid().bfloat16()
    g = torch.randn(b, n_kv * rep, s, d, generator=gen).bfloat16()

    def reference(q, k, v, src, dst):
        kf = k.float()
        gram = kf @ kf.transpose(-1, -2)                                    # (b, kv, key, row)
        aff = gram.clamp_min(0).pow(2 / 3) * src.float().pow(1 / 3).unsqueeze(-1) * dst.float().pow(1 / 3).unsqueeze(-2)
        ell = torch.log1p(-aff.clamp(0, 1 - 1e-6))
        idx = torch.arange(s)
        ell = torch.where(idx.view(1, s) > idx.view(s, 1), ell, torch.zeros(()))
        decay = ell.cumsum(-1).masked_fill(idx.view(1, s) < idx.view(s, 1), -1e12)      # (b, kv, key, row)
        decay = decay.transpose(-1, -2).repeat(1, rep, 1, 1)                # head h -> kv head h % n_kv; (b, h, row, key)
        score = q.float() @ kf.repeat(1, rep, 1, 1).transpose(-1, -2) + decay
        return score.softmax(-1) @ v.float().repeat(1, rep, 1, 1)

    ins = [t.clone().requires_grad_() for t in (q.float(), k.float(), v.float(), src.float(), dst.float())]
    ref = reference(*ins)
    ref.backward(g.float())
    cu = [t.cuda().requires_grad_() for t in (q, k, v, src, dst)]
    out = attention(cu[0], cu[1], cu[2], True, 1.0, cu[3], cu[4])
    assert out.shape == q.shape and out.dtype == q.dtype
    out.backward(g.cuda())
    assert (out.float().cpu() - ref).abs().max() <= 2e-2 + 2.0 ** -8 * ref.abs().max()
    for a, r_, key in zip(cu, ins, ["dq", "dk", "dv", "dsrc", "ddest"]):
        assert rel_fro(a.grad.float().cpu(), r_.grad) <= 5e-2, (key, rel_fro(a.grad.float().cpu(), r_.grad))


@pytest.mark.parametrize("dtype,norm,sig", [(torch.float32, True, True), (torch.bfloat16, True, True), (torch.bfloat16, False, False)])
def test_input_prologue_matches_the_drivers_views(dtype, norm, sig):
    """prepare_inputs against the reference driver's transposes and views (main.py:24-31), with and without the key
    normalisation and gate sigmoid of its harness (_debug.py:470-475), forward and backward."""
    from universal_attention_triton_b200.input_prep import prepare_inputs
    b, s, n, n_kv, d, c = 2, 256, 6, 2, 64, 128
    rep = n // n_kv
    gen = torch.Generator().manual_seed(21)
    qs = torch.randn(b, s, n, d, generator=gen).to(dtype)
    ks = torch.randn(b, s, n_kv, d, generator=gen).to(dtype)
    vs = torch.randn(b, s, n_kv, d, generator=gen).to(dtype)
    gs = torch.randn(b, s, 2 * n_kv, generator=gen).to(dtype)

    def reference(qs, ks, vs, gs):
        if norm:
            ks = ks / (ks.pow(2).sum(-1, True).sqrt() + 1e-6)
        if sig:
            gs = gs.sigmoid()
        xq = qs.transpose(1, 2).reshape(b, n_kv, rep, s, d)
        kc = ks.transpose(1, 2).reshape(b, n_kv, s // c, c, d)
        vc = vs.transpose(1, 2).reshape(b, n_kv, s // c, c, d)
        st = gs.view(b, s, 2, n_kv).permute(2, 0, 3, 1)
        return kc, vc, xq, st[0].reshape(b, n_kv, s // c, c), st[1]

    ref_in = [t.float().clone().requires_grad_() for t in (qs, ks, vs, gs)]
    ref_out = reference(*ref_in)
    cu_in = [t.cuda().requires_grad_() for t in (qs, ks, vs, gs)]
    out = prepare_inputs(*cu_in, chunk=c, normalize_keys=norm, sigmoid_gates=sig)
    gens = [torch.randn(o.shape, generator=gen).to(dtype) for o in ref_out]
    torch.autograd.backward(ref_out, [g.float() for g in gens])
    torch.autograd.backward(out, [g.cuda() for g in gens])
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for a, r_ in zip(out, ref_out):
        assert a.shape == r_.shape and a.dtype == dtype
        assert (a.float().cpu() - r_).abs().max() <= tol * max(1.0, r_.abs().max().item())
    for a, r_, key in zip(cu_in, ref_in, ["query", "key", "value", "gates"]):
        assert rel_fro(a.grad.float().cpu(), r_.grad) <= (1e-5 if dtype == torch.float32 else 1e-2), key



def test_status_word_path_reports_a_timeout_without_any_kernel():
    """The path a host sees when a bounded device-side wait ran out: the first word of the workspace is non-zero and
    ``ua_workspace_status`` returns UA_ERR_TIMEOUT (9).  The word is written by the host here (no kernel, no hang);
    a cleared word reads UA_OK again, and the Python wrapper turns the code into an exception."""
    import ctypes
    from universal_attention_triton_b200 import _lib
    lib = _lib.load()
    ws = torch.zeros(256, dtype=torch.uint8, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.ua_workspace_status(ctypes.c_void_p(ws.data_ptr()), stream) == 0
    ws[0] = 1
    rc = lib.ua_workspace_status(ctypes.c_void_p(ws.data_ptr()), stream)
    assert rc == 9 and b"bounded device-side wait" in lib.ua_error_string(rc)
    with pytest.raises(_lib.UaLibraryError, match="bounded device-side wait"):
        _lib.check(rc, "status")
    ws.zero_()
    assert lib.ua_workspace_status(ctypes.c_void_p(ws.data_ptr()), stream) == 0


def test_bounded_wait_gives_up_and_reports_it():
    """The give-up path of the kernels' device-side waits, run for real but in 2 ms instead of 2 s: a one-block self-test
    whose two waiters (single thread, whole warp) wait on an mbarrier that nothing completes.  The waits run out, the block
    returns with the status word set as the kernels set it, ``ua_workspace_status`` reports UA_ERR_TIMEOUT with the note of
    the first waiter to give up, and the context stays usable (a forward call runs right after).  Nothing traps or hangs."""
    import ctypes, time
    from universal_attention_triton_b200 import _lib
    lib = _lib.load()
    ws = torch.zeros(256, dtype=torch.uint8, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    assert lib.ua_selftest_wait_timeout(ctypes.c_void_p(ws.data_ptr()), 256, 2000, stream) == 0
    rc = lib.ua_workspace_status(ctypes.c_void_p(ws.data_ptr()), stream)
    elapsed = time.perf_counter() - t0
    assert rc == 9
    assert 0.002 <= elapsed < 1.0, elapsed             # gave up after the 2 ms limit, far from the kernels' 2 s
    words = ws[:8].cpu().view(torch.int32)
    assert int(words[0]) == 3
    note = int(words[1])
    assert (note & 0xff) == 1 and (note >> 8) in (0, 32), note      # barrier 0; thread 0 or the leader of warp 1
    # bad arguments are refused before any launch
    assert lib.ua_selftest_wait_timeout(ctypes.c_void_p(ws.data_ptr()), 255, 2000, stream) == 4
    assert lib.ua_selftest_wait_timeout(ctypes.c_void_p(ws.data_ptr()), 256, 0, stream) == 1
    # the context is intact
    ua = _ua()
    ins, ins32 = _bf16_case(1, 1, 1, 256, 128, 64, seed=1)
    out, denom = ua.UniversalAttention.apply(*_cuda(*ins))
    ref_out, _, _ = O.ua_forward(*ins32)
    assert fwd_errors(out.float().cpu(), denom.float().cpu(), ref_out, ref_out.new_zeros(denom.shape), 128)["out_masked"] <= 2e-2


@pytest.mark.parametrize("shape", [(1, 1, 1, 128, 128, 64),        # a single chunk: no rows before any chunk, one tile
                                   (1, 1, 1, 128, 128, 128),
                                   (1, 3, 5, 384, 128, 64),        # odd head counts, R = 5
                                   (2, 1, 8, 256, 128, 128),       # R = 8 at head_dim 128
                                   (3, 1, 1, 640, 128, 64)])       # five chunks: a group of chunks that is not full
def test_small_and_odd_shapes_on_the_tensor_core_kernels(shape):
    """Edge shapes of the tensor-core path (one chunk, head counts that are not powers of two, chunk counts that do not fill
    a group of the rows-before-a-chunk kernels) against the fp32 oracle: out <= 2e-2, gradients <= 5e-2 rel-Frobenius, with
    random upstream gradients on every block (the gradient through the rows before each chunk included)."""
    B, H, R, L, c, D = shape
    ua = _ua()
    ins, ins32 = _bf16_case(*shape, seed=31)
    gen = torch.Generator().manual_seed(13)
    n = L // c
    g_out = torch.randn(B, H, R, L, D, n, generator=gen).bfloat16()
    g_denom = torch.randn(B, H, R, L, n, generator=gen)
    ref_out, ref_denom, _ = O.ua_forward(*ins32)
    ref_grads = O.ua_backward(*ins32, g_out.float(), g_denom)
    out, denom, grads = _run_op(ua.UniversalAttention.apply, _cuda(*ins), g_out.cuda(), g_denom.cuda())
    e = fwd_errors(out.float().cpu(), denom.float().cpu(), ref_out, ref_denom, c)
    assert e["out_masked"] <= 2e-2 and e["masked_denom_ok"], e
    for got, ref, key in zip(grads, ref_grads, GRADS):
        assert torch.isfinite(got.float()).all(), key
        assert rel_fro(got.float().cpu(), ref) <= 5e-2, (key, rel_fro(got.float().cpu(), ref))

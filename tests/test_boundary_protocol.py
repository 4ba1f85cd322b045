"""The drop-in boundary: import paths and Function protocol of the reference (main.py:2-6;
universal_attention_autograd.py:9, :41-44, :104, :166-169; Universal_Attention/universal_attention.py:7, :27-31)."""
import inspect

import pytest
import torch


def _classes():
    from universal_attention_autograd import SMVecMatMul, UniversalAttention, UniversalAttention2
    from Universal_Attention.universal_attention import UniversalAttention as KernelUA
    return UniversalAttention, UniversalAttention2, KernelUA, SMVecMatMul


def test_reference_import_paths_resolve_to_the_cuda_backed_classes():
    import universal_attention_triton_b200 as pkg
    ua1, ua2, kua, smv = _classes()
    assert ua1 is pkg.UniversalAttention and ua2 is pkg.UniversalAttention2 and smv is pkg.SMVecMatMul
    from universal_attention_triton_b200.Universal_Attention.universal_attention import UniversalAttention as inner
    assert kua is inner


def test_functions_follow_the_new_style_protocol():
    for cls in _classes()[:3]:
        params = list(inspect.signature(cls.forward).parameters)
        assert params == ["kc", "vc", "xq", "static_src", "static_dest"], params      # no ctx
        assert list(inspect.signature(cls.setup_context).parameters) == ["ctx", "inputs", "outputs"]
        assert "setup_context" in cls.__dict__ and "backward" in cls.__dict__
    smv = _classes()[3]
    assert list(inspect.signature(smv.forward).parameters) == ["mat", "vec"]


def test_note_on_gradients_that_vanish_before_each_chunk():
    """The note SMVecMatMul.backward leaves on its results (host logic, no GPU): it holds the tensor's version counter,
    an in-place change voids it, and tensors that autograd derives (a sum of two gradients, a hook's replacement) do not carry
    it -- so the operator's backward falls back to the full path whenever the zeros are not guaranteed."""
    from universal_attention_triton_b200 import universal_attention_autograd as M
    g = torch.zeros(2, 3)
    assert not M._masked_zero(g)
    M._mark_masked_zero(g)
    assert M._masked_zero(g)
    assert not M._masked_zero(g + 0)             # a new tensor
    assert not M._masked_zero(g.clone())
    g.add_(1.0)                                  # in-place change: the note is void
    assert not M._masked_zero(g)

    # through autograd: the note reaches the next node only when the tensor itself is handed on
    seen = []

    class Probe(torch.autograd.Function):
        @staticmethod
        def forward(x):
            return x * 1.0

        @staticmethod
        def setup_context(ctx, inputs, output):
            pass

        @staticmethod
        def backward(ctx, g):
            seen.append(M._masked_zero(g))
            return g

    class Source(torch.autograd.Function):
        @staticmethod
        def forward(x):
            return x.sum()

        @staticmethod
        def setup_context(ctx, inputs, output):
            ctx.shape = inputs[0].shape

        @staticmethod
        def backward(ctx, g):
            out = torch.ones(ctx.shape) * g
            M._mark_masked_zero(out)
            return out

    x = torch.randn(4, requires_grad=True)
    Source.apply(Probe.apply(x)).backward()                                  # single consumer: handed on
    y = Probe.apply(x)
    (Source.apply(y) + y.sum()).backward()                                   # two consumers: autograd sums the gradients
    y = Probe.apply(x)
    y.register_hook(lambda g: g * 1.0)                                       # a hook replaces the tensor
    Source.apply(y).backward()
    assert seen == [True, False, False]


def test_cpu_tensors_are_refused_not_computed():
    ua1 = _classes()[0]
    b, h, r, n, c, d = 1, 1, 1, 2, 16, 8
    args = (torch.randn(b, h, n, c, d), torch.randn(b, h, n, c, d), torch.randn(b, h, r, n * c, d),
            torch.rand(b, h, n, c), torch.rand(b, h, n * c))
    with pytest.raises(RuntimeError, match="no CPU path"):
        ua1.apply(*args)


def test_shape_asserts_fire_like_the_reference():
    ua1, ua2, kua, _ = _classes()
    b, h, r, n, c, d = 1, 1, 1, 2, 16, 8
    kc = torch.randn(b, h, n, c, d)
    with pytest.raises(AssertionError):
        ua1.apply(kc, kc, torch.randn(b, h, r, n * c, d), torch.rand(b, h, n, c), torch.rand(b, h, n * c + 1))
    with pytest.raises(AssertionError):
        kua.apply(kc, kc[:, :, :1], torch.randn(b, h, r, n, c, d), torch.rand(b, h, n, c), torch.rand(b, h, n, c))


@pytest.mark.gpu
def test_reference_driver_flow_through_the_import_shims():
    """main.py:41-62 with the reference's own import lines: clone().requires_grad_(), SMVecMatMul, retain_grad on the
    two outputs, pow(2).sum().backward(); all three entry points against the oracle on the driver's rand inputs."""
    from oracle import ua_oracle as O
    from tests._util import rel_fro
    ua1, ua2, kua, smv = _classes()
    b, s, n_kv, rep, d, c = 2, 256, 2, 2, 64, 64
    n_c = s // c
    g = torch.Generator().manual_seed(3)
    q = torch.rand(b, s, n_kv * rep, d, generator=g)
    k = torch.rand(b, s, n_kv, d, generator=g)
    v = torch.rand(b, s, n_kv, d, generator=g)
    st = torch.rand(b, s, 2 * n_kv, generator=g)
    xq = q.transpose(1, 2).reshape(b, n_kv, rep, s, d)
    kc = k.transpose(1, 2).reshape(b, n_kv, n_c, c, d)
    vc = v.transpose(1, 2).reshape(b, n_kv, n_c, c, d)
    st = st.view(b, s, 2, n_kv).permute(2, 0, 3, 1)
    ss, sd = st[0].reshape(b, n_kv, n_c, c), st[1].reshape(b, n_kv, s)
    _, merged_ref, _, _, grads_ref = O.driver_step(kc, vc, xq, ss, sd)
    ref = dict(zip(("dkc", "dvc", "dxq", "dsrc", "ddest"), grads_ref), merged=merged_ref)
    for fn, two_d in ((ua1, False), (ua2, True), (kua, True)):
        kc_, vc_, ss_ = (t.clone().detach().cuda().requires_grad_() for t in (kc, vc, ss))
        if two_d:
            xq_ = xq.view(b, n_kv, rep, n_c, c, d).clone().detach().cuda().requires_grad_()
            sd_ = sd.view(b, n_kv, n_c, c).clone().detach().cuda().requires_grad_()
        else:
            xq_, sd_ = xq.clone().detach().cuda().requires_grad_(), sd.clone().detach().cuda().requires_grad_()
        output, denom = fn.apply(kc_, vc_, xq_, ss_, sd_)
        out = smv.apply(output, denom)
        output.retain_grad()
        denom.retain_grad()
        out.pow(2).sum().backward()
        assert output.grad is not None and denom.grad is not None
        assert (out.cpu().reshape(ref["merged"].shape) - ref["merged"]).abs().max().item() <= 1e-4
        for name, t in (("dkc", kc_), ("dvc", vc_), ("dxq", xq_), ("dsrc", ss_), ("ddest", sd_)):
            assert rel_fro(t.grad.cpu().reshape(ref[name].shape), ref[name]) <= 1e-4, (fn, name)


@pytest.mark.gpu
def test_backward_recomputes_when_only_the_inputs_were_saved():
    """torch.func.grad drives forward / setup_context with its own wrappers; the Function must also work when the
    forward's by-products did not reach setup_context (they are then recomputed)."""
    from oracle import ua_oracle as O
    from tests._util import rel_fro
    from universal_attention_triton_b200 import universal_attention_autograd as M
    ua1, _, _, smv = _classes()
    ins = O.make_inputs(1, 1, 2, 256, 64, 64, dtype=torch.float32, seed=5)
    ref = dict(zip(("dkc", "dvc", "dxq", "dsrc", "ddest"), O.driver_step(*ins)[4]))

    def loss(kc, vc, xq, ss, sd):
        return smv.apply(*ua1.apply(kc, vc, xq, ss, sd)).pow(2).sum()

    grads = torch.func.grad(loss, argnums=(0, 1, 2, 3, 4))(*[t.cuda() for t in ins])
    for name, gr in zip(("dkc", "dvc", "dxq", "dsrc", "ddest"), grads):
        assert rel_fro(gr.cpu(), ref[name]) <= 1e-4, name

    class Ctx:           # setup_context without the by-products: a plain 2-tuple of fresh tensors
        def save_for_backward(self, *ts):
            self.saved_tensors = ts
    xs = [t.cuda() for t in ins]
    out, denom = M._forward(*xs)
    ctx = Ctx()
    M._setup_context(ctx, tuple(xs), (out.clone(), denom.clone()))
    assert not ctx.ua_has_extras and len(ctx.saved_tensors) == 5
    g_out = torch.randn_like(out)
    g_denom = torch.randn_like(denom)
    got = M._backward(ctx, g_out, g_denom)
    want = O.ua_backward(*ins, g_out.cpu(), g_denom.cpu())
    for a, b_, name in zip(got, want, ("dkc", "dvc", "dxq", "dsrc", "ddest")):
        assert rel_fro(a.cpu(), b_) <= 1e-4, name


@pytest.mark.gpu
def test_own_output_is_saved_for_backward_unless_switched_off():
    """By default the Functions save their own output with the inputs (the tensor-core backward takes the row term of the
    softmax gradient from out . g_out); switched off, they save the reference's five inputs plus the two by-products.
    Same gradients either way, up to the rounding of the bf16 output."""
    import universal_attention_triton_b200 as ua
    from oracle import ua_oracle as O
    from tests._util import rel_fro
    from universal_attention_triton_b200 import universal_attention_autograd as M
    ins = O.make_inputs(1, 2, 2, 512, 128, 64, dtype=torch.bfloat16, seed=9)

    class Ctx:
        def save_for_backward(self, *ts):
            self.saved_tensors = ts
    results = {}
    try:
        for on in (True, False):
            ua.set_save_output(on)
            xs = [t.cuda() for t in ins]
            out, denom = M._forward(*xs)
            ctx = Ctx()
            M._setup_context(ctx, tuple(xs), (out, denom))
            assert ctx.ua_has_extras and ctx.ua_has_out == on
            assert (ctx.saved_tensors[-1] is out) == on
            gen = torch.Generator(device="cuda").manual_seed(11)
            g_out = torch.randn(out.shape, generator=gen, device="cuda").to(out.dtype)
            g_denom = torch.randn(denom.shape, generator=gen, device="cuda")
            results[on] = [t.float().cpu() for t in M._backward(ctx, g_out, g_denom)]
    finally:
        ua.set_save_output(True)
    for a, b_, name in zip(results[True], results[False], ("dkc", "dvc", "dxq", "dsrc", "ddest")):
        assert torch.isfinite(a).all() and rel_fro(a, b_) <= 2e-2, (name, rel_fro(a, b_))

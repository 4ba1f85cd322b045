"""The CPU oracle against golden vectors produced by the unmodified reference
(tests/golden/make_golden.py).  fp32 rounding-order noise only."""
import pytest
import torch

from oracle import ua_oracle as O
from tests._util import fwd_errors, load_golden, rel_fro

RANDOM_UPSTREAM = ["tiny_1d_random_upstream", "tiny_2d_random_upstream", "tiny_2d_pruning_gates"]


@pytest.mark.parametrize("name", RANDOM_UPSTREAM)
def test_forward_matches_reference(name):
    g = load_golden(name)
    out, denom, _ = O.ua_forward(g["kc"], g["vc"], g["xq"], g["static_src"], g["static_dest"])
    c = g["kc"].shape[3]
    e = fwd_errors(out, denom, g["out"], g["denom"], c)
    assert e["out_valid"] < 2e-5 and e["out_masked"] < 1e-6, e
    assert e["denom_valid"] < 2e-4 and e["masked_denom_ok"], e
    assert out.shape == g["out"].shape and denom.shape == g["denom"].shape


@pytest.mark.parametrize("name", RANDOM_UPSTREAM)
def test_backward_matches_reference(name):
    g = load_golden(name)
    grads = O.ua_backward(g["kc"], g["vc"], g["xq"], g["static_src"], g["static_dest"], g["g_out"], g["g_denom"])
    for got, key in zip(grads, ["dkc", "dvc", "dxq", "dsrc", "ddest"]):
        assert got.shape == g[key].shape
        assert rel_fro(got, g[key]) < 2e-5, (key, rel_fro(got, g[key]))


@pytest.mark.parametrize("name", ["plumbing_1d_driver", "plumbing_2d_driver"])
def test_driver_flow_matches_reference(name):
    g = load_golden(name)
    loss, merged, out, denom, grads = O.driver_step(g["kc"], g["vc"], g["xq"], g["static_src"], g["static_dest"])
    rs = int(g["row_stride"])
    assert (out[:, :, :, ::rs] - g["out_rows"]).abs().max() < 1e-3          # far chunks are ill-conditioned in fp32
    assert (merged - g["merged"]).abs().max() < 2e-5
    assert abs(loss.item() - g["loss"].item()) / g["loss"].item() < 1e-5
    for got, key in zip(grads, ["dkc", "dvc", "dxq", "dsrc", "ddest"]):
        assert rel_fro(got, g[key]) < 5e-5, (key, rel_fro(got, g[key]))


def test_fp64_arbiter_close_to_fp32():
    g = load_golden("tiny_1d_random_upstream")
    o32, d32, _ = O.ua_forward(g["kc"], g["vc"], g["xq"], g["static_src"], g["static_dest"])
    o64, d64, _ = O.ua_forward(g["kc"], g["vc"], g["xq"], g["static_src"], g["static_dest"], torch.float64)
    c = g["kc"].shape[3]
    e = fwd_errors(o32, d32, o64, d64, c)
    assert e["out_valid"] < 1e-4, e


def test_masked_blocks_are_chunk_mean():
    """Rows before a key chunk see a uniform softmax: out = mean(v_chunk), denom = -1e12
    (universal_attention_autograd.py:28: fp32 absorbs k.q next to -1e12)."""
    g = load_golden("tiny_1d_random_upstream")
    out = g["out"]
    vc = g["vc"]
    n, c = vc.shape[2], vc.shape[3]
    for i in range(1, n):
        mean = vc[:, :, i].mean(dim=2)                      # (b,h,d)
        blk = out[:, :, :, : i * c, :, i]                   # (b,h,r,rows,d)
        assert (blk - mean[:, :, None, None, :]).abs().max() < 1e-6
        assert (g["denom"][:, :, :, : i * c, i] < -9.9e11).all()

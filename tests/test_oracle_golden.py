"""The CPU oracle against the golden vectors produced by the reference itself
(tests/golden/make_golden.py).  fp32 vs fp32: agreement to ~1e-5."""
import pytest
import torch

from oracle import parallax_oracle as orc
from tests._util import golden_names, load_golden

TOL = dict(rtol=2e-4, atol=2e-5)


@pytest.mark.parametrize("name", golden_names("train"))
def test_train_forward_backward(name):
    g = load_golden("train", name)
    f = orc.train_forward(g["q"], g["r"], g["k"], g["v"], None, g["window"])
    torch.testing.assert_close(f["o"], g["o"], **TOL)
    grads = orc.train_backward(g["q"], g["r"], g["k"], g["v"], g["go"].float(), None, g["window"])
    for got, key in zip(grads, ("dq", "dr", "dk", "dv")):
        torch.testing.assert_close(got, g[key], **TOL)
    # statistics are consistent with the output they describe
    assert torch.isfinite(f["m"]).all() and (f["d1"] >= 1.0 - 1e-5).all()


@pytest.mark.parametrize("name", golden_names("train"))
def test_train_row_blocking_is_invisible(name):
    g = load_golden("train", name)
    a = orc.train_backward(g["q"], g["r"], g["k"], g["v"], g["go"].float(), None, g["window"], row_block=1024)
    b = orc.train_backward(g["q"], g["r"], g["k"], g["v"], g["go"].float(), None, g["window"], row_block=17)
    for x, y in zip(a, b):
        torch.testing.assert_close(x, y, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("name", golden_names("varlen"))
def test_varlen(name):
    g = load_golden("varlen", name)
    cu = g["cu_seqlens"].tolist()
    f = orc.varlen_forward(g["q"], g["r"], g["k"], g["v"], cu, None, g["window"])
    torch.testing.assert_close(f["o"], g["o"], **TOL)
    grads = orc.varlen_backward(g["q"], g["r"], g["k"], g["v"], g["go"].float(), cu, None, g["window"])
    for got, key in zip(grads, ("dq", "dr", "dk", "dv")):
        torch.testing.assert_close(got, g[key], **TOL)


@pytest.mark.parametrize("n_splits", [1, 3])
@pytest.mark.parametrize("name", golden_names("decode"))
def test_decode(name, n_splits):
    g = load_golden("decode", name)
    out = orc.decode(g["q"], g["r"], g["k"], g["v"], None, window_size_left=g["window"],
                     cache_start=g.get("cache_start"), seqused_k=g.get("seqused_k"), n_splits=n_splits)
    torch.testing.assert_close(out, g["o"], **TOL)


def test_decode_merge_ignores_empty_ranges():
    g = load_golden("decode", "plain_d64")
    q, r, k, v = g["q"][0, 0], g["r"][0, 0], g["k"][0], g["v"][0]
    whole = orc.decode_merge([orc.decode_partial(q, r, k, v, 0.125, 0, 200)])
    parts = [orc.decode_partial(q, r, k, v, 0.125, 0, 0), orc.decode_partial(q, r, k, v, 0.125, 0, 77),
             orc.decode_partial(q, r, k, v, 0.125, 77, 200), orc.decode_partial(q, r, k, v, 0.125, 200, 200)]
    torch.testing.assert_close(orc.decode_merge(parts), whole, **TOL)
    empty = orc.decode_merge([parts[0]])
    assert torch.equal(empty, torch.zeros_like(empty))


def test_mse_loss_grad_matches_autograd():
    o = torch.randn(2, 3, 5, 4, requires_grad=True)
    o.float().pow(2).mean().backward()
    torch.testing.assert_close(orc.mse_loss_grad(o.detach()), o.grad)

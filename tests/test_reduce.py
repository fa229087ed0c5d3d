"""Sum, Mean, Var and VarMean parity (cases of the reference's tests/test_sum.py, test_mean.py,
test_var.py and test_var_mean.py, seeded, plus wide, ragged and 16-bit rows)."""

import pytest
import torch

import trident_b200 as trident
from oracle import torch_oracle
from tests import util

pytestmark = pytest.mark.gpu

RTOL = ATOL = 1e-5  # fp32 row reductions: the tolerance of the fp32 norms

SHAPES = [(4, 2000, 0), (2000, 4, 1), (2000, 4, 0), (4, 2000, 1), (1, 16, 0), (16, 1, 1), (37, 1024, 1),
          (5, 4096, -1), (3, 12288, 1), (300, 1000, 0), (6, 70000, 1)]


def _scale(x_size, y_size, dim):
    # sums of n unit-variance terms grow like sqrt(n): the absolute tolerance follows
    n = x_size if dim != 0 else y_size
    return max(1.0, n ** 0.5)


@pytest.mark.parametrize("y_size, x_size, dim", SHAPES)
@pytest.mark.parametrize("name", ["sum", "mean", "var"])
def test_forward(name, y_size, x_size, dim, device):
    if name == "var" and (x_size if dim != 0 else y_size) < 2:
        pytest.skip("variance of one element with correction 1 is 0/0 in the oracle too")
    x = util.randn(y_size, x_size, seed=1)
    got = getattr(trident.function, name)(x.to(device), dim)
    want = getattr(torch_oracle, name)(x, dim)
    util.assert_close(got, want, RTOL, ATOL * (_scale(x_size, y_size, dim) if name == "sum" else 1.0), name)


@pytest.mark.parametrize("y_size, x_size, dim", [(4, 2000, 0), (2000, 4, 1), (37, 1024, 1), (9, 4096, -1), (300, 1000, 0)])
@pytest.mark.parametrize("correction", [0, 1])
def test_var_mean_forward(y_size, x_size, dim, correction, device):
    x = util.randn(y_size, x_size, seed=3, mean=0.5)
    got_v, got_m = trident.function.var_mean(x.to(device), dim, correction)
    want_v, want_m = torch_oracle.var_mean(x, dim, correction)
    util.assert_close(got_v, want_v, RTOL, ATOL, "var_mean var")
    util.assert_close(got_m, want_m, RTOL, ATOL, "var_mean mean")


@pytest.mark.parametrize("y_size, x_size, dim", [(2000, 4, 0), (4, 2000, 1), (37, 1024, 1), (9, 4096, -1), (300, 1000, 0), (3, 70000, 1)])
@pytest.mark.parametrize("name", ["sum", "mean", "var"])
def test_backward(name, y_size, x_size, dim, device):
    x = util.randn(y_size, x_size, seed=1)
    dy = util.randn(x_size if dim == 0 else y_size, seed=2)

    def train(fn, dev):
        i = x.detach().clone().to(dev).requires_grad_(True)
        fn(i, dim).backward(dy.to(dev))
        return i.grad

    got = train(getattr(trident.function, name), device)
    want = train(getattr(torch_oracle, name), "cpu")
    util.assert_close(got, want, RTOL, ATOL, f"{name} grad")


@pytest.mark.parametrize("y_size, x_size, dim", [(2000, 4, 0), (4, 2000, 1), (9, 4096, -1)])
@pytest.mark.parametrize("which", ["both", "var", "mean"])
def test_var_mean_backward(y_size, x_size, dim, which, device):
    x = util.randn(y_size, x_size, seed=5, mean=-0.25)
    n_out = x_size if dim == 0 else y_size
    gv, gm = util.randn(n_out, seed=6), util.randn(n_out, seed=7)

    def train(fn, dev):
        i = x.detach().clone().to(dev).requires_grad_(True)
        v, m = fn(i, dim, 1)
        loss = 0
        if which in ("both", "var"):
            loss = loss + (v * gv.to(dev)).sum()
        if which in ("both", "mean"):
            loss = loss + (m * gm.to(dev)).sum()
        loss.backward()
        return i.grad

    util.assert_close(train(trident.function.var_mean, device), train(torch_oracle.var_mean, "cpu"), RTOL, ATOL,
                      "var_mean grad")


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_half_precision(dt, device):
    x = util.randn(64, 4096, seed=9).to(dt)
    dy = util.randn(64, seed=10).to(dt)
    i = x.detach().clone().to(device).requires_grad_(True)
    v, m = trident.function.var_mean(i, -1, 1)
    assert v.dtype == dt and m.dtype == dt
    want_v, want_m = torch_oracle.var_mean(x.float(), -1, 1)
    util.assert_half_close(v, want_v, dt, 1e-2, 1, "var")
    util.assert_half_close(m, want_m, dt, 1e-2, 1, "mean")
    v.backward(dy.to(device))
    j = x.detach().clone().float().requires_grad_(True)
    torch_oracle.var(j, -1, 1).backward(dy.float())
    util.assert_half_close(i.grad, j.grad, dt, 1e-2, 1, "var grad")
    s = trident.function.sum(x.to(device), 1)
    util.assert_half_close(s, x.float().sum(1), dt, 1e-2, 1, "sum")


@pytest.mark.parametrize("module, args", [("Sum", (1,)), ("Mean", (0,)), ("Var", (1, 0)), ("VarMean", (1, 1))])
def test_modules(module, args, device, dtype):
    x = torch.randn(8, 32, device=device, dtype=dtype)
    out = getattr(trident, module)(*args).forward(x)
    outs = out if isinstance(out, tuple) else (out,)
    assert all(o is not None and o.dtype == dtype for o in outs)


def test_strided_input(device):
    x = util.randn(40, 512, seed=11)
    view = x.to(device)[:, ::2]  # not contiguous: the operation densifies it
    util.assert_close(trident.function.mean(view, 1), torch_oracle.mean(x[:, ::2], 1), RTOL, ATOL, "strided mean")


def test_rejects_other_ranks(device):
    with pytest.raises(ValueError):
        trident.function.sum(torch.zeros(2, 3, 4, device=device), 1)


def test_variance_with_outlier_and_large_mean(device):
    """The one-pass variance shifts by a sample of the row: an outlier in the first position and a
    mean far from zero must not cost accuracy."""
    x = util.randn(16, 4096, seed=21) * 0.5 + 300.0
    x[:, 0] = 1.0e4
    got_v, got_m = trident.function.var_mean(x.to(device), 1, 1)
    want_v, want_m = torch.var_mean(x.double(), 1, correction=1)
    assert torch.allclose(got_v.cpu().double(), want_v, rtol=2e-5, atol=0), (got_v.cpu().double() - want_v).abs().max()
    assert torch.allclose(got_m.cpu().double(), want_m, rtol=1e-6, atol=0)
    y = util.randn(8, 1024, seed=22) * 1e-3 + 5.0e3  # spread far below the mean
    got = trident.function.var(y.to(device), 1, 1)
    want = torch.var(y.double(), 1, correction=1)
    assert torch.allclose(got.cpu().double(), want, rtol=1e-3, atol=0), (got.cpu().double() / want)

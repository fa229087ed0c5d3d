"""Edge cases: empty inputs, single rows and columns, non-contiguous inputs and gradients."""

import pytest
import torch

import trident_b200 as trident
from oracle import torch_oracle
from tests import util

pytestmark = pytest.mark.gpu


def _grads(fn, leaves, dy, dev):
    leaves = [None if t is None else t.detach().clone().to(dev).requires_grad_(True) for t in leaves]
    out = fn(*leaves)
    out.backward(dy.to(dev))
    return [out.detach()] + [t.grad for t in leaves if t is not None]


@pytest.mark.parametrize("cols", [8, 1024])
def test_zero_rows(cols, device):
    x, dy = torch.zeros(0, cols), torch.zeros(0, cols)
    w, b = util.randn(cols, seed=1), util.randn(cols, seed=2)
    cases = [
        (lambda i, j, k: trident.function.layer_norm(i, (cols,), j, k), lambda i, j, k: torch_oracle.layer_norm(i, (cols,), j, k), [x, w, b]),
        (lambda i, j, k: trident.function.rms_norm(i, -1.0, j, k), lambda i, j, k: torch_oracle.rms_norm(i, -1.0, j, k), [x, w, b]),
        (lambda i: trident.function.softmax(i, 1), lambda i: torch_oracle.softmax(i, 1), [x]),
    ]
    for ours, ref, leaves in cases:
        got, want = _grads(ours, leaves, dy, device), _grads(ref, leaves, dy, "cpu")
        for g, w_ in zip(got, want):
            assert g.shape == w_.shape
            util.assert_close(g, w_, 1e-5, 1e-5, "zero rows")
    for name in ("sum", "mean"):
        got = getattr(trident.function, name)(x.to(device), 1)
        assert got.shape == (0,)


def test_zero_rows_linear_and_geglu(device):
    x = torch.zeros(1, 0, 64)
    w, b = util.randn(32, 64, seed=1, std=0.1), util.randn(32, seed=2)
    dy = torch.zeros(1, 0, 32)
    got = _grads(trident.function.linear, [x, w, b], dy, device)
    want = _grads(torch_oracle.linear, [x, w, b], dy, "cpu")
    for g, w_ in zip(got, want):
        assert g.shape == w_.shape
        util.assert_close(g, w_, 1e-5, 1e-5, "linear with no rows")
    got = _grads(trident.function.geglu, [x, w, b], torch.zeros(1, 0, 16), device)
    want = _grads(torch_oracle.geglu, [x, w, b], torch.zeros(1, 0, 16), "cpu")
    for g, w_ in zip(got, want):
        assert g.shape == w_.shape
        util.assert_close(g, w_, 1e-5, 1e-5, "geglu with no rows")


def test_single_row_and_single_column(device):
    x = util.randn(1, 1, seed=3)
    util.assert_close(trident.function.softmax(x.to(device), 1), torch.ones(1, 1), 0, 0, "softmax 1x1")
    util.assert_close(trident.function.sum(x.to(device), 1), x.sum(1), 1e-6, 1e-6, "sum 1x1")
    col = util.randn(257, 1, seed=4)
    util.assert_close(trident.function.softmax(col.to(device), 0), torch_oracle.softmax(col, 0), 1e-5, 1e-5, "softmax column")
    util.assert_close(trident.function.var(col.to(device), 0, 1), torch_oracle.var(col, 0, 1), 1e-5, 1e-5, "var column")
    row = util.randn(1, 4096, seed=5)
    w = util.randn(4096, seed=6)
    got = _grads(lambda i, j: trident.function.layer_norm(i, (4096,), j, None), [row, w], util.randn(1, 4096, seed=7), device)
    want = _grads(lambda i, j: torch_oracle.layer_norm(i, (4096,), j, None), [row, w], util.randn(1, 4096, seed=7), "cpu")
    for g, w_ in zip(got, want):
        util.assert_close(g, w_, 1e-5, 2e-5, "layer_norm one row")


def test_non_contiguous_input_and_gradient(device):
    base = util.randn(64, 2048, seed=8)
    dy_base = util.randn(2048, 64, seed=9)
    x = base[:, ::2]            # column-strided view
    dy = dy_base.t()[:, ::2]    # transposed and strided gradient
    w = util.randn(1024, seed=10)

    def ours(i, j):
        return trident.function.layer_norm(i, (1024,), j, None)

    def ref(i, j):
        return torch_oracle.layer_norm(i, (1024,), j, None)

    xi = base.to(device)[:, ::2].detach().requires_grad_(True)
    wi = w.to(device).detach().requires_grad_(True)
    ours(xi, wi).backward(dy_base.to(device).t()[:, ::2])
    xr = x.detach().clone().requires_grad_(True)
    wr = w.detach().clone().requires_grad_(True)
    ref(xr, wr).backward(dy)
    util.assert_close(xi.grad, xr.grad, 1e-5, 2e-5, "strided layer_norm dx")
    util.assert_close(wi.grad, wr.grad, 1e-5, 1e-4, "strided layer_norm dw")
    s = trident.function.softmax(base.to(device)[:, ::2], 1)
    util.assert_close(s, torch_oracle.softmax(x, 1), 1e-5, 1e-5, "strided softmax")

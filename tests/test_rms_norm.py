"""RMSNorm parity (cases of the reference's tests/test_rms_norm.py, seeded)."""

import pytest
import torch

import trident_b200 as trident
from oracle import torch_oracle
from tests import util

pytestmark = pytest.mark.gpu


RTOL = ATOL = 1e-5


@pytest.mark.parametrize("y_size, x_size, p", [(1000, 10, 0.5), (10, 1000, 1.0), (64, 4096, -1.0), (17, 1024, 0.25)])
def test_forward(y_size, x_size, p, device):
    x = util.randn(y_size, x_size, seed=1)
    w = util.randn(x_size, seed=2)
    b = util.randn(x_size, seed=3)
    util.assert_close(
        trident.function.rms_norm(x.to(device), p, w.to(device)), torch_oracle.rms_norm(x, p, w), RTOL, ATOL, "rms fwd"
    )
    util.assert_close(
        trident.function.rms_norm(x.to(device), p, w.to(device), b.to(device)),
        torch_oracle.rms_norm(x, p, w, b),
        RTOL,
        ATOL,
        "rms fwd bias",
    )


@pytest.mark.parametrize("y_size, x_size, p", [(1000, 10, 0.5), (10, 1000, 1.0), (200, 4096, -1.0), (90, 1024, 0.5)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_backward(y_size, x_size, p, with_bias, device):
    x = util.randn(y_size, x_size, seed=1)
    w = util.randn(x_size, seed=2)
    b = util.randn(x_size, seed=3) if with_bias else None
    dy = util.randn(y_size, x_size, seed=4)

    def train(fn, dev):
        i = x.detach().clone().to(dev).requires_grad_(True)
        j = w.detach().clone().to(dev).requires_grad_(True)
        k = None if b is None else b.detach().clone().to(dev).requires_grad_(True)
        fn(i, p, j, k).backward(dy.to(dev))
        return [t.grad for t in (i, j, k) if t is not None]

    for got, want, name in zip(train(trident.function.rms_norm, device), train(torch_oracle.rms_norm, "cpu"), "xwb"):
        util.assert_close(got, want, 1e-5, 1e-5 * max(1.0, y_size ** 0.5), f"rms grad {name}")


def test_strided_rows(device):
    """A column slice of a wider matrix: row stride differs from the width."""
    base = util.randn(50, 2048, seed=9)
    w = util.randn(1024, seed=2)
    x_cpu = base[:, 512:1536]
    x_dev = base.to(device)[:, 512:1536]
    got = trident.operation.RMSNorm.apply(x_dev, -1.0, w.to(device), None, 1e-6)
    util.assert_close(got, torch_oracle.rms_norm(x_cpu, -1.0, w, None, 1e-6), RTOL, ATOL, "rms strided")


def test_three_dim_input(device):
    x = util.randn(3, 7, 256, seed=1)
    w = util.randn(256, seed=2)
    got = trident.function.rms_norm(x.to(device), -1.0, w.to(device))
    util.assert_close(got, torch_oracle.rms_norm(x, -1.0, w), RTOL, ATOL, "rms 3d")


@pytest.mark.parametrize("y_size, x_size", [(4, 16)])
def test_rms_norm(y_size, x_size, device, dtype):
    factory_kwargs = {"device": device, "dtype": dtype}
    input = torch.randn(y_size, x_size, **factory_kwargs, requires_grad=True)
    grad_output = torch.randn_like(input)

    output = trident.RMSNorm(x_size, **factory_kwargs).forward(input)
    assert output is not None and output.dtype == dtype
    output = trident.RMSNorm(x_size, 0.5, **factory_kwargs).forward(input)
    assert output is not None and output.dtype == dtype
    output = trident.RMSNorm(x_size, bias=True, **factory_kwargs).forward(input)
    assert output is not None and output.dtype == dtype
    output = trident.RMSNorm(x_size, 0.5, bias=True, **factory_kwargs).forward(input)
    assert output is not None and output.dtype == dtype

    output.backward(grad_output)
    assert input.grad is not None
    assert input.grad.dtype == dtype

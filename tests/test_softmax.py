"""Softmax parity (cases of the reference's tests/test_softmax.py, seeded)."""

import pytest
import torch

import trident_b200 as trident
from oracle import torch_oracle
from tests import util

pytestmark = pytest.mark.gpu

RTOL = ATOL = 1e-5


@pytest.mark.parametrize(
    "y_size, x_size, dim", [(2, 512, 0), (3, 1000, 1), (5, 4096, 1), (7, 10, 1), (4, 16384, -1), (2, 70000, 1)]
)
def test_forward(y_size, x_size, dim, device):
    x = util.randn(y_size, x_size, seed=1, std=2.0)
    util.assert_close(trident.function.softmax(x.to(device), dim), torch_oracle.softmax(x, dim), RTOL, ATOL, "softmax")


@pytest.mark.parametrize("y_size, x_size, dim", [(3, 1000, 0), (2, 512, 1), (9, 4096, 1), (6, 8192, -1)])
def test_backward(y_size, x_size, dim, device):
    x = util.randn(y_size, x_size, seed=1, std=2.0)
    dy = util.randn(y_size, x_size, seed=2)

    def train(fn, dev):
        i = x.detach().clone().to(dev).requires_grad_(True)
        fn(i, dim).backward(dy.to(dev))
        return i.grad

    util.assert_close(train(trident.function.softmax, device), train(torch_oracle.softmax, "cpu"), RTOL, ATOL, "softmax bwd")


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_half_forward_backward(dt, device):
    """16-bit I/O with fp32 arithmetic: at most one rounding away from the fp32 result."""
    x = util.randn(33, 4096, seed=3, std=2.0, dtype=dt)
    dy = util.randn(33, 4096, seed=4, dtype=dt)
    i = x.to(device).requires_grad_(True)
    y = trident.function.softmax(i, -1)
    y.backward(dy.to(device))
    ref_in = x.float().requires_grad_(True)
    ref = torch_oracle.softmax(ref_in, -1)
    tiny = 6e-8 if dt == torch.float16 else 0.0  # spacing of fp16 subnormals
    util.assert_half_close(y, ref, dt, atol=0.0, ulps=0.51, what="y", tiny=tiny)
    # backward is taken from the rounded y, as the oracle in the same dtype does
    y16 = y.detach().float().cpu()
    want_dx = y16 * (dy.float() - (y16 * dy.float()).sum(-1, keepdim=True))
    util.assert_half_close(i.grad, want_dx, dt, atol=1e-7, ulps=0.51, what="dx", tiny=tiny)


@pytest.mark.parametrize("y_size, x_size, dim", [(1, 32, 0), (1, 32, 1)])
def test_softmax(y_size, x_size, dim, device, dtype):
    factory_kwargs = {"device": device, "dtype": dtype}
    input = torch.randn(y_size, x_size, **factory_kwargs, requires_grad=True)
    grad_output = torch.randn_like(input)
    output = trident.Softmax(dim).forward(input)
    assert output is not None and output.dtype == dtype
    output.backward(grad_output)
    assert input.grad is not None and input.grad.dtype == dtype

"""MaskedSoftmax parity (cases of the reference's tests/test_masked_softmax.py, seeded)."""

import pytest
import torch

import trident_b200 as trident
from oracle import torch_oracle
from tests import util

pytestmark = pytest.mark.gpu

RTOL = ATOL = 1e-5


def build_mask(y_size, x_size, dim, seed, dtype=torch.int64):
    """Random 0/1 mask with row 0 (dim 0) or column 0 (dim 1) forced unmasked, so that no
    slice is fully masked (tests/test_masked_softmax.py:29-33)."""
    mask = torch.randint(0, 2, (y_size, x_size), generator=util.seeded(seed))
    if dim == 0:
        mask[0, :] = 0
    else:
        mask[:, 0] = 0
    return mask.to(dtype)


@pytest.mark.parametrize("y_size, x_size, dim", [(2, 512, 0), (3, 1000, 1), (8, 4096, 1), (5, 10, 1)])
@pytest.mark.parametrize("mask_dtype", [torch.int64, torch.bool, torch.uint8, torch.float32])
def test_forward(y_size, x_size, dim, mask_dtype, device):
    x = util.randn(y_size, x_size, seed=1, std=2.0)
    mask = build_mask(y_size, x_size, dim, 2, mask_dtype)
    got = trident.function.masked_softmax(x.to(device), mask.to(device), dim)
    util.assert_close(got, torch_oracle.masked_softmax(x, mask, dim), RTOL, ATOL, "masked softmax")


@pytest.mark.parametrize("y_size, x_size, dim", [(3, 1000, 0), (2, 512, 1), (8, 4096, 1)])
def test_backward(y_size, x_size, dim, device):
    x = util.randn(y_size, x_size, seed=1, std=2.0)
    dy = util.randn(y_size, x_size, seed=3)
    mask = build_mask(y_size, x_size, dim, 2)

    def train(fn, dev):
        i = x.detach().clone().to(dev).requires_grad_(True)
        fn(i, mask.to(dev), dim).backward(dy.to(dev))
        return i.grad

    util.assert_close(
        train(trident.function.masked_softmax, device), train(torch_oracle.masked_softmax, "cpu"), RTOL, ATOL, "masked bwd"
    )


def test_masked_positions_are_exact_zero(device):
    x = util.randn(16, 4096, seed=1, dtype=torch.float16)
    mask = build_mask(16, 4096, 1, 2, torch.bool)
    i = x.to(device).requires_grad_(True)
    y = trident.function.masked_softmax(i, mask.to(device), 1)
    y.backward(torch.ones_like(y))
    assert (y.detach().cpu()[mask] == 0).all()
    assert (i.grad.cpu()[mask] == 0).all()


@pytest.mark.parametrize("y_size, x_size, dim", [(1, 32, 0), (1, 32, 1)])
def test_masked_softmax(y_size, x_size, dim, device, dtype):
    factory_kwargs = {"device": device, "dtype": dtype}
    input = torch.randn(y_size, x_size, **factory_kwargs, requires_grad=True)
    grad_output = torch.randn_like(input)
    mask = build_mask(y_size, x_size, dim, 5).to(device)
    output = trident.MaskedSoftmax(dim).forward(input, mask)
    assert output is not None and output.dtype == dtype
    output.backward(grad_output)
    assert input.grad is not None and input.grad.dtype == dtype

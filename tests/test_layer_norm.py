"""LayerNorm parity (shapes and cases of the reference's tests/test_layer_norm.py, seeded)."""

import pytest
import torch

import trident_b200 as trident
from oracle import torch_oracle
from tests import util

pytestmark = pytest.mark.gpu


# tolerance for fp32 norms: rtol = atol = 1e-5
RTOL = ATOL = 1e-5


@pytest.mark.parametrize("y_size, x_size", [(2000, 4), (4, 2000), (1, 32), (37, 1024), (5, 4096), (3, 12288)])
@pytest.mark.parametrize("affine", ["none", "weight", "bias", "both"])
def test_forward(y_size, x_size, affine, device):
    x = util.randn(y_size, x_size, seed=1)
    w = util.randn(x_size, seed=2) if affine in ("weight", "both") else None
    b = util.randn(x_size, seed=3) if affine in ("bias", "both") else None
    want = torch_oracle.layer_norm(x, (x_size,), w, b)
    got = trident.function.layer_norm(
        x.to(device), (x_size,), None if w is None else w.to(device), None if b is None else b.to(device)
    )
    util.assert_close(got, want, RTOL, ATOL, "layer_norm fwd")


@pytest.mark.parametrize("y_size, x_size", [(2000, 4), (4, 2000), (300, 1024), (33, 4096), (70, 8192)])
@pytest.mark.parametrize("affine", ["none", "both", "weight"])
def test_backward(y_size, x_size, affine, device):
    x = util.randn(y_size, x_size, seed=1)
    dy = util.randn(y_size, x_size, seed=4)
    w = util.randn(x_size, seed=2) if affine in ("weight", "both") else None
    b = util.randn(x_size, seed=3) if affine == "both" else None

    def train(fn, dev):
        i = x.detach().clone().to(dev).requires_grad_(True)
        j = None if w is None else w.detach().clone().to(dev).requires_grad_(True)
        k = None if b is None else b.detach().clone().to(dev).requires_grad_(True)
        fn(i, (x_size,), j, k).backward(dy.to(dev))
        return [t.grad for t in (i, j, k) if t is not None]

    for got, want, name in zip(train(trident.function.layer_norm, device), train(torch_oracle.layer_norm, "cpu"), "xwb"):
        # column sums over many rows: relative tolerance scaled by the row count
        util.assert_close(got, want, 1e-5, 1e-5 * max(1.0, y_size ** 0.5), f"layer_norm grad {name}")


def test_multi_dim_normalized_shape(device):
    x = util.randn(6, 5, 8, 16, seed=5)
    w, b = util.randn(8, 16, seed=6), util.randn(8, 16, seed=7)
    dy = util.randn(6, 5, 8, 16, seed=8)

    def train(fn, dev):
        i, j, k = (t.detach().clone().to(dev).requires_grad_(True) for t in (x, w, b))
        y = fn(i, (8, 16), j, k)
        y.backward(dy.to(dev))
        return y, i.grad, j.grad, k.grad

    for got, want in zip(train(trident.function.layer_norm, device), train(torch_oracle.layer_norm, "cpu")):
        util.assert_close(got, want, 1e-5, 1e-4, "layer_norm nd")


@pytest.mark.parametrize("y_size, x_size", [(1, 32)])
def test_layer_norm(y_size, x_size, device, dtype):
    factory_kwargs = {"device": device, "dtype": dtype}
    input = torch.randn(y_size, x_size, **factory_kwargs, requires_grad=True)
    grad_output = torch.randn_like(input)

    output = trident.LayerNorm(x_size, **factory_kwargs).forward(input)
    assert output is not None and output.dtype == dtype
    output.backward(grad_output)
    assert input.grad is not None and input.grad.dtype == dtype

    module = trident.LayerNorm(x_size, elementwise_affine=False, **factory_kwargs)
    output = module.forward(input)
    assert output is not None and output.dtype == dtype


@pytest.mark.parametrize("dt, atol", [(torch.float16, 2e-3), (torch.bfloat16, 1.6e-2)])
def test_half_precision_values(dt, atol, device):
    x = util.randn(64, 2048, seed=11, dtype=dt)
    w = util.randn(2048, seed=12, dtype=dt, mean=1.0, std=0.1)
    b = util.randn(2048, seed=13, dtype=dt, std=0.1)
    want = torch_oracle.layer_norm(x.float(), (2048,), w.float(), b.float())
    got = trident.function.layer_norm(x.to(device), (2048,), w.to(device), b.to(device))
    # one rounding of an fp32 result to the 16-bit type
    util.assert_half_close(got, want, dt, atol=1e-6, ulps=0.51, what="y")


def test_large_mean_and_outlier(device):
    """Mean and variance come from one pass of sums shifted by a sample of the row: a mean far from
    zero and an outlier in the first position must not cost accuracy."""
    x = util.randn(32, 1024, seed=31) * 0.5 + 200.0
    x[:, 0] = 5.0e3
    w, b = util.randn(1024, seed=32), util.randn(1024, seed=33)
    want = torch.nn.functional.layer_norm(x.double(), (1024,), w.double(), b.double(), 1e-5)
    got = trident.function.layer_norm(x.to(device), (1024,), w.to(device), b.to(device), 1e-5)
    assert torch.allclose(got.cpu().double(), want, rtol=1e-4, atol=1e-4), (got.cpu().double() - want).abs().max()
    ref32 = torch.nn.functional.layer_norm(x, (1024,), w, b, 1e-5)  # torch's own fp32 result as the yardstick
    assert (got.cpu().double() - want).abs().max() <= 4 * (ref32.double() - want).abs().max() + 1e-5

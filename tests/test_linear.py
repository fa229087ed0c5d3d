"""Linear parity (cases of the reference's tests/test_linear.py, seeded, plus 16-bit cases
that exercise the tensor-core kernel)."""

import pytest
import torch

import trident_b200 as trident
from oracle import torch_oracle
from tests import util

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("num_batches, m_size, n_size, k_size", [(2, 512, 512, 100), (1, 70, 33, 129)])
def test_forward(num_batches, m_size, n_size, k_size, device):
    x = util.randn(num_batches, m_size, k_size, seed=1)
    w = util.randn(n_size, k_size, seed=2)
    b = util.randn(n_size, seed=3)
    f = trident.function.linear
    util.assert_close(f(x.to(device), w.to(device)), torch_oracle.linear(x, w), 1e-5, 2e-4, "linear")
    util.assert_close(f(x.to(device), w.to(device), b.to(device)), torch_oracle.linear(x, w, b), 1e-5, 2e-4, "linear+b")

    # permuted (non-contiguous) operands, tests/test_linear.py:33-36
    xp = util.randn(num_batches, k_size, m_size, seed=4).permute(0, 2, 1)
    wp = util.randn(k_size, n_size, seed=5).permute(1, 0)
    got = f(xp.to(device), wp.to(device))
    util.assert_close(got, torch_oracle.linear(xp, wp), 1e-5, 2e-4, "linear permuted")


@pytest.mark.parametrize("num_batches, m_size, n_size, k_size", [(2, 512, 512, 100), (3, 33, 65, 47)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_backward(num_batches, m_size, n_size, k_size, with_bias, device):
    x = util.randn(num_batches, m_size, k_size, seed=1)
    w = util.randn(n_size, k_size, seed=2)
    b = util.randn(n_size, seed=3) if with_bias else None
    dy = util.randn(num_batches, m_size, n_size, seed=4)

    def train(fn, dev):
        i = x.detach().clone().to(dev).requires_grad_(True)
        j = w.detach().clone().to(dev).requires_grad_(True)
        k = None if b is None else b.detach().clone().to(dev).requires_grad_(True)
        fn(i, j, k).backward(dy.to(dev))
        return [t.grad for t in (i, j, k) if t is not None]

    for got, want, name in zip(train(trident.function.linear, device), train(torch_oracle.linear, "cpu"), "xwb"):
        util.assert_close(got, want, 1e-5, 2e-3, f"linear grad {name}")


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize(
    "num_batches, m_size, n_size, k_size",
    [(1, 128, 256, 64), (1, 256, 512, 256), (2, 300, 520, 136), (1, 1024, 768, 1024), (4, 64, 72, 200)],
)
def test_half_forward_backward(num_batches, m_size, n_size, k_size, dt, device):
    """16-bit operands: fp32 accumulation, one rounding. atol 1e-2 on O(1) outputs."""
    x = util.randn(num_batches, m_size, k_size, seed=1, dtype=dt)
    w = util.randn(n_size, k_size, seed=2, dtype=dt, std=k_size ** -0.5)
    b = util.randn(n_size, seed=3, dtype=dt)
    dy = util.randn(num_batches, m_size, n_size, seed=4, dtype=dt, std=n_size ** -0.5)

    def train(fn, dev, up):
        i, j, k = (t.detach().clone().to(dev).to(up).requires_grad_(True) for t in (x, w, b))
        y = fn(i, j, k)
        y.backward(dy.to(dev).to(up))
        return y, i.grad, j.grad, k.grad

    got = train(trident.function.linear, device, dt)
    want = train(torch_oracle.linear, "cpu", torch.float32)
    for g, wnt, name in zip(got, want, ["y", "dx", "dw", "db"]):
        assert g.dtype == dt
        util.assert_half_close(g, wnt, dt, atol=1e-2, ulps=1.0, what=name)


def test_tensor_core_path_is_taken(device):
    from trident_b200 import _lib

    x = util.randn(1, 256, 256, seed=1, dtype=torch.bfloat16, device=device)
    w = util.randn(512, 256, seed=2, dtype=torch.bfloat16, device=device)
    trident.function.linear(x, w)
    assert _lib.last_kernel() == "gemm_tcgen05"


@pytest.mark.parametrize("num_batches, m_size, n_size, k_size", [(1, 16, 32, 16)])
def test_linear(num_batches, m_size, n_size, k_size, device, dtype):
    factory_kwargs = {"device": device, "dtype": dtype}
    input = torch.randn(num_batches, m_size, k_size, **factory_kwargs, requires_grad=True)
    grad_output = torch.randn(num_batches, m_size, n_size, **factory_kwargs)

    output = trident.Linear(k_size, n_size, **factory_kwargs).forward(input)
    assert output is not None and output.dtype == dtype
    output.backward(grad_output)
    assert input.grad is not None and input.grad.dtype == dtype

    output = trident.Linear(k_size, n_size, bias=False, **factory_kwargs).forward(input[0])
    assert output.shape == (m_size, n_size)

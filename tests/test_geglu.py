"""GEGLU parity (cases of the reference's tests/test_geglu.py, seeded)."""

import pytest
import torch

import trident_b200 as trident
from oracle import torch_oracle
from tests import util

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("num_batches, m_size, n_size, k_size", [(2, 16, 32, 128), (3, 50, 66, 70)])
def test_forward(num_batches, m_size, n_size, k_size, device):
    x = util.randn(num_batches, m_size, k_size, seed=1)
    w = util.randn(n_size, k_size, seed=2)
    b = util.randn(n_size, seed=3)
    # the reference tolerates 1e-1 here (tanh kernel vs erf oracle); erf against erf is tight
    util.assert_close(trident.function.geglu(x.to(device), w.to(device)), torch_oracle.geglu(x, w), 1e-5, 2e-4, "geglu")
    util.assert_close(
        trident.function.geglu(x.to(device), w.to(device), b.to(device)), torch_oracle.geglu(x, w, b), 1e-5, 2e-4, "geglu+b"
    )
    got2d = trident.function.geglu(x[0].to(device), w.to(device), b.to(device))
    util.assert_close(got2d, torch_oracle.geglu(x[0], w, b), 1e-5, 2e-4, "geglu 2-D input")


@pytest.mark.parametrize("num_batches, m_size, n_size, k_size", [(2, 16, 32, 128), (3, 50, 66, 70)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_backward(num_batches, m_size, n_size, k_size, with_bias, device):
    x = util.randn(num_batches, m_size, k_size, seed=1)
    w = util.randn(n_size, k_size, seed=2)
    b = util.randn(n_size, seed=3) if with_bias else None
    dy = util.randn(num_batches, m_size, n_size // 2, seed=4)

    def train(fn, dev):
        i = x.detach().clone().to(dev).requires_grad_(True)
        j = w.detach().clone().to(dev).requires_grad_(True)
        k = None if b is None else b.detach().clone().to(dev).requires_grad_(True)
        fn(i, j, k).backward(dy.to(dev))
        return [t.grad for t in (i, j, k) if t is not None]

    for got, want, name in zip(train(trident.function.geglu, device), train(torch_oracle.geglu, "cpu"), "xwb"):
        util.assert_close(got, want, 1e-5, 2e-3, f"geglu grad {name}")


def test_tanh_flavour(device):
    """config.geglu_tanh_approximation reproduces the reference kernel's tanh GELU."""
    x = util.randn(1, 64, 128, seed=1)
    w = util.randn(64, 128, seed=2, std=0.1)
    trident.config.geglu_tanh_approximation = True
    try:
        got = trident.function.geglu(x.to(device), w.to(device))
    finally:
        trident.config.geglu_tanh_approximation = False
    state, gate = torch_oracle.linear(x, w).chunk(2, -1)
    want = state * torch.nn.functional.gelu(gate, approximate="tanh")
    util.assert_close(got, want, 1e-5, 2e-4, "geglu tanh")


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m_size, n_size, k_size", [(256, 512, 256), (300, 1040, 136), (128, 256, 64)])
def test_half_forward_backward(m_size, n_size, k_size, dt, device):
    x = util.randn(1, m_size, k_size, seed=1, dtype=dt)
    w = util.randn(n_size, k_size, seed=2, dtype=dt, std=k_size ** -0.5)
    b = util.randn(n_size, seed=3, dtype=dt, std=0.1)
    dy = util.randn(1, m_size, n_size // 2, seed=4, dtype=dt, std=n_size ** -0.5)

    def train(fn, dev, up):
        i, j, k = (t.detach().clone().to(dev).to(up).requires_grad_(True) for t in (x, w, b))
        y = fn(i, j, k)
        y.backward(dy.to(dev).to(up))
        return y, i.grad, j.grad, k.grad

    got = train(trident.function.geglu, device, dt)
    want = train(torch_oracle.geglu, "cpu", torch.float32)
    for g, wnt, name in zip(got, want, ["y", "dx", "dw", "db"]):
        assert g.dtype == dt
        # atol 1e-2 plus the roundings of the 16-bit chain the eager oracle also has:
        # state_gate, gelu(gate) and the product are each rounded to the 16-bit type
        util.assert_half_close(g, wnt, dt, atol=1e-2, ulps=3.0, what=name)


@pytest.mark.parametrize("num_batches, m_size, n_size, k_size", [(1, 16, 32, 16)])
def test_geglu(num_batches, m_size, n_size, k_size, device, dtype):
    factory_kwargs = {"device": device, "dtype": dtype}
    input = torch.randn(num_batches, m_size, k_size, **factory_kwargs, requires_grad=True)
    grad_output = torch.randn(num_batches, m_size, n_size // 2, **factory_kwargs)

    output = trident.GEGLU(k_size, n_size, **factory_kwargs).forward(input)
    assert output is not None and output.dtype == dtype
    output.backward(grad_output)
    assert input.grad is not None and input.grad.dtype == dtype

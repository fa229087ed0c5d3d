"""Helpers shared by the tests: seeded tensors and comparisons."""

import torch


def seeded(seed):
    g = torch.Generator()
    g.manual_seed(seed)
    return g


def randn(*shape, seed=0, dtype=torch.float32, device="cpu", std=1.0, mean=0.0):
    t = torch.randn(*shape, generator=seeded(seed), dtype=torch.float32) * std + mean
    return t.to(dtype).to(device)


def rand(*shape, seed=0, dtype=torch.float32, device="cpu"):
    return torch.rand(*shape, generator=seeded(seed), dtype=torch.float32).to(dtype).to(device)


def equal(input: torch.Tensor, other: torch.Tensor, eps: float = 1e-02):
    """The reference's own comparison (tests/util.py:18-19): absolute tolerance only."""
    return torch.allclose(input.detach().float().cpu(), other.detach().float().cpu(), rtol=0, atol=eps)


def close(input, other, rtol, atol):
    return torch.allclose(input.detach().float().cpu(), other.detach().float().cpu(), rtol=rtol, atol=atol)


def max_abs(input, other):
    return (input.detach().float().cpu() - other.detach().float().cpu()).abs().max().item()


def violations(input, other, atol):
    d = (input.detach().float().cpu() - other.detach().float().cpu()).abs()
    return (d > atol).float().mean().item()


def ulp_error(input, other, dtype):
    """Largest |input - other| in units of the spacing of `dtype` at |other|."""
    a, b = input.detach().float().cpu(), other.detach().float().cpu()
    mant = {torch.bfloat16: 7, torch.float16: 10, torch.float32: 23}[dtype]
    exp = torch.floor(torch.log2(b.abs().clamp_min(1e-30)))
    ulp = torch.pow(2.0, exp - mant)
    return ((a - b).abs() / ulp).max().item()


def assert_close(got, want, rtol, atol, what=""):
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} != {tuple(want.shape)}"
    ok = close(got, want, rtol, atol)
    assert ok, f"{what}: max abs err {max_abs(got, want):.3e} (rtol={rtol}, atol={atol})"


# Relative size of one unit in the last place of a 16-bit type: an fp32 result rounded once
# to the type is within half of this of the exact value.
ULP = {torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10, torch.float32: 2.0 ** -23}


def assert_half_close(got, want, dtype, atol, ulps=1.0, what="", tiny=0.0):
    """|got - want| <= atol + ulps * ULP[dtype] * |want| (+ tiny for subnormal outputs).

    `want` is the float32 oracle; the ulp term is the rounding of the result to `dtype`,
    which no kernel that returns `dtype` can avoid.
    """
    g, w = got.detach().float().cpu(), want.detach().float().cpu()
    assert g.shape == w.shape, f"{what}: shape {tuple(g.shape)} != {tuple(w.shape)}"
    bound = atol + ulps * ULP[dtype] * w.abs() + tiny
    excess = ((g - w).abs() - bound).max().item()
    assert excess <= 0, f"{what}: exceeds atol={atol} + {ulps} ulp by {excess:.3e} (max abs err {max_abs(g, w):.3e})"

"""The CUDA kernels against the committed golden vectors (tests/golden/*.npz)."""

import os

import numpy as np
import pytest
import torch

import trident_b200 as trident

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
F = trident.function


def load(name, device):
    with np.load(os.path.join(GOLDEN, name + ".npz")) as z:
        return {k: torch.from_numpy(z[k]).to(device) for k in z.files}


def run(fn, leaves, dy):
    leaves = [v.clone().requires_grad_(True) for v in leaves]
    out = fn(*leaves)
    out.backward(dy)
    return [out.detach()] + [v.grad for v in leaves]


def check(got, want, names, rtol=1e-5, atol=1e-5):
    for g, w, n in zip(got, want, names):
        assert torch.allclose(g, w, rtol=rtol, atol=atol), f"{n}: {(g - w).abs().max().item():.3e}"


def test_layer_norm(device):
    g = load("layer_norm", device)
    got = run(lambda i, j, k: F.layer_norm(i, (96,), j, k, 1e-5), [g["x"], g["w"], g["b"]], g["dy"])
    check(got, [g["y"], g["dx"], g["dw"], g["db"]], ["y", "dx", "dw", "db"], atol=2e-5)


@pytest.mark.parametrize("tag", ["full", "half"])
def test_rms_norm(tag, device):
    g = load("rms_norm_" + tag, device)
    p = float(g["p"])
    got = run(lambda i, j, k: F.rms_norm(i, p, j, k, 1e-6), [g["x"], g["w"], g["b"]], g["dy"])
    check(got, [g["y"], g["dx"], g["dw"], g["db"]], ["y", "dx", "dw", "db"], atol=2e-5)


@pytest.mark.parametrize("dim", [0, 1])
def test_softmax(dim, device):
    g = load(f"softmax_dim{dim}", device)
    check(run(lambda i: F.softmax(i, dim), [g["x"]], g["dy"]), [g["y"], g["dx"]], ["y", "dx"])
    g = load(f"masked_softmax_dim{dim}", device)
    check(run(lambda i: F.masked_softmax(i, g["mask"], dim), [g["x"]], g["dy"]), [g["y"], g["dx"]], ["y", "dx"])


def test_linear_and_geglu(device):
    g = load("linear", device)
    got = run(F.linear, [g["x"], g["w"], g["b"]], g["dy"])
    check(got, [g["y"], g["dx"], g["dw"], g["db"]], ["y", "dx", "dw", "db"], atol=1e-4)
    g = load("geglu", device)
    got = run(F.geglu, [g["x"], g["w"], g["b"]], g["dy"])
    check(got, [g["y"], g["dx"], g["dw"], g["db"]], ["y", "dx", "dw", "db"], atol=1e-4)


def test_attention(device):
    g = load("attention_causal", device)
    got = run(lambda a, b, c: F.scaled_dot_product_attention(a, b, c, is_causal=True), [g["q"], g["k"], g["v"]], g["dy"])
    check(got, [g["y"], g["dq"], g["dk"], g["dv"]], ["y", "dq", "dk", "dv"], atol=1e-4)
    g = load("attention_masked", device)
    got = run(lambda a, b, c: F.scaled_dot_product_attention(a, b, c, attn_mask=g["mask"]), [g["q"], g["k"], g["v"]], g["dy"])
    check(got, [g["y"], g["dq"], g["dk"], g["dv"]], ["y", "dq", "dk", "dv"], atol=1e-4)


@pytest.mark.parametrize("dim", [0, 1])
def test_var_mean_and_sum(dim, device):
    g = load(f"var_mean_dim{dim}", device)
    leaf = g["x"].clone().requires_grad_(True)
    var, mean = F.var_mean(leaf, dim, 1)
    torch.autograd.backward([var, mean], [g["gv"], g["gm"]])
    check([var.detach(), mean.detach(), leaf.grad], [g["var"], g["mean"], g["dx"]], ["var", "mean", "dx"], atol=2e-6)
    check([F.sum(g["x"], dim), F.mean(g["x"], dim), F.var(g["x"], dim, 1)], [g["sum"], g["mean"], g["var"]],
          ["sum", "mean", "var"], atol=2e-5)

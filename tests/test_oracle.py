"""CPU checks of the oracle itself: torch eager callables and the float64 numpy
restatement against each other and against the committed golden vectors."""

import glob
import os

import numpy as np
import pytest
import torch

from oracle import numpy_ref, torch_oracle

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    with np.load(os.path.join(GOLDEN, name + ".npz")) as z:
        return {k: z[k] for k in z.files}


def t(a):
    return torch.from_numpy(np.asarray(a))


def near(a, b, tol=2e-5):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    assert a.shape == b.shape
    assert np.max(np.abs(a - b)) <= tol * max(1.0, np.max(np.abs(b))), np.max(np.abs(a - b))


def torch_grads(fn, leaves, dy):
    leaves = [t(v).clone().requires_grad_(True) for v in leaves]
    out = fn(*leaves)
    out.backward(t(dy))
    return out.detach().numpy(), [v.grad.numpy() for v in leaves]


def test_golden_files_present():
    names = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, "*.npz")))
    assert names == [
        "attention_causal", "attention_masked", "geglu", "layer_norm", "linear",
        "masked_softmax_dim0", "masked_softmax_dim1", "rms_norm_full", "rms_norm_half",
        "softmax_dim0", "softmax_dim1", "var_mean_dim0", "var_mean_dim1",
    ]


def test_layer_norm():
    g = load("layer_norm")
    y, (dx, dw, db) = torch_grads(lambda i, j, k: torch_oracle.layer_norm(i, (96,), j, k, 1e-5), [g["x"], g["w"], g["b"]], g["dy"])
    for a, b in ((y, g["y"]), (dx, g["dx"]), (dw, g["dw"]), (db, g["db"])):
        near(a, b, 2e-6)
    yn, _, _ = numpy_ref.layer_norm_fwd(g["x"], g["w"], g["b"], 1e-5)
    dxn, dwn, dbn = numpy_ref.layer_norm_bwd(g["dy"], g["x"], g["w"], 1e-5)
    for a, b in ((yn, g["y"]), (dxn, g["dx"]), (dwn, g["dw"]), (dbn, g["db"])):
        near(a, b)


@pytest.mark.parametrize("tag", ["full", "half"])
def test_rms_norm(tag):
    g = load("rms_norm_" + tag)
    p = float(g["p"])
    y, (dx, dw, db) = torch_grads(lambda i, j, k: torch_oracle.rms_norm(i, p, j, k, 1e-6), [g["x"], g["w"], g["b"]], g["dy"])
    for a, b in ((y, g["y"]), (dx, g["dx"]), (dw, g["dw"]), (db, g["db"])):
        near(a, b, 2e-6)
    yn, _ = numpy_ref.rms_norm_fwd(g["x"], p, g["w"], g["b"], 1e-6)
    dxn, dwn, dbn = numpy_ref.rms_norm_bwd(g["dy"], g["x"], p, g["w"], 1e-6)
    for a, b in ((yn, g["y"]), (dxn, g["dx"]), (dwn, g["dw"]), (dbn, g["db"])):
        near(a, b)


@pytest.mark.parametrize("dim", [0, 1])
@pytest.mark.parametrize("masked", [False, True])
def test_softmax(dim, masked):
    g = load(("masked_softmax" if masked else "softmax") + f"_dim{dim}")
    mask = g["mask"] if masked else None
    if masked:
        fn = lambda i: torch_oracle.masked_softmax(i, t(mask), dim)  # noqa: E731
    else:
        fn = lambda i: torch_oracle.softmax(i, dim)  # noqa: E731
    y, (dx,) = torch_grads(fn, [g["x"]], g["dy"])
    near(y, g["y"], 2e-6)
    near(dx, g["dx"], 2e-6)
    axis = 0 if dim == 0 else -1
    yn = numpy_ref.softmax_fwd(g["x"], mask, axis)
    near(yn, g["y"])
    near(numpy_ref.softmax_bwd(g["dy"], yn, axis), g["dx"])
    if masked:
        assert np.all(g["y"][mask.astype(bool)] == 0)
    near(g["y"].sum(axis=axis), np.ones_like(g["y"].sum(axis=axis)))


def test_linear_and_geglu():
    g = load("linear")
    y, (dx, dw, db) = torch_grads(torch_oracle.linear, [g["x"], g["w"], g["b"]], g["dy"])
    for a, b in ((y, g["y"]), (dx, g["dx"]), (dw, g["dw"]), (db, g["db"])):
        near(a, b, 1e-6)
    near(numpy_ref.linear_fwd(g["x"], g["w"], g["b"]), g["y"])
    for a, b in zip(numpy_ref.linear_bwd(g["dy"], g["x"], g["w"]), (g["dx"], g["dw"], g["db"])):
        near(a, b)
    g = load("geglu")
    y, (dx, dw, db) = torch_grads(torch_oracle.geglu, [g["x"], g["w"], g["b"]], g["dy"])
    for a, b in ((y, g["y"]), (dx, g["dx"]), (dw, g["dw"]), (db, g["db"])):
        near(a, b, 1e-6)
    near(numpy_ref.geglu_fwd(g["x"], g["w"], g["b"])[0], g["y"])
    for a, b in zip(numpy_ref.geglu_bwd(g["dy"], g["x"], g["w"], g["b"]), (g["dx"], g["dw"], g["db"])):
        near(a, b)
    # the tanh flavour of the reference kernel stays within 5e-4 of the erf oracle
    grid = np.linspace(-6, 6, 2001)
    assert np.max(np.abs(numpy_ref.gelu(grid, True) - numpy_ref.gelu(grid, False))) < 5e-4
    # gelu' restatements against a central difference
    h = 1e-5
    for flavour in (False, True):
        fd = (numpy_ref.gelu(grid + h, flavour) - numpy_ref.gelu(grid - h, flavour)) / (2 * h)
        assert np.max(np.abs(fd - numpy_ref.gelu_grad(grid, flavour))) < 1e-6


@pytest.mark.parametrize("name", ["attention_causal", "attention_masked"])
def test_attention(name):
    g = load(name)
    causal = name.endswith("causal")
    mask = None if causal else g["mask"]
    if causal:
        fn = lambda a, b, c: torch_oracle.scaled_dot_product_attention(a, b, c, is_causal=True)  # noqa: E731
    else:
        fn = lambda a, b, c: torch_oracle.scaled_dot_product_attention(a, b, c, attn_mask=t(mask))  # noqa: E731
    y, (dq, dk, dv) = torch_grads(fn, [g["q"], g["k"], g["v"]], g["dy"])
    for a, b in ((y, g["y"]), (dq, g["dq"]), (dk, g["dk"]), (dv, g["dv"])):
        near(a, b, 1e-6)
    yn, lse = numpy_ref.attention_fwd(g["q"], g["k"], g["v"], mask, causal)
    near(yn, g["y"])
    dqn, dkn, dvn, _ = numpy_ref.attention_bwd(g["dy"], g["q"], g["k"], g["v"], mask, causal)
    near(dqn, g["dq"])
    near(dkn, g["dk"])
    near(dvn, g["dv"])
    assert np.all(np.isfinite(lse))


def test_rms_norm_derivative_is_exact():
    """numpy_ref.rms_norm_bwd against a float64 central difference of rms_norm_fwd."""
    rng = np.random.default_rng(0)
    x, w, dy = rng.normal(size=(3, 12)), rng.normal(size=12), rng.normal(size=(3, 12))
    dx, _, _ = numpy_ref.rms_norm_bwd(dy, x, 0.5, w, 1e-3)
    h = 1e-6
    for idx in [(0, 0), (1, 5), (2, 11)]:
        xp, xm = x.copy(), x.copy()
        xp[idx] += h
        xm[idx] -= h
        fd = ((numpy_ref.rms_norm_fwd(xp, 0.5, w, None, 1e-3)[0] - numpy_ref.rms_norm_fwd(xm, 0.5, w, None, 1e-3)[0]) * dy).sum() / (2 * h)
        assert abs(fd - dx[idx]) < 1e-6


@pytest.mark.parametrize("dim", [0, 1])
def test_var_mean(dim):
    g = load(f"var_mean_dim{dim}")
    leaf = t(g["x"]).clone().requires_grad_(True)
    var, mean = torch_oracle.var_mean(leaf, dim, 1)
    torch.autograd.backward([var, mean], [t(g["gv"]), t(g["gm"])])
    for a, b in ((var.detach().numpy(), g["var"]), (mean.detach().numpy(), g["mean"]), (leaf.grad.numpy(), g["dx"])):
        near(a, b, 2e-6)
    total, mean_n, var_n = numpy_ref.var_mean_fwd(g["x"], dim, 1)
    near(total, g["sum"], 2e-5)
    near(mean_n, g["mean"])
    near(var_n, g["var"])
    near(numpy_ref.var_mean_bwd(g["gv"], g["gm"], g["x"], dim, 1), g["dx"])

"""Generates the golden vectors under tests/golden/ from the torch eager oracle.

    python tests/golden/make_golden.py

Each .npz holds seeded float32 inputs, the explicit grad_output and the oracle's outputs
and gradients for one operation at a small shape. The CPU tests check both oracle layers
(torch eager and the float64 numpy restatement) against them; the GPU tests check the
CUDA kernels against them. Regenerating must reproduce the files bit for bit on the same
torch build (the generator is seeded and runs single-threaded).
"""

import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import torch_oracle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def randn(g, *shape, std=1.0, mean=0.0):
    return torch.randn(*shape, generator=g) * std + mean


def grads(fn, leaves, dy):
    leaves = [t.clone().requires_grad_(True) for t in leaves]
    out = fn(*leaves)
    out.backward(dy)
    return out.detach(), [t.grad for t in leaves]


def save(name, **arrays):
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **{k: v.numpy() for k, v in arrays.items()})


def main():
    torch.set_num_threads(1)
    g = torch.Generator()

    g.manual_seed(100)
    x, w, b, dy = randn(g, 24, 96), randn(g, 96, mean=1.0, std=0.1), randn(g, 96, std=0.1), randn(g, 24, 96)
    y, (dx, dw, db) = grads(lambda i, j, k: torch_oracle.layer_norm(i, (96,), j, k, 1e-5), [x, w, b], dy)
    save("layer_norm", x=x, w=w, b=b, dy=dy, y=y, dx=dx, dw=dw, db=db)

    g.manual_seed(101)
    x, w, b, dy = randn(g, 20, 64), randn(g, 64, mean=1.0, std=0.1), randn(g, 64, std=0.1), randn(g, 20, 64)
    for tag, p in (("full", -1.0), ("half", 0.5)):
        y, (dx, dw, db) = grads(lambda i, j, k: torch_oracle.rms_norm(i, p, j, k, 1e-6), [x, w, b], dy)
        save("rms_norm_" + tag, x=x, w=w, b=b, dy=dy, y=y, dx=dx, dw=dw, db=db, p=torch.tensor(p))

    g.manual_seed(102)
    x, dy = randn(g, 12, 200, std=2.0), randn(g, 12, 200)
    mask = (torch.rand(12, 200, generator=g) < 0.3)
    mask[:, 0] = False
    mask[0, :] = False
    for dim in (0, 1):
        y, (dx,) = grads(lambda i: torch_oracle.softmax(i, dim), [x], dy)
        save(f"softmax_dim{dim}", x=x, dy=dy, y=y, dx=dx)
        y, (dx,) = grads(lambda i: torch_oracle.masked_softmax(i, mask, dim), [x], dy)
        save(f"masked_softmax_dim{dim}", x=x, dy=dy, mask=mask.to(torch.uint8), y=y, dx=dx)

    g.manual_seed(103)
    x, w, b, dy = randn(g, 2, 24, 40), randn(g, 48, 40, std=0.2), randn(g, 48, std=0.1), randn(g, 2, 24, 48)
    y, (dx, dw, db) = grads(torch_oracle.linear, [x, w, b], dy)
    save("linear", x=x, w=w, b=b, dy=dy, y=y, dx=dx, dw=dw, db=db)
    dyg = randn(g, 2, 24, 24)
    y, (dx, dw, db) = grads(torch_oracle.geglu, [x, w, b], dyg)
    save("geglu", x=x, w=w, b=b, dy=dyg, y=y, dx=dx, dw=dw, db=db)

    g.manual_seed(104)
    q, k, v, dy = (randn(g, 2, 2, 32, 16) for _ in range(4))
    mask = randn(g, 2, 1, 32, 32)
    drop = torch.rand(2, 1, 32, 32, generator=g) < 0.1
    drop[..., 0] = False
    mask = mask.masked_fill(drop, float("-inf"))
    y, (dq, dk, dv) = grads(lambda a, b_, c: torch_oracle.scaled_dot_product_attention(a, b_, c, is_causal=True), [q, k, v], dy)
    save("attention_causal", q=q, k=k, v=v, dy=dy, y=y, dq=dq, dk=dk, dv=dv)
    y, (dq, dk, dv) = grads(lambda a, b_, c: torch_oracle.scaled_dot_product_attention(a, b_, c, attn_mask=mask), [q, k, v], dy)
    save("attention_masked", q=q, k=k, v=v, dy=dy, mask=mask, y=y, dq=dq, dk=dk, dv=dv)

    g.manual_seed(105)
    x = randn(g, 18, 120, mean=0.5)
    for dim in (0, 1):
        n_out = 120 if dim == 0 else 18
        gv, gm = randn(g, n_out), randn(g, n_out)
        leaf = x.clone().requires_grad_(True)
        var, mean = torch_oracle.var_mean(leaf, dim, 1)
        torch.autograd.backward([var, mean], [gv, gm])
        save(f"var_mean_dim{dim}", x=x, gv=gv, gm=gm, var=var.detach(), mean=mean.detach(), dx=leaf.grad,
             sum=torch_oracle.sum(x, dim))


if __name__ == "__main__":
    main()

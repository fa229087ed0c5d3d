"""The fused RMSNorm -> GEGLU operation against the chain of the two oracle callables
(tests/test_rms_norm.py:22-39 and tests/test_geglu.py:22-24 of the reference) and against this
library's own unfused chain."""

import pytest
import torch

import trident_b200 as trident
from oracle import torch_oracle
from tests import util
from trident_b200 import _lib

pytestmark = pytest.mark.gpu


def _chain(ns, x, p, nw, w, b, eps):
    return ns.geglu(ns.rms_norm(x, p, nw, None, eps), w, b)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows, K, N, p", [(256, 512, 1024, -1.0), (100, 256, 144, 0.5), (512, 4096, 2048, -1.0)])
def test_forward_backward(rows, K, N, p, dt, device):
    x = util.randn(rows, K, seed=1, dtype=dt)
    nw = util.randn(K, seed=2, dtype=dt, mean=1.0, std=0.1)
    w = util.randn(N, K, seed=3, dtype=dt, std=0.05)
    b = util.randn(N, seed=4, dtype=dt, std=0.1)
    dy = util.randn(rows, N // 2, seed=5, dtype=dt)
    eps = 1e-6

    def train(fn, dev, up):
        leaves = [t.detach().clone().to(dev).to(up).requires_grad_(True) for t in (x, nw, w, b)]
        y = fn(*leaves)
        y.backward(dy.to(dev).to(up))
        return [y.detach()] + [t.grad for t in leaves]

    got = train(lambda i, j, k, l: trident.function.rms_norm_geglu(i, p, j, k, l, eps), device, dt)
    if dt != torch.float32 and K % 8 == 0 and N % 16 == 0:
        pass  # (the fused path; which path ran is checked in test_fused_path_is_taken)
    want = train(lambda i, j, k, l: _chain(torch_oracle, i, p, j, k, l, eps), "cpu", torch.float32)
    unfused = train(lambda i, j, k, l: _chain(trident.function, i, p, j, k, l, eps), device, dt)
    names = ["y", "dx", "dnorm_weight", "dweight", "dbias"]
    for g, w_, u, name in zip(got, want, unfused, names):
        assert g.shape == w_.shape and g.dtype == dt, name
        if dt == torch.float32:
            util.assert_close(g, w_, 1e-4, 1e-4 * max(1.0, rows ** 0.5), name)
        else:
            # same bound as the unfused chain is held to: its own distance from the float32 oracle
            # (Frobenius, with a factor of 1.5 and a floor) since both round at different points
            err = (g.float().cpu() - w_).norm() / w_.norm().clamp_min(1e-6)
            base = (u.float().cpu() - w_).norm() / w_.norm().clamp_min(1e-6)
            assert err <= 1.5 * base + 2.0 ** -9, f"{name}: fused {err:.3e} vs unfused {base:.3e}"


def test_fused_path_is_taken_and_folded_weight(device):
    dt = torch.bfloat16
    x = util.randn(512, 1024, seed=1, dtype=dt, device=device)
    nw = util.randn(1024, seed=2, dtype=dt, device=device, mean=1.0, std=0.1)
    w = util.randn(512, 1024, seed=3, dtype=dt, device=device, std=0.05)
    before = _lib.total_launches()
    a = trident.function.rms_norm_geglu(x, -1.0, nw, w, None, 1e-6)
    assert _lib.last_kernel() == "gemm_tcgen05"
    assert _lib.total_launches() - before == 2  # the statistic pass and one GEMM
    b = trident.function.rms_norm_geglu(x, -1.0, nw, w, None, 1e-6, folded_weight=(w * nw).contiguous())
    assert torch.equal(a, b)

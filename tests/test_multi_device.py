"""Two GPUs in one process: the opt-in of each tensor-core kernel to its dynamic shared-memory size
belongs to the (kernel, device) pair, so a process that launches on a second device must set it
there too (the library keeps the "done" state per device ordinal)."""

import pytest
import torch

import trident_b200 as trident
from oracle import torch_oracle
from tests import util

pytestmark = pytest.mark.gpu


def test_tensor_core_kernels_on_a_second_device(device):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible GPUs")
    dt = torch.bfloat16
    q, k, v, dy = (util.randn(1, 2, 256, 128, seed=s, dtype=dt) for s in (1, 2, 3, 4))
    x, w = util.randn(1, 256, 512, seed=5, dtype=dt), util.randn(512, 512, seed=6, dtype=dt, std=0.05)
    want = torch_oracle.scaled_dot_product_attention(q.float(), k.float(), v.float(), is_causal=True)
    want_lin = torch_oracle.linear(x.float(), w.float())
    for index in (0, 1, 0):
        dev = torch.device("cuda", index)
        with torch.cuda.device(dev):
            i, j, l = (t.to(dev).requires_grad_(True) for t in (q, k, v))
            y = trident.function.scaled_dot_product_attention(i, j, l, is_causal=True)
            y.backward(dy.to(dev))
            util.assert_half_close(y, want, dt, atol=1e-2, ulps=1.0, what=f"attention on cuda:{index}")
            assert torch.isfinite(i.grad.float()).all()
            lin = trident.function.linear(x.to(dev), w.to(dev))
            util.assert_half_close(lin, want_lin, dt, atol=1e-2, ulps=1.0, what=f"linear on cuda:{index}")
            gg = trident.function.geglu(x.to(dev), w.to(dev))
            assert torch.isfinite(gg.float()).all()
            from trident_b200 import _lib

            assert _lib.device_status() == 0

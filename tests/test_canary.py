"""Out-of-bounds-write check: every op, forward and backward, with guard regions around each
output and workspace (tests/canary.py). The kernels behind these calls store with plain vector
stores, bulk tensor copies, red.global.add and bulk tensor reduce-adds; a store outside its
buffer lands in a guard margin and fails the call that made it."""

import pytest
import torch

import trident_b200 as trident
from tests import util
from tests.canary import GuardViolation, guards
from workloads import WORKLOADS

pytestmark = pytest.mark.gpu

F = trident.function


def _fb(fn, inputs, dy):
    leaves = [t.detach().clone().requires_grad_(True) if t is not None and t.is_floating_point() else t for t in inputs]
    y = fn(*leaves)
    y.backward(dy)
    return [y.detach()] + [t.grad for t in leaves if t is not None and t.requires_grad]


def test_guard_detects_a_stray_write(device):
    """The checker itself: a write one element past the end of an output is reported."""
    from tests import canary
    from trident_b200 import _lib

    def stray(y, *rest):
        flat = y.view(-1)
        # storage of the guarded view continues into the margin
        torch.as_strided(flat, (flat.numel() + 1,), (1,))[-1] = 1.0

    saved = _lib.softmax_fwd
    try:
        _lib.softmax_fwd = stray
        with guards():
            with pytest.raises(GuardViolation, match="after the buffer"):
                _lib.softmax_fwd(torch.zeros(4, 8, device=device))
    finally:
        _lib.softmax_fwd = saved
    assert canary.GUARD >= 64 * 1024


@pytest.mark.parametrize(
    "name, kw",
    [
        ("layer_norm", {"scale": 8}),
        ("softmax", {"scale": 32}),
        ("masked_softmax", {"scale": 32}),
        ("rms_norm", {"scale": 16}),
        ("geglu", {"scale": 16, "n_scale": 8}),
        ("attention_causal", {"scale": 32, "S": 1024}),
        ("attention_masked", {"scale": 8, "S": 1024}),
        ("var_mean", {"scale": 32}),
    ],
)
def test_workloads_inside_guards(name, kw, device):
    wl = WORKLOADS[name]
    t = wl.make(0, 1, device, **kw)
    plain = wl.step(t)
    with guards() as stats:
        guarded = wl.step(t)
    assert sum(stats.values()) >= 2, stats
    for key in wl.result_keys:
        if key == "dq":  # accumulated with atomic adds: equal up to the order of the additions
            util.assert_half_close(guarded[key], plain[key].float(), torch.bfloat16, atol=1e-3, ulps=1.0, what=key)
        else:
            assert torch.equal(guarded[key], plain[key]), f"{name}.{key} differs under guards"


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows, cols", [(1, 8), (37, 1000), (300, 1024), (5, 4100), (3, 12288), (129, 36)])
def test_row_ops_odd_shapes(rows, cols, dt, device):
    x = util.randn(rows, cols, seed=1, dtype=dt, device=device)
    dy = util.randn(rows, cols, seed=2, dtype=dt, device=device)
    w = util.randn(cols, seed=3, dtype=dt, device=device)
    b = util.randn(cols, seed=4, dtype=dt, device=device)
    mask = util.rand(rows, cols, seed=5, device=device) < 0.2
    mask[:, 0] = False
    with guards() as stats:
        _fb(lambda i, j, k: F.layer_norm(i, (cols,), j, k), [x, w, b], dy)
        _fb(lambda i, j, k: F.rms_norm(i, -1.0, j, k), [x, w, b], dy)
        _fb(lambda i, j: F.rms_norm(i, 0.5, j), [x, w], dy)
        _fb(lambda i: F.softmax(i, 1), [x], dy)
        _fb(lambda i: F.softmax(i, 0), [x], dy)
        _fb(lambda i: F.masked_softmax(i, mask, 1), [x], dy)
        for name in ("sum", "mean", "var"):
            for dim in (0, 1):
                out = getattr(F, name)(x.detach().clone().requires_grad_(True), dim)
                out.backward(torch.ones_like(out))
    assert len(stats) >= 8, stats


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B, M, N, K", [(1, 128, 256, 64), (2, 100, 72, 40), (1, 257, 512, 192), (3, 1, 16, 8)])
def test_linear_and_geglu_odd_shapes(B, M, N, K, dt, device):
    x = util.randn(B, M, K, seed=1, dtype=dt, device=device)
    w = util.randn(N, K, seed=2, dtype=dt, device=device, std=0.1)
    b = util.randn(N, seed=3, dtype=dt, device=device)
    with guards() as stats:
        _fb(F.linear, [x, w, b], util.randn(B, M, N, seed=4, dtype=dt, device=device))
        _fb(F.geglu, [x, w, b], util.randn(B, M, N // 2, seed=5, dtype=dt, device=device))
    assert stats.get("linear_fwd", 0) >= 1 and stats.get("geglu_fwd", 0) >= 1, stats


@pytest.mark.parametrize(
    "B, H, S, D, dt, mode",
    [
        (1, 2, 128, 64, torch.bfloat16, "causal"),
        (2, 3, 512, 64, torch.bfloat16, "mask"),
        (1, 2, 256, 128, torch.float16, "causal"),
        (2, 1, 256, 128, torch.bfloat16, "mask"),
        (1, 3, 1024, 128, torch.bfloat16, "none"),
        (2, 2, 64, 32, torch.float32, "mask_grad"),
        (2, 2, 256, 64, torch.bfloat16, "mask_grad"),   # dense mask gradient written by the tensor-core backward
        (1, 2, 384, 128, torch.float16, "mask_grad"),
        (1, 1, 16, 16, torch.float32, "causal"),
    ],
)
def test_attention_inside_guards(B, H, S, D, dt, mode, device):
    q, k, v, dy = (util.randn(B, H, S, D, seed=s, dtype=dt, device=device) for s in (1, 2, 3, 4))
    with guards() as stats:
        if mode in ("mask", "mask_grad"):
            m = util.randn(B, 1, S, S, seed=5, dtype=dt, device=device)
            if mode == "mask_grad":
                m = m.requires_grad_(True)
            _fb(lambda a, b_, c: F.scaled_dot_product_attention(a, b_, c, attn_mask=m), [q, k, v], dy)
        else:
            causal = mode == "causal"
            _fb(lambda a, b_, c: F.scaled_dot_product_attention(a, b_, c, is_causal=causal), [q, k, v], dy)
    assert stats.get("attention_fwd", 0) == 1 and stats.get("attention_bwd", 0) == 1, stats

"""Both ways the norm backward kernels fold their per-CTA weight/bias gradient rows: inside the
cooperative launch (the default) and in a second finalize kernel (otherwise only taken when the
grid cannot be co-resident). The hook that selects the second path is thread-local, so these
tests call the C ABI on the thread that sets it (autograd would run the backward on its own
worker thread). dx must be bit-equal between the two; dw/db agree with the float64 oracle."""

import pytest
import torch

from tests import util
from trident_b200 import _lib

pytestmark = pytest.mark.gpu


def _ws(nbytes, device):
    return torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=device)


@pytest.mark.parametrize("rows, cols", [(300, 1024), (33, 4096), (2000, 64), (70, 8192)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_layer_norm_bwd_both_paths(rows, cols, dt, device):
    x = util.randn(rows, cols, seed=1, dtype=dt, device=device)
    dy = util.randn(rows, cols, seed=2, dtype=dt, device=device)
    w = util.randn(cols, seed=3, dtype=dt, device=device, mean=1.0, std=0.1)
    y = torch.empty_like(x)
    mean = torch.empty(rows, device=device, dtype=torch.float32)
    rstd = torch.empty_like(mean)
    _lib.layer_norm_fwd(y, mean, rstd, x, w, None, rows, cols, 1e-5)
    outs = {}
    for mode in (True, False):
        old = _lib.set_norm_fused_finalize(mode)
        try:
            dx, dw, db = torch.empty_like(x), torch.empty_like(w), torch.empty_like(w)
            _lib.layer_norm_bwd(dx, dw, db, dy, x, w, mean, rstd, _ws(_lib.layer_norm_bwd_workspace(rows, cols), device),
                                rows, cols)
            outs[mode] = (dx, dw, db)
        finally:
            _lib.set_norm_fused_finalize(old)
    assert torch.equal(outs[True][0], outs[False][0])
    xd, dyd = x.double().cpu(), dy.double().cpu()
    xh = (xd - xd.mean(-1, keepdim=True)) / torch.sqrt(xd.var(-1, unbiased=False, keepdim=True) + 1e-5)
    want_dw, want_db = (dyd * xh).sum(0), dyd.sum(0)
    tol = 1e-5 * max(1.0, rows ** 0.5) if dt == torch.float32 else 0.0
    for mode in (True, False):
        for got, want, name in ((outs[mode][1], want_dw, "dw"), (outs[mode][2], want_db, "db")):
            if dt == torch.float32:
                util.assert_close(got, want.float(), 1e-5, tol, f"{name} fused={mode}")
            else:
                util.assert_half_close(got, want.float(), dt, atol=2e-2, ulps=1.0, what=f"{name} fused={mode}")


@pytest.mark.parametrize("rows, cols, with_bias", [(64, 4096, False), (513, 1024, True), (1000, 16, True)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_rms_norm_bwd_both_paths(rows, cols, with_bias, dt, device):
    x = util.randn(rows, cols, seed=1, dtype=dt, device=device)
    dy = util.randn(rows, cols, seed=2, dtype=dt, device=device)
    w = util.randn(cols, seed=3, dtype=dt, device=device, mean=1.0, std=0.1)
    b = util.randn(cols, seed=4, dtype=dt, device=device) if with_bias else None
    eps = 1e-6
    y = torch.empty_like(x)
    rms = torch.empty(rows, device=device, dtype=torch.float32)
    _lib.rms_norm_fwd(y, rms, x, w, b, rows, cols, cols, 1, cols, eps)
    outs = {}
    for mode in (True, False):
        old = _lib.set_norm_fused_finalize(mode)
        try:
            dx, dw = torch.empty_like(x), torch.empty_like(w)
            db = torch.empty_like(w) if with_bias else None
            _lib.rms_norm_bwd(dx, dw, db, dy, x, w, rms, _ws(_lib.rms_norm_bwd_workspace(rows, cols), device),
                              rows, cols, cols, 1, cols, eps)
            outs[mode] = (dx, dw, db)
        finally:
            _lib.set_norm_fused_finalize(old)
    assert torch.equal(outs[True][0], outs[False][0])
    xd, dyd = x.double().cpu(), dy.double().cpu()
    r = torch.sqrt((xd * xd).mean(-1, keepdim=True))
    want_dw = (dyd * xd / (r + eps)).sum(0)
    want_db = dyd.sum(0)
    for mode in (True, False):
        pairs = [(outs[mode][1], want_dw, "dw")]
        if with_bias:
            pairs.append((outs[mode][2], want_db, "db"))
        for got, want, name in pairs:
            if dt == torch.float32:
                util.assert_close(got, want.float(), 1e-5, 1e-5 * max(1.0, rows ** 0.5), f"{name} fused={mode}")
            else:
                util.assert_half_close(got, want.float(), dt, atol=2e-2, ulps=1.0, what=f"{name} fused={mode}")

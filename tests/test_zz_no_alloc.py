"""The allocation-free LayerNorm backward entry point (tb200_layer_norm_bwd_static).

It serves callers that cannot allocate device memory where they call the library (all of
the GPU already handed to a private arena, or a no-cudaMalloc rule on the request path), so
it takes no workspace and uses the library's built-in scratch array instead. The test calls
it through the C ABI twice in a row and compares with the regular entry point, which gets a
caller-allocated workspace. This file sorts last on purpose: a run that stops at the first
failure has then already exercised every other test.
"""

import pytest
import torch

from trident_b200 import _lib

pytestmark = pytest.mark.gpu


def _problem(rows, cols, dtype, device, seed):
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    x = torch.randn(rows, cols, generator=g).to(dtype).to(device)
    dy = torch.randn(rows, cols, generator=g).to(dtype).to(device)
    w = (torch.randn(cols, generator=g) * 0.1 + 1.0).to(dtype).to(device)
    b = (torch.randn(cols, generator=g) * 0.1).to(dtype).to(device)
    y = torch.empty_like(x)
    mean = torch.empty(rows, device=device, dtype=torch.float32)
    rstd = torch.empty(rows, device=device, dtype=torch.float32)
    _lib.layer_norm_fwd(y, mean, rstd, x, w, b, rows, cols, 1e-5)
    return x, dy, w, mean, rstd


def _regular(x, dy, w, mean, rstd):
    rows, cols = x.shape
    dx, dw, db = torch.empty_like(x), torch.empty_like(w), torch.empty_like(w)
    ws = torch.empty(max(_lib.layer_norm_bwd_workspace(rows, cols), 16), dtype=torch.uint8, device=x.device)
    _lib.layer_norm_bwd(dx, dw, db, dy, x, w, mean, rstd, ws, rows, cols)
    return dx, dw, db


def _static(x, dy, w, mean, rstd):
    rows, cols = x.shape
    dx, dw, db = torch.empty_like(x), torch.empty_like(w), torch.empty_like(w)
    _lib.layer_norm_bwd_static(dx, dw, db, dy, x, w, mean, rstd, rows, cols)
    return dx, dw, db


@pytest.mark.parametrize(
    "rows, cols, dtype",
    [
        (4096, 1024, torch.float32),
        (513, 4096, torch.bfloat16),
        (300, 8192, torch.float16),
        (70, 36, torch.float32),
        # 2048 vectors per row: beyond the grouped kernel, and more rows than the 2 MiB array holds
        # partial rows for (32 of [2, 8192] floats), so the grid is cut down to what fits
        (64, 8192, torch.float32),
    ],
)
def test_matches_regular_entry_point_on_two_calls_in_a_row(rows, cols, dtype, device):
    first = _problem(rows, cols, dtype, device, seed=1)
    second = _problem(rows, cols, dtype, device, seed=2)
    # two calls back to back share the scratch array; the second must not see the first
    got_first = _static(*first)
    got_second = _static(*second)
    want_first = _regular(*first)
    want_second = _regular(*second)
    torch.cuda.synchronize()
    # The two entry points may pick differently shaped kernels (the built-in scratch holds
    # fewer partial rows than a caller's workspace), so row sums and column sums are folded
    # in a different order: they agree to fp32 summation-order accuracy, plus one rounding of
    # the output type (rtol = atol = 1e-5, the column sums scaled by sqrt(rows) as in
    # tests/test_layer_norm.py).
    tol = 1e-5 * max(1.0, rows ** 0.5)
    for got, want in ((got_first, want_first), (got_second, want_second)):
        for g, w_, name in zip(got, want, ("dx", "dweight", "dbias")):
            g32, w32 = g.float(), w_.float()
            ulp = {torch.float32: 0.0, torch.float16: 2.0 ** -10, torch.bfloat16: 2.0 ** -7}[dtype]
            bound = (1e-5 if name == "dx" else tol) + (1e-5 + ulp) * w32.abs()
            assert ((g32 - w32).abs() <= bound).all(), f"{name}: {(g32 - w32).abs().max().item():.3e}"


def test_without_weight_and_bias_gradients(device):
    x, dy, w, mean, rstd = _problem(64, 2048, torch.float32, device, seed=3)
    rows, cols = x.shape
    dx = torch.empty_like(x)
    _lib.layer_norm_bwd_static(dx, None, None, dy, x, w, mean, rstd, rows, cols)
    assert torch.allclose(dx, _regular(x, dy, w, mean, rstd)[0], rtol=1e-5, atol=1e-5)


def test_rejects_rows_wider_than_the_built_in_scratch(device):
    x, dy, w, mean, rstd = _problem(4, 8192 + 8, torch.float32, device, seed=4)
    with pytest.raises(_lib.Tb200Error, match="exceed the built-in scratch"):
        _static(x, dy, w, mean, rstd)


@pytest.mark.parametrize("which", ["weight_only", "bias_only"])
@pytest.mark.parametrize("rows, cols", [(300, 1024), (64, 8192)])
def test_one_column_gradient_only(which, rows, cols, device):
    x, dy, w, mean, rstd = _problem(rows, cols, torch.float32, device, seed=5)
    want = _regular(x, dy, w, mean, rstd)
    dx, g = torch.empty_like(x), torch.empty_like(w)
    if which == "weight_only":
        _lib.layer_norm_bwd_static(dx, g, None, dy, x, w, mean, rstd, rows, cols)
    else:
        _lib.layer_norm_bwd_static(dx, None, g, dy, x, w, mean, rstd, rows, cols)
    tol = 1e-5 * max(1.0, rows ** 0.5)
    assert torch.allclose(dx, want[0], rtol=1e-5, atol=1e-5)
    assert torch.allclose(g, want[1 if which == "weight_only" else 2], rtol=1e-5, atol=tol)


def test_empty_problem_zero_fills_like_the_regular_entry_point(device):
    cols = 256
    dw = torch.full((cols,), 7.0, device=device)
    db = torch.full((cols,), 7.0, device=device)
    stream = torch.cuda.current_stream(dw.device).cuda_stream
    rc = _lib.load().tb200_layer_norm_bwd_static(
        None, dw.data_ptr(), db.data_ptr(), None, None, None, None, None, 0, cols, _lib.dtype_code(dw.dtype), stream
    )
    assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    assert (dw == 0).all() and (db == 0).all()

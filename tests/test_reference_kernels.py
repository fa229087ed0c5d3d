"""This library against the reference's OWN kernels on the same GPU and the same inputs.

baseline/_ref/ (made by baseline/make_ref.py, git-ignored) holds a copy of the reference's
`trident` package patched only where the installed Triton's API differs from the one the
reference was written for; its kernels, tiles and accumulation types are the reference's. The
shapes are those of the reference's tests and benchmarks (tests/test_*.py,
benchmarks/benchmark_attention.py:22-57, benchmarks/benchmark_layer_norm.py:22,40), in float32,
where the reference itself claims agreement with torch to atol = 1e-2, rtol = 0
(tests/util.py:18-19; GEGLU 1e-1 forward and 3e-1 backward, tests/test_geglu.py:32-36). The same
bound is asked of |ours - reference's|.

Attention is only run at sequence lengths of at least the reference's largest tile (64): below
that its kernel loads whole tiles without a bounds check (trident/kernel/attention.py:115,140,148).

The reference autotunes every kernel per shape, which takes minutes for its GEMMs (about three
per Linear / GEGLU shape) and half a minute per attention shape. By default the quick cases run
(the row operations and the reference's own attention test shape, about a minute); setting the
environment variable TB200_REFERENCE_FULL=1 adds Linear, GEGLU and the other attention shapes
(about eight minutes).
"""

import os
import sys

import pytest
import torch

import trident_b200 as ours

pytestmark = pytest.mark.gpu

FULL = os.environ.get("TB200_REFERENCE_FULL", "0") == "1"
slow = pytest.mark.skipif(not FULL, reason="minutes of reference autotuning: set TB200_REFERENCE_FULL=1")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")


@pytest.fixture
def ref(device):
    if not os.path.isdir(os.path.join(REF_DIR, "trident")):
        pytest.skip("baseline/_ref is absent: run `python baseline/make_ref.py` where the reference sources are")
    sys.path.insert(0, REF_DIR)
    try:
        import trident  # cached by Python after the first test
    finally:
        sys.path.remove(REF_DIR)
    return trident


def _fb(fn, leaves, dy):
    ls = [t.detach().clone().requires_grad_(True) for t in leaves]
    y = fn(*ls)
    y.backward(dy)
    return [y.detach()] + [t.grad for t in ls]


def _compare(got, want, atol, what):
    for i, (g, w) in enumerate(zip(got, want)):
        err = (g.float() - w.float()).abs().max().item()
        assert err <= atol, f"{what}[{i}]: |ours - reference's| = {err:.3e} > {atol}"


def _randn(*shape, seed, device):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)).to(device)


@pytest.mark.parametrize("rows, cols", [(5, 32), (4, 2000), (2048, 1280)])
def test_layer_norm(ref, rows, cols, device):
    x, w, b, dy = (_randn(*s, seed=i, device=device) for i, s in enumerate([(rows, cols), (cols,), (cols,), (rows, cols)]))
    got = _fb(lambda i, j, k: ours.function.layer_norm(i, (cols,), j, k, 1e-5), [x, w, b], dy)
    want = _fb(lambda i, j, k: ref.function.layer_norm(i, (cols,), j, k, 1e-5), [x, w, b], dy)
    _compare(got, want, 1e-2, "layer_norm")


@pytest.mark.parametrize("rows, cols, dim", [(2, 512, 0), (3, 1000, 1), (2048, 4096, 1)])
def test_softmax_and_masked_softmax(ref, rows, cols, dim, device):
    x, dy = _randn(rows, cols, seed=1, device=device), _randn(rows, cols, seed=2, device=device)
    _compare(_fb(lambda i: ours.function.softmax(i, dim), [x], dy), _fb(lambda i: ref.function.softmax(i, dim), [x], dy),
             1e-2, "softmax")
    mask = torch.randint(0, 2, (rows, cols), generator=torch.Generator().manual_seed(3)).to(device)
    mask[0, :] = 0
    mask[:, 0] = 0
    _compare(_fb(lambda i: ours.function.masked_softmax(i, mask, dim), [x], dy),
             _fb(lambda i: ref.function.masked_softmax(i, mask, dim), [x], dy), 1e-2, "masked_softmax")


@pytest.mark.parametrize("rows, cols, p", [(1000, 10, 0.5), (10, 1000, 1.0), (512, 4096, -1.0)])
def test_rms_norm(ref, rows, cols, p, device):
    x, w, dy = _randn(rows, cols, seed=1, device=device), _randn(cols, seed=2, device=device), _randn(rows, cols, seed=3, device=device)
    # (the reference's backward uses rms^2 + eps where the exact derivative has (rms + eps)^2,
    # trident/kernel/rms_norm.py:213: with the eps of its tests, 1e-8, the two agree far below 1e-2)
    got = _fb(lambda i, j: ours.function.rms_norm(i, p, j, None, 1e-8), [x, w], dy)
    want = _fb(lambda i, j: ref.function.rms_norm(i, p, j, None, 1e-8), [x, w], dy)
    _compare(got, want, 1e-2, "rms_norm")


@slow
@pytest.mark.parametrize("B, M, N, K", [(2, 16, 32, 128), (2, 512, 512, 100)])
def test_linear_and_geglu(ref, B, M, N, K, device):
    x, w, b = _randn(B, M, K, seed=1, device=device), _randn(N, K, seed=2, device=device), _randn(N, seed=3, device=device)
    dy = _randn(B, M, N, seed=4, device=device)
    _compare(_fb(ours.function.linear, [x, w, b], dy), _fb(ref.function.linear, [x, w, b], dy), 1e-2, "linear")
    dyg = _randn(B, M, N // 2, seed=5, device=device)
    # the reference's kernel uses the tanh approximation of GELU; this library's switch selects the
    # same form (its default is the exact one, the oracle of the reference's test)
    old = ours.config.geglu_tanh_approximation
    ours.config.geglu_tanh_approximation = True
    try:
        got = _fb(ours.function.geglu, [x, w, b], dyg)
    finally:
        ours.config.geglu_tanh_approximation = old
    want = _fb(ref.function.geglu, [x, w, b], dyg)
    _compare(got, want, 1e-2, "geglu")


@pytest.mark.parametrize(
    "B, H, S, D, causal",
    [
        (4, 8, 128, 64, True),
        pytest.param(4, 8, 256, 32, False, marks=slow),
        pytest.param(64, 8, 256, 64, False, marks=slow),
    ],
)
def test_attention(ref, B, H, S, D, causal, device):
    assert S >= 64  # never below the reference's tile size (see the module docstring)
    q = torch.rand(B, H, S, D, generator=torch.Generator().manual_seed(1)).to(device)
    k, v, dy = (_randn(B, H, S, D, seed=s, device=device) for s in (2, 3, 4))
    got = _fb(lambda a, b_, c: ours.function.scaled_dot_product_attention(a, b_, c, is_causal=causal), [q, k, v], dy)
    want = _fb(lambda a, b_, c: ref.function.scaled_dot_product_attention(a, b_, c, is_causal=causal), [q, k, v], dy)
    _compare(got, want, 1e-2, "attention")
    if not causal and B <= 8:
        mask = _randn(B, H, S, S, seed=5, device=device)
        got = _fb(lambda a, b_, c: ours.function.scaled_dot_product_attention(a, b_, c, attn_mask=mask), [q, k, v], dy)
        want = _fb(lambda a, b_, c: ref.function.scaled_dot_product_attention(a, b_, c, attn_mask=mask), [q, k, v], dy)
        _compare(got, want, 1e-2, "attention with mask")

"""Parity at the benchmark configurations (BASELINE.json configs).

Two kinds of checks per configuration:
  * against the CPU oracle on a bounded slice of the full-size problem (whole rows, or whole
    (batch, head) slices, so the slice is itself an exact sub-problem), and
  * size-independent properties on the full-size result (softmax rows sum to one, masked
    positions are exact zeros, normalised rows have zero mean and unit variance, the
    gradients of one (batch, head) slice do not depend on the other slices, finiteness).
Tolerances: fp32 rtol = atol = 1e-5; fp16/bf16 atol 1e-2 plus the rounding of the 16-bit
output (one ulp relative; three for GEGLU's chain of roundings).
"""

import pytest
import torch

import trident_b200 as trident
from oracle import torch_oracle
from tests import util
from workloads import WORKLOADS

pytestmark = pytest.mark.gpu


def _to(tensors, device):
    return {k: v.to(device) for k, v in tensors.items()}


def test_layer_norm_config(device):
    wl = WORKLOADS["layer_norm"]
    t = wl.make(0, 1, device)
    got = wl.step(t)
    want = wl.run(_to(t, "cpu"), torch_oracle)
    util.assert_close(got["y"], want["y"], 1e-5, 1e-5, "y")
    util.assert_close(got["dx"], want["dx"], 1e-5, 1e-5, "dx")
    util.assert_close(got["dw"], want["dw"], 1e-5, 1e-5 * 64, "dw")  # sums over 4096 rows
    util.assert_close(got["db"], want["db"], 1e-5, 1e-5 * 64, "db")
    xhat = (got["y"] - t["b"]) / t["w"]
    assert xhat.mean(-1).abs().max() < 1e-4
    assert (xhat.var(-1, unbiased=False) - 1).abs().max() < 1e-3


@pytest.mark.parametrize("name", ["softmax", "masked_softmax"])
def test_softmax_config(name, device):
    wl = WORKLOADS[name]
    t = wl.make(0, 1, device)
    got = wl.step(t)
    y = got["y"].float()
    assert (y.sum(-1) - 1).abs().max() < 2e-3  # 4096 fp16 roundings per row
    assert torch.isfinite(got["dx"].float()).all()
    # dx sums to zero along a row (up to the fp16 rounding of y and dx)
    assert got["dx"].float().sum(-1).abs().max() < 5e-2
    if "mask" in t:
        assert (got["y"][t["mask"]] == 0).all() and (got["dx"][t["mask"]] == 0).all()
    rows = slice(0, 512)
    sub = {k: v[rows].cpu() for k, v in t.items()}
    ref = wl.run({k: (v.float() if v.is_floating_point() else v) for k, v in sub.items()}, torch_oracle)
    util.assert_half_close(got["y"][rows], ref["y"], torch.float16, atol=0.0, ulps=0.51, what="y", tiny=6e-8)
    y16 = got["y"][rows].float().cpu()
    dy = sub["dy"].float()
    want_dx = y16 * (dy - (y16 * dy).sum(-1, keepdim=True))
    util.assert_half_close(got["dx"][rows], want_dx, torch.float16, atol=1e-7, ulps=0.51, what="dx", tiny=6e-8)


def test_rms_norm_config(device):
    wl = WORKLOADS["rms_norm"]
    t = wl.make(0, 1, device)
    got = wl.step(t)
    f32 = {k: v.float().cpu() for k, v in t.items()}
    want = wl.run(f32, torch_oracle)
    util.assert_half_close(got["y"], want["y"], torch.bfloat16, atol=1e-6, ulps=0.51, what="y")
    util.assert_half_close(got["dx"], want["dx"], torch.bfloat16, atol=1e-5, ulps=0.51, what="dx")
    # dw sums 8192 rows in fp32 and rounds once
    util.assert_half_close(got["dw"], want["dw"], torch.bfloat16, atol=1e-3, ulps=0.51, what="dw")


def test_geglu_config_slice(device):
    """Full K and N of the configuration on 512 of its 8192 rows (dw, db are then the partial
    sums over those rows, which is also what a row shard of a multi-GPU run produces)."""
    wl = WORKLOADS["geglu"]
    t = wl.make(0, 1, device, scale=16)
    got = wl.step(t)
    want = wl.run({k: v.float().cpu() for k, v in t.items()}, torch_oracle)
    # y: atol 1e-2 plus GEGLU's three roundings. The gradients go through d_state_gate, which is
    # rounded to bf16 between the elementwise kernel and the GEMMs (as the 16-bit eager oracle
    # rounds it); against the float32 oracle that rounding random-walks over the reduction
    # (22016 terms for dx, 512 for dw and db), so they are held to a relative error of the
    # whole tensor (Frobenius, 2^-8) and a worst element of 2^-6 of the largest value.
    util.assert_half_close(got["y"], want["y"], torch.bfloat16, atol=1e-2, ulps=3.0, what="y")
    for key in ("dx", "dw", "db"):
        g, w_ = got[key].float().cpu(), want[key].float()
        rel = (g - w_).norm() / w_.norm()
        assert rel < 2.0 ** -8, f"{key}: relative Frobenius error {rel:.3e}"
        assert (g - w_).abs().max() <= 2.0 ** -6 * w_.abs().max(), f"{key}: max abs err {(g - w_).abs().max():.3e}"
    from trident_b200 import _lib

    assert _lib.last_kernel() in ("gemm_tcgen05", "colsum")
    assert _lib.device_status() == 0


def test_geglu_config_full_properties(device):
    """Full configuration: finiteness, and linearity of the backward pass in grad_output."""
    wl = WORKLOADS["geglu"]
    t = wl.make(0, 1, device)
    a = wl.step(t)
    for v in a.values():
        assert torch.isfinite(v.float()).all()
    t2 = dict(t)
    t2["dy"] = t["dy"] * 2
    b = wl.step(t2)
    assert torch.equal(b["y"], a["y"])
    # doubling grad_output doubles every gradient exactly (a power of two commutes with rounding)
    for key in ("dx", "dw", "db"):
        assert torch.equal(b[key], a[key] * 2), key


@pytest.mark.parametrize("name, S", [("attention_causal", 4096), ("attention_masked", 16384)])
def test_attention_config(name, S, device):
    """The configuration's sequence length and head size on a few (batch, head) slices against
    the CPU oracle; and independence of slices on a larger run."""
    wl = WORKLOADS[name]
    small = wl.make(0, 8, device, scale=16, S=S)  # one block: 1 (masked) or 1 (causal) slice
    got = wl.step(small)
    want = wl.run({k: v.float().cpu() for k, v in small.items()}, torch_oracle)
    for key in ("y", "dq", "dk", "dv"):
        util.assert_half_close(got[key], want[key], torch.bfloat16, atol=1e-2, ulps=1.0, what=f"{name} {key}")
    from trident_b200 import _lib

    assert _lib.last_kernel() == "attn_tcgen05" and _lib.device_status() == 0
    # a wider run must reproduce the same slice (dq up to its reduction order)
    wide = wl.make(0, 4, device, scale=16, S=S)  # blocks 0 and 1; block 0 is the slice above
    got_wide = wl.step(wide)
    assert torch.equal(wide["q"][:1, :1], small["q"][:1, :1])
    assert torch.equal(got_wide["y"][:1, :1], got["y"][:1, :1])
    assert torch.equal(got_wide["dk"][:1, :1], got["dk"][:1, :1])
    assert torch.equal(got_wide["dv"][:1, :1], got["dv"][:1, :1])
    util.assert_half_close(got_wide["dq"][:1, :1], got["dq"][:1, :1].float(), torch.bfloat16, atol=1e-3, ulps=1.0,
                           what="dq across runs")


def test_attention_causal_full_config_properties(device):
    wl = WORKLOADS["attention_causal"]
    t = wl.make(0, 1, device)
    assert tuple(t["q"].shape) == (4, 32, 4096, 128)
    out = wl.step(t)
    for v in out.values():
        assert torch.isfinite(v.float()).all()
    # the first query row attends to key 0 only: its output is exactly v[0]
    assert torch.equal(out["y"][:, :, 0], t["v"][:, :, 0])
    # the last key row receives gradient from the last query row only
    from trident_b200 import _lib

    assert _lib.device_status() == 0


def test_attention_masked_full_config_properties(device):
    """BASELINE.json config 4 at full size, [8,16,16384,64] with the [8,1,S,S] mask: everything
    finite, no bounded wait expired, and one (batch, head) slice taken out of the full-size run
    equals the same slice run alone (y, dk, dv bit for bit; dq up to its reduction order), which
    in turn matches the CPU oracle."""
    from trident_b200 import _lib

    wl = WORKLOADS["attention_masked"]
    t = wl.make(0, 1, device)
    assert tuple(t["q"].shape) == (8, 16, 16384, 64) and tuple(t["mask"].shape) == (8, 1, 16384, 16384)
    out = wl.step(t)
    assert _lib.last_kernel() == "attn_tcgen05" and _lib.device_status() == 0
    for name, v in out.items():
        assert torch.isfinite(v.float()).all(), name
    b, h = 5, 11
    alone_in = {k: v[b:b + 1, h:h + 1].contiguous() for k, v in t.items() if k != "mask"}
    alone_in["mask"] = t["mask"][b:b + 1]
    alone = wl.step(alone_in)
    for key in ("y", "dk", "dv"):
        assert torch.equal(out[key][b:b + 1, h:h + 1], alone[key]), f"{key} of slice ({b},{h}) depends on the other slices"
    util.assert_half_close(out["dq"][b:b + 1, h:h + 1], alone["dq"].float(), torch.bfloat16, atol=1e-3, ulps=1.0,
                           what="dq of the slice, full run against alone")
    del out, t
    want = wl.run({k: v.float().cpu() for k, v in alone_in.items()}, torch_oracle)
    for key in ("y", "dq", "dk", "dv"):
        util.assert_half_close(alone[key], want[key], torch.bfloat16, atol=1e-2, ulps=1.0, what=f"slice {key}")
    assert _lib.device_status() == 0

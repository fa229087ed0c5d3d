"""Three figures per 16-bit output and gradient of the bf16 configurations (BASELINE.json configs
2, 3 and 4, on a bounded slice each):

  1. the literal verdict of the reference's comparison, allclose(rtol=0, atol=1e-2)
     (tests/util.py:18-19 of the reference), against the torch eager oracle run in bf16, with the
     fraction of elements that violate it;
  2. the largest error against that oracle in units of the bf16 spacing at the oracle's value
     (over the elements of at least 1/16 of the tensor's largest magnitude);
  3. the error against the torch eager oracle run in float32 (largest and root-mean-square),
     beside the error torch's own bf16 run makes against the same float32 oracle.

A bf16 unit in the last place is 2^-7 relative: 0.0156 at |v| = 2 and 0.125 at |v| = 16, so figure 1
cannot hold for large-magnitude gradients whoever computes them; figures 2 and 3 tell a rounding
difference from a bug. The test asserts figure 3: this library is not further from the float32
oracle than torch's bf16 eager path is. The table is printed (pytest -s) and, when the environment
variable TB200_REPORT_DIR names a directory, written there as tolerance_report.json.
"""

import json
import os

import pytest
import torch

from oracle import torch_oracle
from tests import util
from workloads import WORKLOADS

pytestmark = pytest.mark.gpu

CASES = [
    ("geglu", {"scale": 16}, "x[512,4096] of the 8192 rows, full W[22016,4096]"),
    ("attention_causal", {"scale": 128, "S": 4096}, "one (batch, head) slice [1,1,4096,128]"),
    ("attention_masked", {"scale": 16, "S": 4096}, "one batch, one head, S cut to 4096: [1,1,4096,64] + mask"),
]

_ROWS = []


def _ulps(got, ref):
    """Largest error in units of the bf16 spacing at the oracle's value, over the elements whose
    magnitude is at least 1/16 of the tensor's largest (in units of a near-zero value's spacing
    any absolute error is astronomically large and says nothing)."""
    big = ref.abs() >= ref.abs().max() / 16
    return float(util.ulp_error(got[big], ref[big], torch.bfloat16))


def _figures(got, bf16_ref, f32_ref):
    g, r16, r32 = got.float().cpu(), bf16_ref.float().cpu(), f32_ref.float().cpu()
    d16 = (g - r16).abs()
    ours32, torch32 = (g - r32).abs(), (r16 - r32).abs()
    return {
        "allclose_atol_1e-2": bool((d16 <= 1e-2).all()),
        "violating_fraction": float((d16 > 1e-2).float().mean()),
        "max_abs_vs_bf16_oracle": float(d16.max()),
        "max_ulp_vs_bf16_oracle": _ulps(g, r16),
        "max_abs_vs_f32_oracle": float(ours32.max()),
        "torch_bf16_max_abs_vs_f32_oracle": float(torch32.max()),
        "rms_vs_f32_oracle": float(ours32.pow(2).mean().sqrt()),
        "torch_bf16_rms_vs_f32_oracle": float(torch32.pow(2).mean().sqrt()),
        "max_abs_value": float(r32.abs().max()),
    }


@pytest.mark.parametrize("name, kw, note", CASES, ids=[c[0] for c in CASES])
def test_three_figures(name, kw, note, device):
    wl = WORKLOADS[name]
    t = wl.make(0, 8 if name != "geglu" else 1, device, **kw)
    got = wl.step(t)
    cpu = {k: v.cpu() for k, v in t.items()}
    ref16 = wl.run(cpu, torch_oracle)                                   # torch eager in bf16
    ref32 = wl.run({k: v.float() for k, v in cpu.items()}, torch_oracle)  # torch eager in float32
    for key in wl.result_keys:
        f = _figures(got[key], ref16[key], ref32[key])
        _ROWS.append({"workload": name, "slice": note, "tensor": key, **f})
        print(
            f"{name:17s} {key:3s} allclose(atol=1e-2)={f['allclose_atol_1e-2']!s:5s} "
            f"violating={f['violating_fraction']:.2e} max_ulp={f['max_ulp_vs_bf16_oracle']:.2f} "
            f"vs f32: ours max {f['max_abs_vs_f32_oracle']:.3e} rms {f['rms_vs_f32_oracle']:.3e} | "
            f"torch bf16 max {f['torch_bf16_max_abs_vs_f32_oracle']:.3e} rms {f['torch_bf16_rms_vs_f32_oracle']:.3e} "
            f"(max |v| {f['max_abs_value']:.1f})"
        )
    out_dir = os.environ.get("TB200_REPORT_DIR")
    if out_dir and os.path.isdir(out_dir):
        with open(os.path.join(out_dir, "tolerance_report.json"), "w") as fh:
            json.dump(_ROWS, fh, indent=1)
    # figure 3, asserted: not further from the float32 oracle than torch's own bf16 path
    # (root-mean-square within 10 %, worst element within a factor of two)
    for row in _ROWS:
        if row["workload"] != name:
            continue
        assert row["rms_vs_f32_oracle"] <= 1.10 * row["torch_bf16_rms_vs_f32_oracle"] + 1e-6, row
        assert row["max_abs_vs_f32_oracle"] <= 2.0 * row["torch_bf16_max_abs_vs_f32_oracle"] + 1e-3, row

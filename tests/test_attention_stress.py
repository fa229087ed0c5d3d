"""Repeat runs of the masked D = 64 attention kernels (BASELINE.json config 4's geometry, cut down).

The tensor-core kernels hand shared-memory and tensor-memory buffers between a bulk-copy
producer, the MMA issuer and the softmax / compute warps. A missing fence in such a hand-over
shows as a few wrong rows in a few runs out of many, so these tests repeat the same forward +
backward many times and demand identical bits for y, lse-dependent dk and dv (dq is accumulated
with atomic adds in no fixed order and is compared with a tolerance), plus one comparison with
the CPU oracle. A mismatch is reported with the tensor, the number of differing elements and the
(batch, head, 128-row tile, row, column) of the first one, so that one failing run names the
hand-over to look at. The tests only compare results: a wrong result fails, nothing can fault.
"""

import pytest
import torch

import trident_b200 as trident
from oracle import torch_oracle
from tests import util

pytestmark = pytest.mark.gpu


def _describe_diff(name, got, want):
    diff = (got != want) & ~(torch.isnan(got) & torch.isnan(want))
    n = int(diff.sum())
    if n == 0:
        return None
    idx = diff.nonzero()[0].tolist()
    b, h, s, d = idx
    rows = diff.any(-1)  # [B,H,S]
    tiles = rows.reshape(rows.shape[0], rows.shape[1], -1, 128).any(-1).nonzero().tolist()
    return (
        f"{name}: {n} differing elements in {int(rows.sum())} rows; first at batch {b} head {h} "
        f"tile {s // 128} row {s % 128} column {d} (got {got[b, h, s, d].item()!r}, first run "
        f"{want[b, h, s, d].item()!r}); (batch, head, tile) with differences: {tiles[:12]}"
    )


def _run(q, k, v, dy, mask):
    i, j, l = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    y = trident.function.scaled_dot_product_attention(i, j, l, attn_mask=mask)
    y.backward(dy)
    return {"y": y.detach(), "dq": i.grad, "dk": j.grad, "dv": l.grad}


def _mask(B, S, device, seed):
    drop = torch.rand((B, 1, S, S), generator=torch.Generator(device=device).manual_seed(seed), device=device) < 0.1
    drop[..., 0] = False
    m = torch.zeros((B, 1, S, S), device=device, dtype=torch.bfloat16)
    return m.masked_fill_(drop, float("-inf"))


@pytest.mark.parametrize(
    "B, H, S, repeats",
    [(1, 16, 2048, 120), (2, 1, 16384, 24), (1, 3, 4096, 60)],
    ids=["16heads_S2048", "1head_S16384", "3heads_S4096"],
)
def test_masked_d64_forward_backward_repeats(B, H, S, repeats, device):
    from trident_b200 import _lib

    dt, D = torch.bfloat16, 64
    g = torch.Generator(device=device).manual_seed(1234 + S)
    q, k, v, dy = (torch.randn((B, H, S, D), generator=g, device=device).to(dt) for _ in range(4))
    mask = _mask(B, S, device, 99)
    first = _run(q, k, v, dy, mask)
    assert _lib.last_kernel() == "attn_tcgen05"
    torch.cuda.synchronize()
    problems = []
    for it in range(repeats):
        again = _run(q, k, v, dy, mask)
        for key in ("y", "dk", "dv"):
            msg = _describe_diff(key, again[key], first[key])
            if msg:
                problems.append(f"repeat {it}: {msg}")
        err = (again["dq"].float() - first["dq"].float()).abs()
        bound = 1e-3 + util.ULP[dt] * first["dq"].float().abs()
        if bool((err > bound).any()):
            where = (err > bound).nonzero()[0].tolist()
            problems.append(f"repeat {it}: dq differs beyond its reduction order at {where}, by {err.max().item():.3e}")
        if len(problems) >= 4:
            break
    assert not problems, "\n".join(problems)
    assert _lib.device_status() == 0
    # and the repeated result is the right one: one (batch, head) slice against the CPU oracle
    if S <= 4096:
        sl = (slice(0, 1), slice(H - 1, H))
        cpu = [t[sl].float().cpu().requires_grad_(True) for t in (q, k, v)]
        want_y = torch_oracle.scaled_dot_product_attention(*cpu, attn_mask=mask[:1].float().cpu())
        want_y.backward(dy[sl].float().cpu())
        for key, want in zip(("y", "dq", "dk", "dv"), (want_y, cpu[0].grad, cpu[1].grad, cpu[2].grad)):
            util.assert_half_close(first[key][sl], want, dt, atol=1e-2, ulps=1.0, what=f"stress {key}")

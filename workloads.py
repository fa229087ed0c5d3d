"""Seeded synthetic workloads: the five benchmark configurations, shardable over ranks.

Every workload is split into 8 fixed blocks (rows for the row operations and GEGLU,
batch x head slices for attention). Block i is always generated from seed
`seed * 1000003 + i`, and rank r of a world of w ranks owns blocks [8r/w, 8(r+1)/w), so
the concatenation of all ranks' shards is the same data for every world size. There is
no exchange between ranks: each shard is a complete, independent problem.

`scale` divides the sharded dimension (rows, or batch x heads) so that tests can run a
configuration's exact row width / head size / sequence length on fewer rows or heads.
"""

import math
from dataclasses import dataclass, field
from typing import Callable, Dict, List

import torch

import trident_b200 as trident

NUM_BLOCKS = 8


def owned_blocks(rank: int, world: int) -> range:
    if world < 1 or NUM_BLOCKS % world != 0:
        raise ValueError(f"world size {world} must divide {NUM_BLOCKS}")
    per = NUM_BLOCKS // world
    return range(rank * per, (rank + 1) * per)


_REPLICA = 0


def set_replica(replica: int) -> None:
    """Selects which independent replica of the data `make` generates (weak scaling: rank r
    of a multi-GPU benchmark run works on replica r of the full configuration)."""
    global _REPLICA
    _REPLICA = int(replica)


def _gen(seed: int, block: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed * 1000003 + 10007 * _REPLICA + block)
    return g


def _randn(shape, g, device, dtype, mean=0.0, std=1.0):
    t = torch.randn(shape, generator=g, device=device, dtype=torch.float32)
    if std != 1.0:
        t.mul_(std)
    if mean != 0.0:
        t.add_(mean)
    return t.to(dtype)


@dataclass
class Workload:
    name: str
    config_index: int          # index into BASELINE.json "configs"
    bound: str                 # "hbm" or "tensor"
    dtype: torch.dtype
    seed: int
    describe: str
    make: Callable             # (rank, world, device, scale) -> dict of tensors
    run: Callable              # (tensors, ns) -> dict of results; runs forward + backward with
                               # the functions of namespace `ns` (trident_b200.function here;
                               # tests pass a namespace of reference callables instead)
    work: Callable             # (tensors) -> algorithmic bytes (hbm) or flops (tensor) of the shard
    input_keys: List[str] = field(default_factory=list)   # tensors a step reads from HBM
    result_keys: List[str] = field(default_factory=list)

    def step(self, tensors):
        """Forward + backward through this package's public functional API."""
        return self.run(tensors, trident.function)


def _leaf(t):
    return t.detach().requires_grad_(True)


# ------------------------------------------------------------------------- LayerNorm C1
def _ln_make(rank, world, device, scale=1):
    rows, cols, seed = 4096 // scale, 1024, 0
    per = rows // NUM_BLOCKS
    xs, gs = [], []
    for b in owned_blocks(rank, world):
        g = _gen(seed, b, device)
        xs.append(_randn((per, cols), g, device, torch.float32))
        gs.append(_randn((per, cols), g, device, torch.float32))
    g = _gen(seed, 1000, device)
    return {
        "x": torch.cat(xs), "dy": torch.cat(gs),
        "w": _randn((cols,), g, device, torch.float32, 1.0, 0.1),
        "b": _randn((cols,), g, device, torch.float32, 0.0, 0.1),
    }


def _ln_run(t, fn):
    x, w, b = _leaf(t["x"]), _leaf(t["w"]), _leaf(t["b"])
    y = fn(x, (x.shape[-1],), w, b, 1e-5)
    y.backward(t["dy"])
    return {"y": y.detach(), "dx": x.grad, "dw": w.grad, "db": b.grad}


# ------------------------------------------------------------- Softmax / MaskedSoftmax C2
def _sm_make(rank, world, device, scale=1, masked=False):
    rows, cols, seed = 16384 // scale, 4096, 1
    per = rows // NUM_BLOCKS
    xs, gs, ms = [], [], []
    for b in owned_blocks(rank, world):
        g = _gen(seed, b, device)
        xs.append(_randn((per, cols), g, device, torch.float16, 0.0, 2.0))
        gs.append(_randn((per, cols), g, device, torch.float16))
        if masked:
            m = torch.rand((per, cols), generator=g, device=device) < 0.1
            m[:, 0] = False  # at least one unmasked element per row
            ms.append(m)
    out = {"x": torch.cat(xs), "dy": torch.cat(gs)}
    if masked:
        out["mask"] = torch.cat(ms)
    return out


def _sm_run(t, fn, masked_fn):
    x = _leaf(t["x"])
    y = masked_fn(x, t["mask"], -1) if "mask" in t else fn(x, -1)
    y.backward(t["dy"])
    return {"y": y.detach(), "dx": x.grad}


def _var_mean_run(t, fn):
    x = _leaf(t["x"])
    var, mean = fn(x, -1, 1)
    # the first two columns of the seeded gradient tensor serve as the gradients of the outputs
    torch.autograd.backward([var, mean], [t["dy"][:, 0].contiguous(), t["dy"][:, 1].contiguous()])
    return {"var": var.detach(), "mean": mean.detach(), "dx": x.grad}


# --------------------------------------------------------------------- RMSNorm / GEGLU C3
def _c3_make(rank, world, device, scale=1, with_geglu=False, n_scale=1):
    rows, k, n, seed = 8192 // scale, 4096, 2 * 11008 // n_scale, 2
    per = rows // NUM_BLOCKS
    xs, gs = [], []
    for b in owned_blocks(rank, world):
        g = _gen(seed, b, device)
        xs.append(_randn((per, k), g, device, torch.bfloat16))
        if with_geglu:
            gs.append(_randn((per, n // 2), g, device, torch.bfloat16))
        else:
            gs.append(_randn((per, k), g, device, torch.bfloat16))
    g = _gen(seed, 1000, device)
    out = {"x": torch.cat(xs), "dy": torch.cat(gs)}
    if with_geglu:
        out["w"] = _randn((n, k), g, device, torch.bfloat16, 0.0, 0.02)
        out["b"] = torch.zeros(n, device=device, dtype=torch.bfloat16)
    else:
        out["w"] = _randn((k,), g, device, torch.bfloat16, 1.0, 0.02)
    return out


def _rms_run(t, fn):
    x, w = _leaf(t["x"]), _leaf(t["w"])
    y = fn(x, -1.0, w, None, 1e-6)
    y.backward(t["dy"])
    return {"y": y.detach(), "dx": x.grad, "dw": w.grad}


def _geglu_run(t, fn):
    x, w, b = _leaf(t["x"]), _leaf(t["w"]), _leaf(t["b"])
    y = fn(x, w, b)
    y.backward(t["dy"])
    return {"y": y.detach(), "dx": x.grad, "dw": w.grad, "db": b.grad}


# -------------------------------------------------------------------------- Attention C4/C5
def _attn_make(rank, world, device, scale, B, H, S, D, seed, masked):
    """Blocks are slices of the batch (C5, so that a rank holds only its own mask slabs)
    or of batch x heads folded into the batch dimension (C4)."""
    qs, ks, vs, gs, ms = [], [], [], [], []
    if masked:
        per_b, heads = max(B // NUM_BLOCKS, 1), max(H // scale, 1)
    else:
        # fold: 8 blocks over (B*H) / scale units, each block a [units, 1...] slab
        units = max(B * H // scale // NUM_BLOCKS, 1)
        per_b, heads = 1, units
    for b in owned_blocks(rank, world):
        g = _gen(seed, b, device)
        shape = (per_b, heads, S, D)
        qs.append(_randn(shape, g, device, torch.bfloat16))
        ks.append(_randn(shape, g, device, torch.bfloat16))
        vs.append(_randn(shape, g, device, torch.bfloat16))
        gs.append(_randn(shape, g, device, torch.bfloat16))
        if masked:
            drop = torch.rand((per_b, 1, S, S), generator=g, device=device) < 0.1
            drop[..., 0] = False  # key 0 is always kept
            m = torch.zeros((per_b, 1, S, S), device=device, dtype=torch.bfloat16)
            m.masked_fill_(drop, float("-inf"))
            ms.append(m)
    out = {"q": torch.cat(qs), "k": torch.cat(ks), "v": torch.cat(vs), "dy": torch.cat(gs)}
    if masked:
        out["mask"] = torch.cat(ms)
    else:
        # the (batch, head) units are independent: present them with the configuration's head
        # count when they divide evenly ([4, 32, S, D] for the full causal configuration)
        units = out["q"].shape[0] * out["q"].shape[1]
        if units % H == 0:
            out = {name: t.reshape(units // H, H, S, D) for name, t in out.items()}
    return out


def _attn_run(t, fn, causal):
    q, k, v = _leaf(t["q"]), _leaf(t["k"]), _leaf(t["v"])
    if "mask" in t:
        y = fn(q, k, v, attn_mask=t["mask"])
    else:
        y = fn(q, k, v, is_causal=causal)
    y.backward(t["dy"])
    return {"y": y.detach(), "dq": q.grad, "dk": k.grad, "dv": v.grad}


def _attn_flops(t, causal):
    B, H, S, D = t["q"].shape
    fwd = 4.0 * B * H * S * S * D * (0.5 if causal else 1.0)
    return 3.5 * fwd  # backward counted as 2.5x forward


def _bytes(*tensors):
    return float(sum(x.numel() * x.element_size() for x in tensors))


def build_workloads() -> Dict[str, Workload]:
    w: Dict[str, Workload] = {}
    w["layer_norm"] = Workload(
        "layer_norm", 0, "hbm", torch.float32, 0,
        "LayerNorm fwd+bwd fp32 x[4096,1024], affine, eps 1e-5",
        _ln_make,
        lambda t, ns: _ln_run(t, ns.layer_norm),
        lambda t: 5.0 * _bytes(t["x"]),
        ["x", "dy", "w", "b"], ["y", "dx", "dw", "db"],
    )
    w["softmax"] = Workload(
        "softmax", 1, "hbm", torch.float16, 1,
        "Softmax fwd+bwd fp16 x[16384,4096] ~N(0,2), dim=-1",
        lambda r, n, d, scale=1: _sm_make(r, n, d, scale, False),
        lambda t, ns: _sm_run(t, ns.softmax, ns.masked_softmax),
        lambda t: 5.0 * _bytes(t["x"]),
        ["x", "dy"], ["y", "dx"],
    )
    w["masked_softmax"] = Workload(
        "masked_softmax", 1, "hbm", torch.float16, 1,
        "MaskedSoftmax fwd+bwd fp16 x[16384,4096] ~N(0,2), bool mask p=0.1, dim=-1",
        lambda r, n, d, scale=1: _sm_make(r, n, d, scale, True),
        lambda t, ns: _sm_run(t, ns.softmax, ns.masked_softmax),
        lambda t: 5.0 * _bytes(t["x"]) + _bytes(t["mask"]),
        ["x", "dy", "mask"], ["y", "dx"],
    )
    w["rms_norm"] = Workload(
        "rms_norm", 2, "hbm", torch.bfloat16, 2,
        "RMSNorm fwd+bwd bf16 x[8192,4096], weight ~N(1,0.02), eps 1e-6, p=-1",
        lambda r, n, d, scale=1: _c3_make(r, n, d, scale, False),
        lambda t, ns: _rms_run(t, ns.rms_norm),
        lambda t: 5.0 * _bytes(t["x"]),
        ["x", "dy", "w"], ["y", "dx", "dw"],
    )
    w["geglu"] = Workload(
        "geglu", 2, "tensor", torch.bfloat16, 2,
        "GEGLU fwd+bwd bf16 x[8192,4096], W[22016,4096] ~N(0,0.02), bias zeros",
        lambda r, n, d, scale=1, n_scale=1: _c3_make(r, n, d, scale, True, n_scale),
        lambda t, ns: _geglu_run(t, ns.geglu),
        lambda t: 3.0 * 2.0 * t["x"].shape[0] * t["w"].shape[0] * t["w"].shape[1],
        ["x", "dy", "w", "b"], ["y", "dx", "dw", "db"],
    )
    w["attention_causal"] = Workload(
        "attention_causal", 3, "tensor", torch.bfloat16, 3,
        "causal attention fwd+bwd bf16 q,k,v[4,32,4096,128], scale 1/sqrt(128)",
        lambda r, n, d, scale=1, S=4096: _attn_make(r, n, d, scale, 4, 32, S, 128, 3, False),
        lambda t, ns: _attn_run(t, ns.scaled_dot_product_attention, True),
        lambda t: _attn_flops(t, True),
        ["q", "k", "v", "dy"], ["y", "dq", "dk", "dv"],
    )
    w["attention_masked"] = Workload(
        "attention_masked", 4, "tensor", torch.bfloat16, 4,
        "masked attention fwd+bwd bf16 q,k,v[8,16,16384,64], additive mask [8,1,S,S] 10% -inf, scale 1/8",
        lambda r, n, d, scale=1, S=16384: _attn_make(r, n, d, scale, 8, 16, S, 64, 4, True),
        lambda t, ns: _attn_run(t, ns.scaled_dot_product_attention, False),
        lambda t: _attn_flops(t, False),
        ["q", "k", "v", "dy", "mask"], ["y", "dq", "dk", "dv"],
    )
    # beyond BASELINE.json's configurations: the row reductions on the softmax configuration's input
    w["var_mean"] = Workload(
        "var_mean", -1, "hbm", torch.float16, 1,
        "VarMean fwd+bwd fp16 x[16384,4096] ~N(0,2), dim=-1, correction 1 (not a BASELINE.json config)",
        lambda r, n, d, scale=1: _sm_make(r, n, d, scale, False),
        lambda t, ns: _var_mean_run(t, ns.var_mean),
        lambda t: 3.0 * _bytes(t["x"]),
        ["x", "dy"], ["var", "mean", "dx"],
    )
    return w


WORKLOADS = build_workloads()


def to_device(tensors, device):
    return {k: v.to(device) for k, v in tensors.items()}


def scale_note(scale: int) -> str:
    return "full size" if scale == 1 else f"sharded dimension divided by {scale}"


def roofline_seconds(workload: Workload, work: float, hbm_gbs: float, bf16_tflops: float) -> float:
    """Time the shard would take at the measured peak of the resource that bounds it."""
    return work / (hbm_gbs * 1e9) if workload.bound == "hbm" else work / (bf16_tflops * 1e12)


def sdpa_scale(D: int) -> float:
    return 1.0 / math.sqrt(D)

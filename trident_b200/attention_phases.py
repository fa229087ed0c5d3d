"""Per-phase clock profile of the tcgen05 attention kernels.

`python -m trident_b200.attention_phases [--build-only]` compiles attention_fwd_tc.cu and
attention_bwd_tc.cu with -DTB200_ATTN_PROFILE (the kernels then accumulate clock64()
differences between their synchronisation points, for CTA (0, 0) only), links them with the
regular objects into build/libtb200_phases.so, runs causal attention on q,k,v [1, 8, 4096, 128]
bf16 and prints the average cycles per key tile (forward) or query tile (backward) that each
role (MMA issuer, softmax / compute warps, dQ drain warps) spends in each phase.

The instrumented library is a measuring device, not the product: the clock reads perturb the
kernels by a few percent. Build with --build-only where there is no GPU, run where there is.
"""

import ctypes
import os
import subprocess
import sys

from . import build as _build

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(_build.OBJ_DIR, "libtb200_phases.so")
INSTRUMENTED = ("attention_fwd_tc.cu", "attention_bwd_tc.cu")

FWD_PHASES = {
    0: ("MMA issuer", ["loop top", "wait P(tile 0)", "wait V", "issue P.V(tile 0)", "wait K(next)",
                       "issue Q.K^T(tile 0, next)", "wait P(tile 1)", "issue P.V(tile 1), Q.K^T(tile 1, next)"]),
    1: ("softmax warps, tile 0", ["loop top", "wait S", "load S + maximum", "rescale check", "exp2 + store P",
                                  "store wait + arrive"]),
    2: ("softmax warps, tile 1", ["loop top", "wait S", "load S + maximum", "rescale check", "exp2 + store P",
                                  "store wait + arrive"]),
}
# At D = 64 the issuer's loop is ordered differently (P has columns of its own, the next score
# product of a tile is issued before its P V product).
FWD_PHASES_D64 = dict(FWD_PHASES)
FWD_PHASES_D64[0] = ("MMA issuer", ["issue P.V(tile 1) + loop top", "wait S free(tile 0) + K(next)",
                                    "issue Q.K^T(tile 0, next)", "wait P(tile 0) + V", "issue P.V(tile 0)",
                                    "wait S free(tile 1)", "issue Q.K^T(tile 1, next)", "wait P(tile 1)"])
BWD_PHASES = {
    0: ("MMA issuer", ["wait dQ drained", "issue dP^T", "wait P^T", "issue dV", "wait Q/dO(next)", "issue S^T(next)",
                       "wait dS^T", "issue dK, dQ"]),
    1: ("compute warps", ["A: second load wait (+ loop top)", "wait Q/dO", "wait S^T", "A: load S^T", "A: exp2",
                          "A: barrier", "A: store P^T + arrive", "wait dP^T", "B: load dP^T", "B: dS^T + stores",
                          "B: barrier", "B: store dS^T + arrive"]),
    2: ("dQ drain warps", ["loop top", "wait dQ", "load dQ (+ first reductions) + release", "reductions"]),
}


def build_instrumented():
    """Returns the path of the instrumented library (built next to the regular objects)."""
    _build.build()
    flags = [f for f in _build.NVCC_FLAGS if f not in ("-Xptxas", "-v")]
    objs = []
    for src in _build.SOURCES:
        if src in INSTRUMENTED:
            obj = os.path.join(_build.OBJ_DIR, src.replace(".cu", ".phases.o"))
            cmd = [_build._nvcc(), *flags, "-DTB200_ATTN_PROFILE", "-c", os.path.join(_build.CSRC, src), "-o", obj]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}:\n{res.stderr}")
        else:
            obj = os.path.join(_build.OBJ_DIR, src.replace(".cu", ".o"))
        objs.append(obj)
    res = subprocess.run([_build._nvcc(), "-shared", "-o", LIB, *objs, "-lcudart"], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stderr}")
    return LIB


def _table(title, buf, phases, steps):
    print(title)
    for role, (name, labels) in phases.items():
        vals = [buf[role * 16 + i] / steps for i in range(len(labels))]
        print(f"  {name}: {sum(vals):.0f} cycles per tile")
        for label, v in zip(labels, vals):
            print(f"      {label:44s} {v:8.0f}")


def run(B=1, H=8, S=4096, D=128, causal=True, masked=False):
    import torch

    from . import _lib

    if not os.path.exists(LIB):
        raise RuntimeError(f"{LIB} is missing: run with --build-only first")
    _lib.LIB_PATH = LIB
    lib = _lib.load()
    for fn in (lib.tb200_debug_read_prof_fwd, lib.tb200_debug_read_prof):
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.c_void_p]
    g = torch.Generator(device="cuda")
    g.manual_seed(0)
    q, k, v, dy = [torch.randn(B, H, S, D, device="cuda", dtype=torch.bfloat16, generator=g) for _ in range(4)]
    out, lse = torch.empty_like(q), torch.empty(B, H, S, device="cuda")
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    ws = torch.empty(_lib.attention_bwd_workspace(B, H, S, D, q.dtype), dtype=torch.uint8, device="cuda")
    scale = D ** -0.5
    mask = None
    if masked:  # additive mask broadcast over heads, 10 % -inf, first key never masked
        causal = False
        mask = torch.zeros(B, 1, S, S, device="cuda", dtype=torch.bfloat16)
        mask.masked_fill_(torch.rand(B, 1, S, S, device="cuda", generator=g) < 0.1, float("-inf"))
        mask[..., 0] = 0
    for _ in range(3):
        _lib.attention_fwd(out, lse, q, k, v, mask, causal, scale)
        _lib.attention_bwd(dq, dk, dv, None, dy, q, k, v, out, lse, mask, ws, causal, scale)
    torch.cuda.synchronize()
    buf = (ctypes.c_longlong * 64)()
    tiles = S // 128  # CTA (0, 0) owns the longest row of tiles in both kernels
    lib.tb200_debug_read_prof_fwd(buf)
    _table(f"forward, q,k,v [{B},{H},{S},{D}] bf16, causal={causal}, masked={masked}: CTA (0,0), {tiles} key tiles",
           buf, FWD_PHASES_D64 if D == 64 else FWD_PHASES, tiles)
    lib.tb200_debug_read_prof(buf)
    _table(f"backward, same inputs: CTA (0,0), {tiles} query tiles", buf, BWD_PHASES, tiles)
    print("device status", _lib.device_status(False))


if __name__ == "__main__":
    path = build_instrumented()
    if "--build-only" in sys.argv:
        print(path)
    else:
        if "--masked" in sys.argv:  # the long-sequence configuration's head size and mask, shorter sequence
            run(B=1, H=16, S=4096, D=64, masked=True)
        else:
            run(causal="--full" not in sys.argv)

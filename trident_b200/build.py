"""Builds libtb200.so (the C-ABI kernel library) in-tree with nvcc for sm_100a.

Usage: python -m trident_b200.build [--force] [--verbose]
"""

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "build")
LIB_PATH = os.path.join(HERE, "libtb200.so")

SOURCES = [
    "api.cu",
    "row_norm.cu",
    "softmax.cu",
    "reduce.cu",
    "gemm_simt.cu",
    "gemm_tc.cu",
    "attention_simt.cu",
    "attention_fwd_tc.cu",
    "attention_bwd_tc.cu",
]

NVCC_FLAGS = [
    "-std=c++17",
    "-O3",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas",
    "-v",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _headers():
    out = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    out.append(os.path.join(HERE, "..", "include", "tb200.h"))
    return out


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _compile(src, force, verbose):
    obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
    path = os.path.join(CSRC, src)
    if not force and not _stale(obj, [path] + _headers()):
        return obj, ""
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", path, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{res.stdout}\n{res.stderr}")
    log = res.stderr
    with open(obj + ".ptxas.log", "w") as f:
        f.write(log)
    if verbose:
        sys.stderr.write(log)
    return obj, log


def build(force=False, verbose=False):
    """Compiles every .cu file and links libtb200.so; returns the library path."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as pool:
        results = list(pool.map(lambda s: _compile(s, force, verbose), SOURCES))
    objs = [r[0] for r in results]
    if force or _stale(LIB_PATH, objs):
        cmd = [_nvcc(), "-shared", "-o", LIB_PATH, *objs, "-lcudart", "-Xlinker", "-z,defs"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))

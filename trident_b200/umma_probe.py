"""Throughput probe of tcgen05.mma on its own (a measuring device, not part of the library).

`python -m trident_b200.umma_probe [launches]` compiles csrc/umma_probe.cu into build/umma_probe
and runs it: cycles per instruction for N = 64 / 128 / 256, operands in shared or tensor memory,
idle or busy neighbour warps, and three ways of entering the issuing loop. With a large `launches`
(1500 is about three seconds per configuration) the run is long enough for the power cap to set
the clock; sample `nvidia-smi --query-gpu=clocks.sm,power.draw` beside it. `--build-only` compiles
without running (no GPU needed).
"""

import os
import subprocess
import sys

from . import build as _build

EXE = os.path.join(_build.OBJ_DIR, "umma_probe")


def build_probe():
    os.makedirs(_build.OBJ_DIR, exist_ok=True)
    src = os.path.join(_build.CSRC, "umma_probe.cu")
    cmd = [_build._nvcc(), "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-I", os.path.join(os.path.dirname(_build.CSRC), "..", "include"), "-o", EXE, src]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on umma_probe.cu:\n{res.stderr}")
    return EXE


if __name__ == "__main__":
    exe = build_probe()
    args = [a for a in sys.argv[1:] if a != "--build-only"]
    if "--build-only" in sys.argv:
        print(exe)
    else:
        sys.exit(subprocess.run([exe, *args]).returncode)

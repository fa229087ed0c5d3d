"""Makes baseline/_ref/: a copy of the reference's `trident` package that imports and runs under
the Triton installed in this image (3.6), for timing and comparing the reference's own kernels.

    python baseline/make_ref.py [--source /path/to/reference]

The reference was written against an unpinned Triton of 2023; a handful of call sites no longer
match the current API. The copy is patched at exactly those sites (listed in PATCHES below, each
with the reason) and nowhere else: the kernels' algorithms, tile shapes, launch grids and
accumulation types stay the reference's. `nvtx` (not installed here) is replaced by a no-op
stand-in. The output folder is git-ignored: it holds reference sources and is not part of this
repository; it only travels to the GPU machine next to it.

The copy is used by `bench.py --impl reference` (class "triton") and by
tests/test_reference_kernels.py. Attention at sequence lengths below the reference's tile size is
never run through it: the reference's attention kernel loads whole tiles without a bounds check
(trident/kernel/attention.py:115,140,148), which reads out of bounds there.
"""

import argparse
import os
import re
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

NVTX_STUB = '''"""No-op stand-in for the nvtx package (tracing is off by default in the reference)."""


def push_range(*args, **kwargs):
    return None


def pop_range(*args, **kwargs):
    return None
'''

# (file, pattern, replacement, reason). Patterns are regular expressions; each must match.
PATCHES = [
    (
        "util/util.py",
        r"configs if config\.use_autotune else \[configs\[0\]\], key, prune_configs_by, reset_to_zero, warmup, rep",
        "configs=configs if config.use_autotune else [configs[0]], key=key, prune_configs_by=prune_configs_by, "
        "reset_to_zero=reset_to_zero, warmup=warmup, rep=rep",
        "triton.autotune gained parameters before warmup/rep: pass them by keyword",
    ),
    (
        "language/standard.py",
        r"tl\.dot\(input, other, allow_tf32=use_accelerator, out_dtype=tl\.float16\)\.to\(dtype\)",
        "tl.dot(input, other, allow_tf32=use_accelerator, out_dtype=tl.float32).to(dtype)",
        "tl.dot no longer accepts a float16 accumulator for bfloat16 operands",
    ),
    (
        "language/math/gelu.py",
        r"tl\.math\.tanh\(",
        "_tanh(",
        "tl.math.tanh is gone: tanh(x) = 2 * sigmoid(2x) - 1 (helper added to the file)",
    ),
    (
        "language/combine.py",
        r"tl\.math\.pow\(mean_b - mean_a, 2\.0\)",
        "((mean_b - mean_a) * (mean_b - mean_a))",
        "tl.math.pow is gone",
    ),
    (
        "operation/attention.py",
        r"torch\.random\.seed\(\),",
        "torch.random.seed() & 0x7FFFFFFF,",
        "the launcher no longer truncates a 64-bit Python int passed for a tl.int32 parameter (the dropout seed)",
    ),
]

# applied to every file of the package
GLOBAL_PATCHES = [
    (r"tl\.math\.fast_expf\(", "tl.exp(", "tl.math.fast_expf is gone"),
    (r"tl\.math\.max\(", "tl.maximum(", "tl.math.max is gone"),
]

TANH_HELPER = '''

@triton.jit
def _tanh(x):
    return (2.0 * tl.sigmoid(2.0 * x.to(tl.float32)) - 1.0).to(x.dtype)

'''


def build(source):
    pkg_src = os.path.join(source, "trident")
    if not os.path.isdir(pkg_src):
        raise SystemExit(f"{pkg_src} not found")
    if os.path.isdir(OUT):
        shutil.rmtree(OUT)
    os.makedirs(OUT)
    pkg = os.path.join(OUT, "trident")
    shutil.copytree(pkg_src, pkg, ignore=shutil.ignore_patterns("__pycache__"))
    with open(os.path.join(OUT, "nvtx.py"), "w") as f:
        f.write(NVTX_STUB)
    log = []
    for rel, pattern, repl, why in PATCHES:
        path = os.path.join(pkg, rel)
        text = open(path).read()
        new, n = re.subn(pattern, repl, text)
        if n == 0:
            raise SystemExit(f"patch did not apply: {rel}: {pattern}")
        if rel == "language/math/gelu.py":
            new = new.replace("\n\nclass GELU:", TANH_HELPER + "\nclass GELU:", 1)
        open(path, "w").write(new)
        log.append(f"{rel}: {n} site(s): {why}")
    for root, _, files in os.walk(pkg):
        for name in files:
            if not name.endswith(".py"):
                continue
            path = os.path.join(root, name)
            text = open(path).read()
            new = text
            for pattern, repl, why in GLOBAL_PATCHES:
                new, n = re.subn(pattern, repl, new)
                if n:
                    log.append(f"{os.path.relpath(path, pkg)}: {n} site(s): {why}")
            if new != text:
                open(path, "w").write(new)
    with open(os.path.join(OUT, "PATCHES.txt"), "w") as f:
        f.write("\n".join(log) + "\n")
    return log


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--source", default="/root/reference")
    args = ap.parse_args()
    for line in build(args.source):
        print(line)
    sys.path.insert(0, OUT)
    import trident  # noqa: E402,F401

    print("import trident: ok,", trident.__version__)

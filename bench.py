#!/usr/bin/env python
"""Benchmark of the trident_b200 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one forward + backward pass of a workload (a BASELINE configuration) over one
batch of seeded synthetic input through the public functional API. Rank 0 prints ONE JSON
line. With N > 1 (launched by torch.distributed.run, one rank per GPU) ONE configuration is split
over the ranks (batch x head slices for attention, rows for the row operations and GEGLU; rank r
of w owns blocks [8r/w, 8(r+1)/w) of 8), so the total work is fixed ("scaling": "strong") and
`value` is the whole configuration's work over the slowest rank's device time. Nothing is
exchanged between ranks except the barrier and the max-over-ranks of the device time. The former
measurement, one full-size replica per rank, rides along under the key "weak".

  value     whole-job throughput with inputs resident in HBM; the step is replayed from a
            CUDA graph captured through the public API, timed with CUDA events
  e2e       the same metric through the public API with HOST (pinned) buffers: host->device
            copies of every input and device->host copies of every result inside the timed
            region
  roofline  the dominant kernel alone, timed with CUDA events inside this run
  cpu_baseline  the torch eager CPU oracle on a bounded sample of the same workload

`--impl reference` times the reference's CPU implementation of the path: the torch eager
callables its tests use as oracle (the reference itself has no CPU kernels), on all host cores,
for the --steps / --warmup asked for, on a bounded sample of the same configuration.

The last key of the line, "summary", repeats the main figures of every workload in a compact
form (see "summary_keys").
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

DEFAULT_WORKLOAD = "attention_causal"
L2_BYTES = 126 * 1024 * 1024

# Bounded CPU samples: keyword arguments of Workload.make that shrink the sharded dimension.
CPU_SAMPLE = {
    "layer_norm": ({}, "full configuration"),
    "softmax": ({"scale": 4}, "4096 of 16384 rows"),
    "masked_softmax": ({"scale": 4}, "4096 of 16384 rows"),
    "rms_norm": ({"scale": 4}, "2048 of 8192 rows"),
    "geglu": ({"scale": 32}, "256 of 8192 rows, full weight"),
    "attention_causal": ({"scale": 16}, "8 of 128 (batch, head) slices"),
    "attention_masked": ({"scale": 16, "_world": 8}, "1 of 128 (batch, head) slices, one mask slab"),
    "var_mean": ({"scale": 4}, "4096 of 16384 rows"),
}


_JSON_FD = None


def capture_stdout():
    """Routes everything libraries print on stdout (NCCL's version banner, for one) to stderr, so
    that the only thing on stdout is the one JSON line written by emit()."""
    global _JSON_FD
    if _JSON_FD is None:
        sys.stdout.flush()
        _JSON_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line):
    sys.stdout.flush()
    if _JSON_FD is None:
        print(json.dumps(line), flush=True)
    else:
        os.write(_JSON_FD, (json.dumps(line) + "\n").encode())


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def unit_of(wl):
    return "GB/s" if wl.bound == "hbm" else "TFLOP/s"


def rate(wl, work, seconds):
    return work / seconds / (1e9 if wl.bound == "hbm" else 1e12)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc, self.thread = index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, local, world


def reduce_max(value, world, device):
    if world == 1:
        return value
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def reduce_sum(value, world, device):
    if world == 1:
        return value
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def gather_all(value, world, device):
    if world == 1:
        return [value]
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device=device)
    out = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(out, t)
    return [float(x.item()) for x in out]


def barrier(world):
    if world > 1:
        import torch.distributed as dist

        dist.barrier()


def clone_set(tensors):
    return {k: v.clone() for k, v in tensors.items()}


def set_bytes(wl, tensors):
    return sum(tensors[k].numel() * tensors[k].element_size() for k in wl.input_keys if k in tensors)


def launches_of_one_step(wl, tensors):
    """Kernels the library launches for one forward + backward step (its own counter)."""
    from trident_b200 import _lib

    before = _lib.total_launches()
    wl.step(tensors)
    torch.cuda.synchronize()
    return _lib.total_launches() - before


def time_device(wl, sets, steps, warmup, world, device):
    """Device time of `steps` steps (graph replays rotating over the input sets)."""
    for i in range(max(warmup, 3)):
        wl.step(sets[i % len(sets)])
    torch.cuda.synchronize()
    graphs, mode = [], "cuda_graph"
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for s in sets:
                wl.step(s)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        for s in sets:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                keep = wl.step(s)
            graphs.append((g, keep))
        for g, _ in graphs:
            g.replay()
        torch.cuda.synchronize()
    except Exception as exc:  # capture is an optimisation of the launch path, not of the kernels
        sys.stderr.write(f"[bench] CUDA graph capture failed ({exc!r}); timing eager launches\n")
        graphs, mode = [], "eager"
        torch.cuda.synchronize()

    def one(i):
        if graphs:
            graphs[i % len(graphs)][0].replay()
        else:
            wl.step(sets[i % len(sets)])

    for i in range(max(warmup, 3)):
        one(i)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    barrier(world)
    start.record()
    for i in range(steps):
        one(i)
    stop.record()
    torch.cuda.synchronize()
    barrier(world)
    ms = start.elapsed_time(stop)
    per_rank = gather_all(ms, world, device)
    return max(per_rank) / 1e3, mode, per_rank


def time_e2e(wl, tensors, steps, warmup, world, device):
    """Public API with host buffers: every step copies its inputs from pinned host memory to the
    device, runs forward + backward through trident_b200.function and copies every result back to
    pinned host memory, all inside the timed region. The three phases run on three streams over two
    sets of device buffers, so that the copies of neighbouring steps overlap the compute of this one
    (what a user's input pipeline does); every step still pays for all of its own bytes."""
    host_in = {k: v.cpu().pin_memory() for k, v in tensors.items()}
    nbuf = 2
    dev_in = [{k: torch.empty_like(v, device=device) for k, v in host_in.items()} for _ in range(nbuf)]
    first = wl.step(tensors)
    host_out = [{k: torch.empty_like(v, device="cpu").pin_memory() for k, v in first.items()} for _ in range(nbuf)]
    del first
    h2d = sum(v.numel() * v.element_size() for v in host_in.values())
    d2h = sum(v.numel() * v.element_size() for v in host_out[0].values())
    s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(nbuf)]      # inputs of the slot are on the device
    ev_run = [torch.cuda.Event() for _ in range(nbuf)]     # the step on the slot is done (inputs free)
    ev_out = [torch.cuda.Event() for _ in range(nbuf)]     # results of the slot are on the host
    issued = [False] * nbuf

    def one(i):
        slot = i % nbuf
        with torch.cuda.stream(s_in):
            if issued[slot]:
                s_in.wait_event(ev_run[slot])   # the previous step on this slot has read its inputs
            for k, v in host_in.items():
                dev_in[slot][k].copy_(v, non_blocking=True)
            ev_in[slot].record(s_in)
        with torch.cuda.stream(s_run):
            s_run.wait_event(ev_in[slot])
            res = wl.step(dev_in[slot])
            ev_run[slot].record(s_run)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_run[slot])
            if issued[slot]:
                s_out.wait_event(ev_out[slot])  # (same stream: ordering is implied; kept for clarity)
            for k, v in res.items():
                v.record_stream(s_out)
                host_out[slot][k].copy_(v, non_blocking=True)
            ev_out[slot].record(s_out)
        issued[slot] = True

    def drain():
        for st in (s_in, s_run, s_out):
            st.synchronize()

    cur = torch.cuda.current_stream()
    for st in (s_in, s_run, s_out):
        st.wait_stream(cur)
    for i in range(max(warmup, 3)):
        one(i)
    drain()
    torch.cuda.synchronize()
    barrier(world)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(cur)
    for st in (s_in, s_run, s_out):
        st.wait_event(start)
    for i in range(steps):
        one(i)
    for st in (s_in, s_run, s_out):
        cur.wait_stream(st)
    stop.record(cur)
    torch.cuda.synchronize()
    barrier(world)
    return reduce_max(start.elapsed_time(stop), world, device) / 1e3, h2d, d2h


def ncu_traffic(name):
    """DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of one full-size launch of the
    workload's dominant kernel, from the ncu capture recorded in profiles/traffic.json together with
    the commit the capture was taken at. Bytes still in L2 when the kernel ends are not in it."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    try:
        with open(path) as f:
            rec = json.load(f).get(name)
    except (OSError, ValueError):
        rec = None
    if not rec:
        return None, "not captured"
    return float(rec["bytes_per_launch"]), f"ncu capture of {rec['kernel']} at commit {rec['commit']} ({rec['scaled']})"


def dominant_kernel(wl, tensors):
    """(label, launch closure, algorithmic work per launch) of the workload's dominant kernel,
    called directly through the ctypes binding of the C ABI."""
    from trident_b200 import _lib

    dev = tensors[wl.input_keys[0]].device
    if wl.name in ("softmax", "masked_softmax"):
        x, dy = tensors["x"], tensors["dy"]
        y, dx = torch.empty_like(x), torch.empty_like(x)
        _lib.softmax_fwd(y, x, None, x.shape[0], x.shape[1], x.stride(0), 1)
        return ("softmax_bwd_vec", lambda: _lib.softmax_bwd(dx, dy, y, x.shape[0], x.shape[1], x.stride(0), 1),
                3.0 * x.numel() * x.element_size())
    if wl.name == "var_mean":
        x, dy = tensors["x"], tensors["dy"]
        rows, cols = x.shape
        dx = torch.empty_like(x)
        gv, gm = dy[:, 0].contiguous(), dy[:, 1].contiguous()
        return ("reduce_bwd_vec (var_mean)",
                lambda: _lib.reduce_bwd(dx, gv, gm, x, rows, cols, x.stride(0), 1, "var_mean", 1.0),
                2.0 * x.numel() * x.element_size())
    if wl.name == "layer_norm":
        x, dy, w = tensors["x"], tensors["dy"], tensors["w"]
        rows, cols = x.shape
        y, dx = torch.empty_like(x), torch.empty_like(x)
        mean = torch.empty(rows, device=dev)
        rstd = torch.empty(rows, device=dev)
        dw, db = torch.empty_like(w), torch.empty_like(w)
        ws = torch.empty(_lib.layer_norm_bwd_workspace(rows, cols), dtype=torch.uint8, device=dev)
        _lib.layer_norm_fwd(y, mean, rstd, x, w, tensors["b"], rows, cols, 1e-5)
        return ("norm_bwd_grouped (fused column sums)",
                lambda: _lib.layer_norm_bwd(dx, dw, db, dy, x, w, mean, rstd, ws, rows, cols),
                3.0 * x.numel() * x.element_size())
    if wl.name == "rms_norm":
        x, dy, w = tensors["x"], tensors["dy"], tensors["w"]
        rows, cols = x.shape
        y, dx = torch.empty_like(x), torch.empty_like(x)
        rms = torch.empty(rows, device=dev)
        dw = torch.empty_like(w)
        ws = torch.empty(_lib.rms_norm_bwd_workspace(rows, cols), dtype=torch.uint8, device=dev)
        _lib.rms_norm_fwd(y, rms, x, w, None, rows, cols, cols, 1, cols, 1e-6)
        return ("norm_bwd_grouped (fused column sums)",
                lambda: _lib.rms_norm_bwd(dx, dw, None, dy, x, w, rms, ws, rows, cols, cols, 1, cols, 1e-6),
                3.0 * x.numel() * x.element_size())
    if wl.name == "geglu":
        x, w, b = tensors["x"].unsqueeze(0), tensors["w"], tensors["b"]
        M, K = tensors["x"].shape
        N = w.shape[0]
        out = torch.empty(1, M, N // 2, device=dev, dtype=x.dtype)
        sg = torch.empty(1, M, N, device=dev, dtype=x.dtype)
        return ("geglu_fwd gemm", lambda: _lib.geglu_fwd(out, sg, x, w, b, False, False), 2.0 * M * N * K)
    if wl.name.startswith("attention"):
        q, k, v, dy = tensors["q"], tensors["k"], tensors["v"], tensors["dy"]
        mask = tensors.get("mask")
        causal = mask is None
        B, H, S, D = q.shape
        scale = D ** -0.5
        out = torch.empty_like(q)
        lse = torch.empty(B, H, S, device=dev)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
        ws = torch.empty(_lib.attention_bwd_workspace(B, H, S, D, q.dtype), dtype=torch.uint8, device=dev)
        _lib.attention_fwd(out, lse, q, k, v, mask, causal, scale)
        fwd = 4.0 * B * H * S * S * D * (0.5 if causal else 1.0)
        return ("attention_bwd",
                lambda: _lib.attention_bwd(dq, dk, dv, None, dy, q, k, v, out, lse, mask, ws, causal, scale),
                2.5 * fwd)
    raise KeyError(wl.name)


def time_dominant(wl, sets, steps, warmup):
    """Average duration of the dominant kernel: `steps` back-to-back launches between one pair
    of CUDA events, rotating over input sets whose total size exceeds L2 (so that a launch
    never finds its inputs cached), captured in a CUDA graph to keep launch gaps out."""
    launches, label, work = [], None, None
    for s in sets:
        label, fn, work = dominant_kernel(wl, s)
        launches.append(fn)
    for i in range(max(warmup, 3)):
        launches[i % len(launches)]()
    torch.cuda.synchronize()
    n = max(steps, len(launches))
    graph = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            launches[0]()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(n):
                launches[i % len(launches)]()
        graph.replay()
        torch.cuda.synchronize()
    except Exception as exc:
        sys.stderr.write(f"[bench] dominant-kernel graph capture failed ({exc!r}); eager launches\n")
        graph = None
        torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    if graph is not None:
        graph.replay()
    else:
        for i in range(n):
            launches[i % len(launches)]()
    b.record()
    b.synchronize()
    note = (f"rotating {len(sets)} input sets" if len(sets) > 1 else "inputs exceed L2")
    return label, work, a.elapsed_time(b) / 1e3 / n, note + f"; {n} back-to-back launches"


def cpu_run(wl, steps, warmup):
    """The torch eager CPU oracle on a bounded sample; returns (rate, cores, sample text)."""
    from oracle import torch_oracle

    kw, text = CPU_SAMPLE[wl.name]
    kw = dict(kw)
    world = kw.pop("_world", 1)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    tensors = wl.make(0, world, "cpu", **kw)
    work = wl.work(tensors)
    for _ in range(warmup):
        wl.run(tensors, torch_oracle)
    t0 = time.perf_counter()
    for _ in range(steps):
        wl.run(tensors, torch_oracle)
    dt = (time.perf_counter() - t0) / steps
    return rate(wl, work, dt), cores, text, dt


def config_of(wl, args):
    """The `config` object of the JSON line: the same for this repo's arm and the reference arm
    of one (workload, N) pair. What depends on the arm or on the run sits under "run"."""
    n = args.gpus
    return {
        "workload": wl.describe + ("" if args.scale == 1 else f" [sharded dimension / {args.scale}]"),
        "baseline_config": wl.config_index,
        "l2": "inputs larger than 2x L2, or rotation over input sets whose total is (exact figures under 'run')",
        "shard": ("one GPU, the whole configuration" if n == 1 else
                  f"one configuration split over {n} ranks: blocks [8r/{n}, 8(r+1)/{n}) of 8 to rank r, no exchange"),
    }


# Bounded samples for the reference's own Triton kernels (its attention backward runs one
# program of two warps per (batch, head): 0.25 s per slice at S = 4096).
TRITON_SAMPLE = {
    "attention_causal": ({"scale": 64}, "2 of 128 (batch, head) slices"),
    "attention_masked": ({"scale": 16, "_world": 8}, "1 of 128 (batch, head) slices, one mask slab"),
    "geglu": ({"scale": 4}, "2048 of 8192 rows, full weight"),
}
REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def triton_reference_run(wl, steps, warmup, local):
    """The reference's own kernels (the patched copy under baseline/_ref) on this GPU."""
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device")
    if not os.path.isdir(os.path.join(REF_DIR, "trident")):
        raise RuntimeError("baseline/_ref is absent (python baseline/make_ref.py builds it)")
    sys.path.insert(0, REF_DIR)
    try:
        import trident as reference
    finally:
        sys.path.remove(REF_DIR)
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    kw, text = TRITON_SAMPLE.get(wl.name, ({}, "full configuration"))
    kw = dict(kw)
    world = kw.pop("_world", 1)
    tensors = wl.make(0, world, device, **kw)
    work = wl.work(tensors)
    for _ in range(max(warmup, 1)):  # the first call autotunes and compiles
        wl.run(tensors, reference.function)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        wl.run(tensors, reference.function)
    stop.record()
    torch.cuda.synchronize()
    dt = start.elapsed_time(stop) / 1e3 / steps
    return rate(wl, work, dt), text, dt


def run_reference(args, wl):
    rank, local, world = dist_env()
    if rank != 0:
        return
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    kind, why_cpu = "cpu", None
    if args.reference_kind in ("auto", "triton"):
        try:
            value, text, dt = triton_reference_run(wl, steps, warmup, local)
            kind = "triton"
        except Exception as exc:  # no GPU here, no copy, or the copy fails under this Triton
            why_cpu = f"{type(exc).__name__}: {exc}"[:300]
            if args.reference_kind == "triton":
                emit({"impl": "reference", "unavailable": f"the reference's Triton kernels did not run: {why_cpu}"})
                return
    if kind == "triton":
        emit({
            "impl": "reference", "reference_kind": "triton", "metric": f"{wl.name} fwd+bwd {unit_of(wl)}",
            "value": value, "unit": unit_of(wl), "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
            "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak",
            "vs_baseline": None, "dtype": str(wl.dtype).replace("torch.", ""), "data": "synthetic",
            "config": config_of(wl, args),
            "run": {"sample": text, "what": "the reference's own Triton kernels (copy patched for the installed "
                                            "Triton's API, autotuning on) through trident.function on one GPU; "
                                            "each step is one forward + backward over the sample"},
            "cpu_baseline": {"value": value, "unit": unit_of(wl), "cores": 0, "kind": "reference",
                             "sample": text + "; the reference's own kernels on the same GPU (not a CPU run)"},
            "e2e": {"value": value, "unit": unit_of(wl), "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        })
        return
    value, cores, text, dt = cpu_run(wl, steps, warmup)
    line = {
        "impl": "reference", "metric": f"{wl.name} fwd+bwd {unit_of(wl)}", "value": value, "unit": unit_of(wl),
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None,
        "dtype": str(wl.dtype).replace("torch.", ""), "data": "synthetic",
        "config": config_of(wl, args),
        "reference_kind": "cpu",
        "run": {"sample": text, "what": "torch eager on the host cores (the oracle the reference's tests use); "
                                        "each step is one pass over the sample",
                "why_not_triton": why_cpu},
        "cpu_baseline": {"value": value, "unit": unit_of(wl), "cores": cores, "kind": "port",
                         "sample": text + "; torch eager CPU (the oracle the reference's tests use)"},
        "e2e": {"value": value, "unit": unit_of(wl), "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


def input_sets(wl, tensors):
    """Enough copies of the inputs that a rotation over them never finds a set in L2."""
    nbytes = set_bytes(wl, tensors)
    nsets = 1 if nbytes >= 2 * L2_BYTES else min(64, -(-3 * L2_BYTES // max(nbytes, 1)))
    return [tensors] + [clone_set(tensors) for _ in range(nsets - 1)], nsets, nbytes


def measure(wl, args, rank, world, device, with_cpu, sampler=None):
    from workloads import set_replica

    pk = peaks()
    kw = {"scale": args.scale} if args.scale > 1 else {}
    set_replica(0)
    tensors = wl.make(rank, world, device, **kw)  # this rank's shard of the one configuration
    work_local = wl.work(tensors)
    sets, nsets, nbytes = input_sets(wl, tensors)
    launches = launches_of_one_step(wl, tensors)
    if sampler:
        sampler.start()
    secs, mode, per_rank_ms = time_device(wl, sets, args.steps, args.warmup, world, device)
    clocks = sampler.stop() if sampler else None
    work_total = reduce_sum(work_local, world, device)
    value = rate(wl, work_total * args.steps, secs)
    peak = pk["hbm_gbs"] if wl.bound == "hbm" else pk["bf16_tflops"]
    label, kwork, ksecs, l2note = time_dominant(wl, sets, min(args.steps, 20), args.warmup)
    del sets[1:]
    achieved = rate(wl, kwork, ksecs)
    traffic, traffic_src = ncu_traffic(wl.name)
    if traffic is not None:
        traffic = traffic / args.scale / world
    e2e_steps = max(3, min(args.steps, 20))
    esecs, h2d, d2h = time_e2e(wl, tensors, e2e_steps, 1, world, device)
    e2e_value = rate(wl, work_total * e2e_steps, esecs)
    out = {
        "metric": f"{wl.name} fwd+bwd {unit_of(wl)}", "value": value, "unit": unit_of(wl), "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
        "dtype": str(wl.dtype).replace("torch.", ""), "data": "synthetic",
        "config": config_of(wl, args),
        "run": {"launch": mode,
                "l2": (f"rotating {nsets} input sets ({nsets * nbytes / 2**20:.0f} MiB)" if nsets > 1
                       else f"inputs {nbytes / 2**20:.0f} MiB exceed L2"),
                "per_rank_ms_per_step": [round(m / args.steps, 5) for m in per_rank_ms]},
        "step_frac_of_peak": value / (peak * world),
        "roofline": {"bound": wl.bound, "kernel": label, "achieved": achieved, "peak": peak,
                     "unit": unit_of(wl), "frac": achieved / peak, "traffic": traffic,
                     "traffic_source": traffic_src,
                     "peak_source": pk["source"], "l2": l2note, "seconds_per_launch": ksecs},
        "e2e": {"value": e2e_value, "unit": unit_of(wl), "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "overlap": "copy-in, step and copy-out on three streams over two buffer sets",
                "steps": e2e_steps},
        "gpu_launches": launches * args.steps,
        "gpu_launches_per_step": launches,
    }
    del tensors, sets
    torch.cuda.empty_cache()
    if world > 1:
        # the earlier measurement: every rank runs a full-size replica of its own (per-GPU work fixed)
        set_replica(rank)
        full = wl.make(0, 1, device, **kw)
        set_replica(0)
        fsets, _, _ = input_sets(wl, full)
        wsecs, _, wper = time_device(wl, fsets, args.steps, args.warmup, world, device)
        wwork = reduce_sum(wl.work(full), world, device)
        out["weak"] = {"value": rate(wl, wwork * args.steps, wsecs), "unit": unit_of(wl),
                       "ms_per_step": wsecs / args.steps * 1e3,
                       "what": f"each of {world} ranks runs one full-size replica (replica = rank)"}
        del full, fsets
        torch.cuda.empty_cache()
    if clocks is not None:
        out["clocks"] = clocks
    if with_cpu:
        v, cores, text, _ = cpu_run(wl, 2, 1)
        out["cpu_baseline"] = {"value": v, "unit": unit_of(wl), "cores": cores, "kind": "port",
                               "sample": text + "; torch eager CPU (the oracle the reference's tests use)"}
    return out


SUMMARY_KEYS = ["value", "ms_per_step", "step_frac_of_peak", "roofline.frac", "e2e.value", "cpu_baseline.value"]


def summary_row(m):
    def sig(x):
        return None if x is None else float(f"{x:.4g}")

    return [sig(m.get("value")), sig(m.get("ms_per_step")), sig(m.get("step_frac_of_peak")),
            sig(m.get("roofline", {}).get("frac")), sig(m.get("e2e", {}).get("value")),
            sig(m.get("cpu_baseline", {}).get("value"))]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--reference-kind", default="auto", choices=["auto", "triton", "cpu"],
                    help="--impl reference: the reference's own Triton kernels on the GPU (a patched copy under "
                         "baseline/_ref; 'auto' takes them when they run) or torch eager on the host cores")
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--scale", type=int, default=1,
                    help="divide the sharded dimension (rows, batch x heads) by this: small cases for profiling")
    ap.add_argument("--others", default="auto",
                    help="comma list of further workloads reported under 'workloads' (auto: all of them; "
                         "'none' to skip)")
    args = ap.parse_args()

    rank, local, world = dist_env()
    if not (args.gpus > 1 and world == 1):
        capture_stdout()
    if args.gpus > 1 and world == 1:
        os.execvp(sys.executable, [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                                   f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1",
                                   "--master-port", os.environ.get("MASTER_PORT", "29533"), __file__] + sys.argv[1:])

    from workloads import WORKLOADS

    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, wl)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
    from trident_b200 import _lib

    _lib.load()
    sampler = ClockSampler(local) if rank == 0 else None
    line = measure(wl, args, rank, world, device, with_cpu=(rank == 0 and world == 1), sampler=sampler)
    others = args.others
    if others == "auto":
        others = ",".join(n for n in WORKLOADS if n != wl.name)
    extra = {}
    summary = {wl.name: summary_row(line)}
    if others != "none":
        for name in [n for n in others.split(",") if n]:
            try:
                sub = measure(WORKLOADS[name], args, rank, world, device, with_cpu=(rank == 0 and world == 1))
                extra[name] = {k: sub[k] for k in ("value", "unit", "ms_per_step", "step_frac_of_peak", "roofline",
                                                   "e2e", "gpu_launches_per_step", "dtype", "run", "weak") if k in sub}
                if "cpu_baseline" in sub:
                    extra[name]["cpu_baseline"] = sub["cpu_baseline"]
                extra[name]["config"] = sub["config"]["workload"]
                summary[name] = summary_row(sub)
            except Exception as exc:
                extra[name] = {"error": repr(exc)}
                if world > 1:
                    raise  # a rank that left a collective half way would hang the others
            torch.cuda.empty_cache()
    if extra:
        line["workloads"] = extra
    # last on the line, so that it survives a truncated record
    line["summary_keys"] = SUMMARY_KEYS
    line["summary"] = summary
    if rank == 0:
        emit(line)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


if __name__ == "__main__":
    main()

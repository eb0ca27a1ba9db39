#!/usr/bin/env python
"""Benchmark of the b200 backend: HBM GB/s against the roofline and tokens/s per op.

    python bench.py [--gpus N] [--steps K] [--warmup W]            # the CUDA backend
    python bench.py --impl reference [--steps K] [--warmup W]      # the reference's CPU path
    torchrun --nproc-per-node N ... bench.py --gpus N ...          # one process per GPU

Headline (the JSON line's `value`): tokens/s of the fused residual-add + RMSNorm
configuration (bf16, x and residual [16384, 8192]).  A step is one launch of the
op over one batch.  With N GPUs every rank runs the full configuration on its
own tokens (token-sharded data parallel, no collective on the data path), so
the job processes N batches per step: weak scaling.

The same line also carries, under `per_op`, achieved GB/s, the fraction of the
measured HBM peak and tokens/s for all five configurations (RMSNorm fp32,
add+RMSNorm bf16, rotary q/k bf16, SwiGLU bf16, MoE route/index/permute/unpermute),
with the five fractions repeated compactly in `roofline.per_config_frac_of_measured`;
beside them the incumbents on the same GPU (PyTorch eager, and popcorn's own CUDA
SwiGLU and Triton rotary kernels from the unmodified package under baseline/_ref).
With N > 1 GPUs `strong_scaling` times every configuration on 1/N of its tokens
per GPU (max over ranks, every rank's time listed) and the expert-parallel MoE
exchange is timed and checked for bit-equality with the single-GPU chain
(`per_op.moe_bf16_expert_parallel_*.ep_check`).

`--impl reference` runs popcorn's registered PyTorch reference of the headline op
from the unmodified package on the host cores, one full configuration per step.

Timing: CUDA events on the launching stream (torch's current stream), warm-up
first, a device synchronize and a barrier on both sides, max over ranks.  Every
timed launch streams more bytes than the 126 MB L2 holds; configurations whose
footprint is close to L2 rotate through disjoint buffer sets.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))

FALLBACK_HBM_GBS = 6650.0  # used only when MEASURED_PEAKS.json is absent
SPEC_HBM_GBS = 8000.0
L2_BYTES = 126 * 1024 * 1024

HEADLINE_PROFILE = REPO / "profiles" / "rms_rows_kernel_add_rms_norm_bf16.md"


def profiled_traffic_bytes() -> int | None:
    """DRAM bytes (read + write) per launch of the headline kernel at the full configuration, from the line
    `dram_bytes_per_launch: <n>` of the committed ncu summary; None when the summary or the line is missing."""
    import re

    try:
        found = re.search(r"^dram_bytes_per_launch:\s*([0-9_,]+)", HEADLINE_PROFILE.read_text(), re.MULTILINE)
    except OSError:
        return None
    return int(found.group(1).replace(",", "").replace("_", "")) if found else None


def headline_config(tokens: int) -> dict:
    """The `config` object of the JSON line; both arms print the same one."""
    return {
        "workload": f"add_rms_norm bf16 x,residual [{tokens}, 8192], weight [8192], eps 1e-5 (benchmark configuration 2), per GPU",
        "sharding": "tokens, one full batch per GPU, no collective", "l2": "inputs_larger_than_L2 (1 GiB streamed per launch)",
        "timing": "CUDA events on the launching stream, max over ranks",
    }


def measured_peak() -> tuple[float, str]:
    path = REPO / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return FALLBACK_HBM_GBS, "fallback"


# ------------------------------------------------------------------ clocks --

class ClockSampler:
    """nvidia-smi sampling in the background; only reads, never sets, GPU state."""

    FIELDS = "timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown," \
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int) -> None:
        self.proc = None
        self.windows: list[tuple[float, float]] = []
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
        except OSError:
            self.proc = None

    def mark(self, start: float, end: float) -> None:
        self.windows.append((start, end))

    def finish(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        import datetime

        clocks, max_clocks, power, reasons = [], [], [], set()
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 8:
                continue
            try:
                stamp = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                sm, sm_max, watts = float(parts[1]), float(parts[2]), float(parts[3])
            except ValueError:
                continue
            if self.windows and not any(lo <= stamp <= hi for lo, hi in self.windows):
                continue
            clocks.append(sm)
            max_clocks.append(sm_max)
            power.append(watts)
            for name, flag in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[4:]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples inside the timed windows"]}
        return {"sm_mhz": statistics.median(clocks), "sm_max_mhz": max(max_clocks), "power_w_max": max(power),
                "samples": len(clocks), "reasons": sorted(reasons)}


# ------------------------------------------------------------- op runners --

def make_runner(workload, device):
    """Returns (run, n_buffer_sets): `run(i)` enqueues one launch on buffer set i straight through the
    C ABI, with outputs allocated up front, so the timed loop holds no allocation and no tensor bookkeeping."""
    import ctypes

    from popcorn_b200 import _lib

    w = workload
    lib = _lib.library()
    footprint = sum(w.algorithmic_bytes.values())
    nsets = max(1, min(8, -(-4 * L2_BYTES // max(footprint, 1))))
    sets = [{k: v.to(device).clone() for k, v in w.inputs.items()} for _ in range(nsets)]
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    keep = [sets]

    def bind(name, arg_sets):
        fn = getattr(lib, name)

        def run(i: int) -> None:
            status = fn(*arg_sets[i % nsets])
            if status != 0:
                raise _lib.B200Error(name, status, lib.b200_status_string(status).decode(), lib.b200_last_error().decode())

        run.keep = keep  # the buffers live as long as the closure
        return run, nsets

    if w.name == "rms_norm":
        rows, cols = sets[0]["x"].shape
        outs = [torch.empty_like(s["x"]) for s in sets]
        keep.append(outs)
        return bind("b200_rms_norm", [(p(s["x"]), p(sets[0]["weight"]), ctypes.c_void_p(0), p(o), rows, cols, cols, cols,
                                       _lib.F32, w.args["eps"], stream) for s, o in zip(sets, outs)])
    if w.name == "add_rms_norm":
        rows, cols = sets[0]["x"].shape
        outs = [(torch.empty_like(s["x"]), torch.empty_like(s["x"])) for s in sets]
        keep.append(outs)
        return bind("b200_add_rms_norm", [(p(s["x"]), p(s["residual"]), p(sets[0]["weight"]), p(o[0]), p(o[1]), rows, cols,
                                           cols, cols, cols, cols, _lib.BF16, w.args["eps"], w.args["offset"], stream)
                                          for s, o in zip(sets, outs)])
    if w.name == "rotary_embedding":
        b, sq, hq, d = sets[0]["q"].shape
        hk = sets[0]["k"].shape[2]
        return bind("b200_rope_qk", [(p(s["q"]), p(s["k"]), p(sets[0]["cos"]), p(sets[0]["sin"]), b, sq, hq, hk, d, d // 2,
                                      sq * hq * d, hq * d, d, sq * hk * d, hk * d, d, _lib.BF16, _lib.F32, 0, stream) for s in sets])
    if w.name == "rope":
        b, hq, sq, d = sets[0]["q"].shape
        hk = sets[0]["k"].shape[1]
        outs = [(torch.empty_like(s["q"]), torch.empty_like(s["k"])) for s in sets]
        keep.append(outs)
        return bind("b200_rope_paired", [(p(s["q"]), p(s["k"]), p(sets[0]["cos"]), p(sets[0]["sin"]), p(o[0]), p(o[1]), b, hq, hk, sq, d, 1,
                                          hq * sq * d, sq * d, d, hk * sq * d, sq * d, d, hq * sq * d, sq * d, d, hk * sq * d, sq * d, d,
                                          _lib.BF16, stream) for s, o in zip(sets, outs)])
    if w.name == "swiglu":
        rows, cols = sets[0]["gate_up"].shape[0], w.args["cols"]
        outs = [torch.empty((rows, cols), dtype=torch.bfloat16, device=device) for _ in sets]
        keep.append(outs)
        return bind("b200_swiglu", [(p(s["gate_up"]), ctypes.c_void_p(s["gate_up"].data_ptr() + 2 * cols), p(o), rows, cols,
                                     2 * cols, 2 * cols, cols, _lib.BF16, stream) for s, o in zip(sets, outs)])
    raise ValueError(w.name)


def time_launches(run, steps: int, warmup: int, device) -> float:
    """Average milliseconds per call of run(i) over `steps` back-to-back calls."""
    for i in range(warmup):
        run(i)
    torch.cuda.synchronize(device)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        run(i)
    end.record()
    torch.cuda.synchronize(device)
    return start.elapsed_time(end) / steps


def time_launches_with_clock(run, steps: int, warmup: int, device) -> dict:
    """time_launches, with the SM clock and the board power read through NVML every few milliseconds while the GPU works
    through the queued launches (reads only).  time x median clock = SM cycles per launch."""
    for i in range(warmup):
        run(i)
    torch.cuda.synchronize(device)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        run(i)
    end.record()
    clocks, watts = [], []
    try:
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(device.index or 0)
        while not end.query():
            clocks.append(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM))
            watts.append(pynvml.nvmlDeviceGetPowerUsage(handle) / 1000.0)
            time.sleep(0.005)
    except Exception:  # no NVML on this machine: the time alone
        pass
    torch.cuda.synchronize(device)
    ms = start.elapsed_time(end) / steps
    out = {"ms": round(ms, 4), "steps": steps}
    if clocks:
        mhz = statistics.median(clocks)
        out.update(sm_mhz=mhz, power_w=round(statistics.median(watts), 1), clock_samples=len(clocks), sm_mcycles_per_launch=round(ms * mhz / 1e3, 2))
    return out


def steps_for(nbytes: int, target_s: float = 0.4, lo: int = 20, hi: int = 2000) -> int:
    return max(lo, min(hi, int(target_s / (nbytes / 6.0e12))))


def time_graph_replay(run, steps: int, warmup: int, device, stream) -> float:
    """Average milliseconds per call of run(i) when the `steps` back-to-back calls are captured once into a CUDA graph
    (on `stream`, the stream `run` launches into) and replayed: the host then issues one launch instead of `steps`, so
    kernels of a few microseconds are timed at the GPU's pace, not at the pace of the host's launch calls."""
    with torch.cuda.stream(stream):
        for i in range(warmup):
            run(i)
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        for i in range(steps):
            run(i)
    graph.replay()
    torch.cuda.synchronize(device)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    graph.replay()
    end.record()
    torch.cuda.synchronize(device)
    return start.elapsed_time(end) / steps


def bench_single_kernel_ops(device, peak_gbs: float, sampler, which: list[str], scale: float = 1.0,
                            steps: int | None = None, warmup: int = 5, graph: bool = False) -> dict:
    from popcorn_b200 import workloads

    out = {}
    side = torch.cuda.Stream(device) if graph else None
    for key in which:
        w = workloads.CONFIGS[key](scale=scale)
        nbytes = sum(w.algorithmic_bytes.values())
        if graph:
            with torch.cuda.stream(side):  # the runner binds the stream that is current now: graphs cannot capture the default one
                run, nsets = make_runner(w, device)
        else:
            run, nsets = make_runner(w, device)
        n_steps = steps or steps_for(nbytes, hi=500 if graph else 2000)
        t0 = time.time()
        ms = time_graph_replay(run, n_steps, warmup, device, side) if graph else time_launches(run, n_steps, warmup, device)
        if sampler is not None:
            sampler.mark(t0, time.time())
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[key] = {"ms": round(ms, 5), "gb_s": round(gbs, 1), "frac_of_measured_peak": round(gbs / peak_gbs, 4),
                    "frac_of_8tbs": round(gbs / SPEC_HBM_GBS, 4), "tokens_per_s": round(w.tokens / (ms * 1e-3), 1),
                    "algorithmic_bytes": nbytes, "steps": n_steps, "buffer_sets": nsets,
                    "timing": "one CUDA graph of all steps, replayed" if graph else "back-to-back launches"}
        del run, w
        torch.cuda.empty_cache()
    return out


def bench_moe(device, peak_gbs: float, sampler, scale: float = 1.0, fixed_steps: int | None = None, warmup: int = 3) -> dict:
    """Config 5 phase by phase: route, index (3 small kernels), permute, unpermute."""
    from popcorn_b200 import ops, workloads

    w = workloads.moe_bf16(scale=scale)
    x, logits = w.inputs["x"].to(device), w.inputs["router_logits"].to(device)
    experts, top_k = w.args["experts"], w.args["top_k"]
    idx, wts = ops.moe_route(logits, top_k)
    counts, offsets, perm, pos = ops.moe_index(idx, experts)
    rows, *_ = ops.moe_permute(x, idx, experts)

    from popcorn_b200 import _lib
    import ctypes

    tokens, hidden = x.shape
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    y = torch.empty_like(x)
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    need = ctypes.c_size_t(0)
    _lib.call("b200_moe_index_scratch_bytes", tokens, top_k, experts, ctypes.byref(need))
    scratch = torch.empty(max(need.value, 16), dtype=torch.uint8, device=device)
    idx2, wts2 = torch.empty_like(idx), torch.empty_like(wts)
    counts2, offsets2, perm2, pos2 = (torch.empty_like(t) for t in (counts, offsets, perm, pos))
    phases = {
        # every phase straight through the C ABI into outputs allocated up front, like the other configurations
        "route": lambda i: _lib.call("b200_moe_route", p(logits), p(idx2), p(wts2), tokens, experts, top_k, experts, _lib.F32, stream),
        "index": lambda i: _lib.call("b200_moe_index", p(idx), tokens, top_k, experts, p(counts2), p(offsets2), p(perm2), p(pos2),
                                     p(scratch), ctypes.c_size_t(scratch.numel()), stream),
        # what a layer runs: routing and the index through one call, without the list of token ids per sorted row
        # (permute and unpermute read the inverse map `pos` only)
        "route_index": lambda i: _lib.call("b200_moe_route_index", p(logits), p(idx2), p(wts2), tokens, experts, top_k, experts, _lib.F32,
                                           p(counts2), p(offsets2), ctypes.c_void_p(0), p(pos2), p(scratch), ctypes.c_size_t(scratch.numel()), stream),
        # permute and unpermute alone, straight through the C ABI (moe_permute the op also rebuilds the index)
        "permute": lambda i: _lib.call("b200_moe_permute", p(x), p(pos), p(rows), tokens, top_k, hidden, hidden, hidden, _lib.BF16, stream),
        "unpermute": lambda i: _lib.call("b200_moe_unpermute", p(rows), p(wts), p(pos), p(y), tokens, top_k, hidden, hidden, hidden, _lib.BF16, stream),
    }
    out = {}
    total_ms = 0.0
    for name, run in phases.items():
        nbytes = w.algorithmic_bytes["route"] + w.algorithmic_bytes["index"] if name == "route_index" else w.algorithmic_bytes[name]
        steps = fixed_steps or steps_for(nbytes, hi=300)
        t0 = time.time()
        ms = time_launches(run, steps, warmup, device)
        if sampler is not None:
            sampler.mark(t0, time.time())
        if name not in ("route", "index"):  # the whole path = one-launch routing + index, permute, unpermute
            total_ms += ms
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"ms": round(ms, 5), "gb_s": round(gbs, 1), "frac_of_measured_peak": round(gbs / peak_gbs, 4),
                     "frac_of_8tbs": round(gbs / SPEC_HBM_GBS, 4), "algorithmic_bytes": nbytes, "steps": steps}
    out["tokens_per_s"] = round(w.tokens / (total_ms * 1e-3), 1)
    out["ms"] = round(total_ms, 5)
    out["ms_with_separate_route_and_index_calls"] = round(total_ms - out["route_index"]["ms"] + out["route"]["ms"] + out["index"]["ms"], 5)
    return out


def torch_eager_incumbent(device, per_op: dict, records_root: str | None) -> None:
    """The incumbent on the same GPU: the references' own PyTorch code run eagerly on CUDA tensors.

    Adds `torch_eager_gpu_ms` (and the speed-up over it) to each single-kernel entry of `per_op`, and, when
    `records_root` is given, writes popcorn report rows (schema 3) for the configurations popcorn can
    represent as a case, with error gauges measured against an fp64 evaluation on a 512-token sample."""
    from oracle import reference_ops as reference
    from popcorn_b200 import autograd as differentiable
    from popcorn_b200 import ops, records, workloads

    def timed(fn, reps=10):
        for _ in range(2):
            fn()
        torch.cuda.synchronize(device)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(reps):
            fn()
        end.record()
        torch.cuda.synchronize(device)
        return start.elapsed_time(end) / reps

    def gauge(mine, native, truth):
        return {"err": float((mine.double() - truth).abs().max()), "budget": float((native.double() - truth).abs().max()),
                "scale": max(1.0, float(truth.abs().max()))}

    rows = []
    cases = records.benchmark_configs()
    for key in ("rms_norm_fp32", "add_rms_norm_bf16", "rotary_bf16", "swiglu_bf16"):
        w = workloads.CONFIGS[key]().to(device)
        i = w.inputs
        if key == "rms_norm_fp32":
            call = lambda f, t: (f.rms_norm(t["x"], t["weight"], None, w.args["eps"]),)  # noqa: E731
        elif key == "add_rms_norm_bf16":
            call = lambda f, t: f.add_rms_norm(t["x"], t["residual"], t["weight"], w.args["eps"], w.args["offset"])  # noqa: E731
        elif key == "rotary_bf16":
            call = lambda f, t: (f.rotary_embedding(t["q"], t["cos"], t["sin"]), f.rotary_embedding(t["k"], t["cos"], t["sin"]))  # noqa: E731
        else:
            c = w.args["cols"]
            call = lambda f, t: (f.swiglu(t["gate_up"][:, :c], t["gate_up"][:, c:]),)  # noqa: E731
        eager_ms = timed(lambda: call(reference, i))
        per_op[key]["torch_eager_gpu_ms"] = round(eager_ms, 4)
        per_op[key]["speedup_vs_torch_eager_gpu"] = round(eager_ms / per_op[key]["ms"], 2)
        if records_root and key in cases:
            op_name, config = cases[key]
            sample = {k: (v[:512] if v.dim() == 2 and v.shape[0] > 512 else v) for k, v in i.items()}
            wide = {k: v.double() for k, v in sample.items()}
            mine, native, truth = call(ops, sample), call(reference, sample), call(reference, wide)
            gauges = {str(n): gauge(m, nat, tr) for n, (m, nat, tr) in enumerate(zip(mine, native, truth))}
            status, reason = records.grade(config["dtype"], gauges)
            rows.append(records.make_row(op_name, config, device=torch.cuda.get_device_name(device), torch_version=torch.__version__,
                                         fwd_ms=per_op[key]["ms"], ref_fwd_ms=eager_ms, gauges=gauges, reps=per_op[key]["steps"],
                                         status=status, reason=reason))
            # the training-call row of the same case: forward with gradients enabled, the backward pass alone
            # (bench/compare.py:135-174), and gradient gauges named after the op's parameters, on the sample
            if key == "swiglu_bf16":
                named = lambda t: {"a": t["gate_up"][:, :c], "b": t["gate_up"][:, c:]}  # noqa: E731
                grad_call = lambda f, t: (f.swiglu(t["a"], t["b"]),)  # noqa: E731
            else:
                named, grad_call = (lambda t: t), call

            def leaves_of(tensors, cast=lambda t: t):
                return {k: cast(v).detach().clone().requires_grad_() for k, v in named(tensors).items()}

            def passes(f, tensors):
                held = leaves_of(tensors)
                fwd = timed(lambda: grad_call(f, held))
                outs = grad_call(f, held)
                seeds = [torch.ones_like(o) for o in outs]
                bwd = timed(lambda: torch.autograd.grad(outs, list(held.values()), seeds, retain_graph=True, allow_unused=True))
                return fwd, bwd

            def grads_of(f, tensors, cast=lambda t: t):
                held = leaves_of(tensors, cast)
                outs = grad_call(f, held)
                found = torch.autograd.grad(outs, list(held.values()), [torch.ones_like(o) for o in outs], allow_unused=True)
                return dict(zip(held, found))

            fwd_ms, bwd_ms = passes(differentiable, i)
            ref_fwd_ms, ref_bwd_ms = passes(reference, i)
            mine_g, native_g, truth_g = grads_of(differentiable, sample), grads_of(reference, sample), grads_of(reference, sample, lambda t: t.double())
            grad_gauges = {k: gauge(mine_g[k], native_g[k], truth_g[k]) for k in truth_g if truth_g[k] is not None}
            status, reason = records.grade(config["dtype"], gauges, grad_gauges)
            rows.append(records.make_row(op_name, config, device=torch.cuda.get_device_name(device), torch_version=torch.__version__,
                                         fwd_ms=fwd_ms, ref_fwd_ms=ref_fwd_ms, gauges=gauges, reps=10, status=status, reason=reason,
                                         grad_gauges=grad_gauges, bwd_ms=bwd_ms, ref_bwd_ms=ref_bwd_ms))
            per_op[key]["training_call"] = {"fwd_ms": round(fwd_ms, 4), "bwd_ms": round(bwd_ms, 4), "torch_eager_fwd_ms": round(ref_fwd_ms, 4),
                                            "torch_eager_bwd_ms": round(ref_bwd_ms, 4)}
        del w, i
        torch.cuda.empty_cache()
    if records_root and rows:
        paths = records.write_rows(rows, records_root)
        per_op["popcorn_report_rows"] = [str(path) for path in paths]


def popcorn_incumbents(device, per_op: dict) -> None:
    """popcorn's own first-party GPU kernels for two of the five configurations, on the same GPU in the same run:
    the CUDA SwiGLU (src/popcorn/impls/swiglu.cu:25-41, 77-101, built by popcorn's own JIT loader) on configuration 4
    and the Triton rotary kernel (src/popcorn/impls/rotary_embedding_tl.py:17-110) on configuration 3.  They are
    imported directly from the unmodified package: popcorn's dispatcher gates its `popcorn` backend on a Triton
    version this image does not have.  Adds `popcorn_incumbent` to the two entries of `per_op`."""
    from popcorn_b200 import workloads

    if reference_popcorn() is None:
        note = {"unavailable": "the popcorn package is not installed under baseline/_ref"}
        per_op["swiglu_bf16"]["popcorn_incumbent"] = per_op["rotary_bf16"]["popcorn_incumbent"] = note
        return

    def guarded(key, body):
        try:
            per_op[key]["popcorn_incumbent"] = body()
        except Exception as error:  # a JIT build or a Triton compile that fails on this box is a finding, not a crash
            per_op[key]["popcorn_incumbent"] = {"error": f"{type(error).__name__}: {error}"[:300]}
        torch.cuda.empty_cache()

    def build_swiglu_extension(limit_s: int = 300) -> float:
        """popcorn builds its CUDA extension on first use (torch's JIT loader: ninja + nvcc, about a minute when the
        prebuilt copy under baseline/_ext does not match).  That first use happens in a child process with a time
        limit, so that a build that cannot finish (a lock file left by an interrupted build, a broken toolchain) costs
        this leg, not the whole benchmark."""
        lock = Path(os.environ.get("TORCH_EXTENSIONS_DIR", "")) / "popcorn_swiglu" / "lock"
        if lock.is_file():  # nobody else builds here: a lock can only be left over
            lock.unlink()
        code = "import sys, warnings; warnings.filterwarnings('ignore'); from popcorn.impls import _cuda; _cuda.load('swiglu')"
        env = {**os.environ, "PYTHONPATH": os.pathsep.join(p for p in sys.path if p)}
        t0 = time.time()
        done = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=limit_s)
        if done.returncode != 0:
            raise RuntimeError(f"popcorn's JIT build of swiglu.cu failed: {done.stderr.strip().splitlines()[-1] if done.stderr.strip() else done.returncode}")
        return time.time() - t0

    def swiglu_leg():
        build_s = build_swiglu_extension()
        from popcorn.impls.swiglu_cu import swiglu as incumbent

        w = workloads.swiglu_bf16().to(device)
        cols, gate_up = w.args["cols"], w.inputs["gate_up"]
        a, b = gate_up[:, :cols], gate_up[:, cols:]
        t0 = time.time()
        incumbent(a[:8], b[:8])
        load_s = time.time() - t0
        strided = time_launches(lambda i: incumbent(a, b), 20, 3, device)
        a_c, b_c = a.contiguous(), b.contiguous()
        contiguous = time_launches(lambda i: incumbent(a_c, b_c), 20, 3, device)
        mine = per_op["swiglu_bf16"]["ms"]
        return {"kernel": "popcorn.impls.swiglu_cu.swiglu (impls/swiglu.cu fwd_kernel)", "build_s": round(build_s, 1), "load_s": round(load_s, 1),
                "ms_on_the_configs_strided_halves": round(strided, 4), "ms_on_contiguous_copies": round(contiguous, 4),
                "b200_speedup_strided": round(strided / mine, 2), "b200_speedup_contiguous": round(contiguous / mine, 2),
                "note": "the incumbent copies strided inputs to contiguous tensors first (swiglu.cu:80-81) and rounds once, "
                        "so it is not bit-equal to popcorn's registered reference"}

    def rotary_leg():
        from popcorn.impls.rotary_embedding_tl import rotary_embedding as incumbent

        w = workloads.rotary_bf16().to(device)
        q, k, cos, sin = (w.inputs[name] for name in ("q", "k", "cos", "sin"))
        incumbent(q[:1], cos, sin, False)
        both = time_launches(lambda i: (incumbent(q, cos, sin, False), incumbent(k, cos, sin, False)), 20, 5, device)
        mine = per_op["rotary_bf16"]["ms"]
        return {"kernel": "popcorn.impls.rotary_embedding_tl.rotary_embedding (Triton _rotary_kernel), q then k, out of place",
                "ms": round(both, 4), "b200_speedup": round(both / mine, 2)}

    guarded("swiglu_bf16", swiglu_leg)
    guarded("rotary_bf16", rotary_leg)


def bench_extra_ops(device, peak_gbs: float, sampler, scale: float = 1.0, steps: int = 50, match: str = "") -> dict:
    """The ops beyond the five benchmark configurations, at the benchmark shapes they correspond to.

    Timed through the public op functions (outputs allocated per call by the caching allocator, which does
    not synchronise), 50 launches each; bytes = every input read once + every output written once."""
    from popcorn_b200 import ops, workloads

    out = {}

    def run(name, fn, nbytes):
        if match not in name:
            return
        nbytes = int(nbytes)
        t0 = time.time()
        ms = time_launches(lambda i: fn(), steps, 3, device)
        if sampler is not None:
            sampler.mark(t0, time.time())
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"ms": round(ms, 5), "gb_s": round(gbs, 1), "frac_of_measured_peak": round(gbs / peak_gbs, 4),
                     "frac_of_8tbs": round(gbs / SPEC_HBM_GBS, 4), "algorithmic_bytes": nbytes}

    w = workloads.swiglu_bf16(scale).to(device)
    gu, cols = w.inputs["gate_up"], w.args["cols"]
    a, b = gu[:, :cols], gu[:, cols:]
    grad = torch.randn(gu.shape[0], cols, device=device).to(torch.bfloat16)
    n = a.numel() * 2
    run("geglu_bf16 [32768, 2x14336]", lambda: ops.geglu(a, b), 3 * n)
    run("swiglu_backward_bf16 [32768, 14336]", lambda: ops.swiglu_backward(grad, a, b), 5 * n)
    run("geglu_backward_bf16 [32768, 14336]", lambda: ops.geglu_backward(grad, a, b), 5 * n)
    run("sigmoid_gate_backward_bf16 [32768, 14336]", lambda: ops.sigmoid_gate_backward(grad, a, b), 5 * n)
    del w, gu, a, b, grad
    torch.cuda.empty_cache()

    w = workloads.add_rms_norm_bf16(scale).to(device)
    x, r, weight = w.inputs["x"], w.inputs["residual"], w.inputs["weight"]
    n = x.numel() * 2
    run("rms_norm_gated_bf16 [16384, 8192]", lambda: ops.rms_norm_gated(x, r, weight), 3 * n)
    run("layer_norm_bf16 [16384, 8192]", lambda: ops.layer_norm(x, weight, weight), 2 * n)
    run("rms_norm_backward_bf16 [16384, 8192]", lambda: ops.rms_norm_backward(r, x, weight), 3 * n)
    run("add_rms_norm_backward_bf16 [16384, 8192]", lambda: ops.add_rms_norm_backward(r, r, x, weight, 1e-5), 4 * n)
    run("layer_norm_backward_bf16 [16384, 8192]", lambda: ops.layer_norm_backward(r, x, weight, True), 3 * n)
    run("l2_norm_backward_bf16 [16384, 8192]", lambda: ops.l2_norm_backward(r, x), 3 * n)
    heads = x.view(-1, 128)  # per-head q/k normalisation: 1,048,576 rows of 128
    run("l2_norm_bf16 [1048576, 128]", lambda: ops.l2_norm(heads), 2 * n)
    run("l2_norm_backward_bf16 [1048576, 128]", lambda: ops.l2_norm_backward(r.view(-1, 128), heads), 3 * n)
    head_weight_row = weight[:128].contiguous()
    run("rms_norm_bf16 [1048576, 128]", lambda: ops.rms_norm(heads, head_weight_row), 2 * n)
    run("rms_norm_backward_bf16 [1048576, 128]", lambda: ops.rms_norm_backward(r.view(-1, 128), heads, head_weight_row), 3 * n)
    run("layer_norm_backward_bf16 [1048576, 128]", lambda: ops.layer_norm_backward(r.view(-1, 128), heads, head_weight_row, True), 3 * n)
    del w, x, r, weight, heads
    torch.cuda.empty_cache()

    # the combine's backward on the rows of config 5: reads grad_y once per token and the expert rows, writes the
    # scaled gradient rows and the per-slot dot products
    w = workloads.moe_bf16(scale).to(device)
    idx, wts = ops.moe_route(w.inputs["router_logits"], w.args["top_k"])
    rows, _, _, _, pos = ops.moe_permute(w.inputs["x"], idx, w.args["experts"])
    grad_y = torch.randn_like(w.inputs["x"])
    run("moe_unpermute_backward_bf16 [65536 x 8, 4096]", lambda: ops.moe_unpermute_backward(grad_y, rows, wts, pos),
        2 * rows.numel() * 2 + grad_y.numel() * 2 + 3 * pos.numel() * 4)
    del w, idx, wts, rows, pos, grad_y
    torch.cuda.empty_cache()

    # the rotary siblings at the shapes of config 3 (8 x 4096 positions, 32 + 8 heads of 128)
    w = workloads.paired_rope_bf16(scale).to(device)
    q, k, cos, sin = (w.inputs[name] for name in ("q", "k", "cos", "sin"))
    head_weight = (1 + 0.1 * torch.randn(128, device=device)).to(torch.bfloat16)
    n = 2 * (q.numel() + k.numel()) * 2
    run("qk_norm_rope_bf16 q[8,32,4096,128] k[8,8,4096,128]", lambda: ops.qk_norm_rope(q, k, head_weight, head_weight, cos, sin),
        n + 2 * cos.numel() * 2 + 2 * 128 * 2)
    grad_q, grad_k = torch.randn_like(q), torch.randn_like(k)
    run("qk_norm_rope_backward_bf16 q[8,32,4096,128] k[8,8,4096,128]",
        lambda: ops.qk_norm_rope_backward(grad_q, grad_k, q, k, head_weight, head_weight, cos, sin), 1.5 * n + 2 * cos.numel() * 2)
    del grad_q, grad_k
    w3 = workloads.rotary_bf16(scale).to(device)
    q3, k3 = w3.inputs["q"], w3.inputs["k"]
    freqs = torch.stack((w3.inputs["cos"], w3.inputs["sin"]), -1).to(torch.bfloat16)
    run("llama4_rope_bf16 q[8,4096,32,128] k[8,4096,8,128]", lambda: ops.llama4_rope(q3, k3, freqs), n + freqs.numel() * 2)
    cos3, sin3 = w3.inputs["cos"], w3.inputs["sin"]
    table = 2 * cos3.numel() * cos3.element_size()
    run("rotary_interleaved_bf16 q[8,4096,32,128]", lambda: ops.rotary_embedding(q3, cos3, sin3, True), 2 * q3.numel() * 2 + table)
    half = cos3[:, : cos3.shape[1] // 2].contiguous(), sin3[:, : sin3.shape[1] // 2].contiguous()
    run("rotary_partial_bf16 q[8,4096,32,128] (first 64 channels rotated)", lambda: ops.rotary_embedding(q3, half[0], half[1]),
        2 * q3.numel() * 2 + table // 2)
    return out


def per_config_fractions(per_op: dict) -> dict | None:
    """achieved GB/s / measured copy peak for the kernels of all five configurations, compactly (same run, rank 0)."""
    if not per_op:
        return None
    out = {key: per_op[key]["frac_of_measured_peak"] for key in ("rms_norm_fp32", "add_rms_norm_bf16", "rotary_bf16", "swiglu_bf16") if key in per_op}
    for phase in ("route", "index", "route_index", "permute", "unpermute"):
        if phase in per_op.get("moe_bf16", {}):
            out[f"moe_{phase}"] = per_op["moe_bf16"][phase]["frac_of_measured_peak"]
    return out


def measured_tensor_peak() -> tuple[float, float, str]:
    """(burst, sustained) dense bf16 TFLOP/s of cuBLAS on this pool's B200s, else the fallback figures."""
    try:
        peaks = json.loads((REPO / "MEASURED_PEAKS.json").read_text())
        return float(peaks["bf16_tflops"]), float(peaks["bf16_tflops_sustained"]), "measured"
    except (OSError, KeyError, ValueError):
        return 1590.0, 1400.0, "fallback"


def bench_grouped_gemm(device, sampler, scale: float = 1.0, steps: int = 10, warmup: int = 3, inter: int = 1536) -> dict:
    """The expert MLP on the rows of config 5: 65536 tokens x top-8 = 524288 rows of 4096 over 64 experts (8192 rows each
    on average, routed by the config's own seeded logits), SwiGLU MLP with an intermediate size of 1536 per expert.

    Two launches per forward step: gate/up projection + SwiGLU (2 * rows * 4096 * 3072 flop), down projection
    (2 * rows * 1536 * 4096 flop); then the training launches, each timed on its own: both pre-activations kept,
    the two row gradients and the weight gradients.  Tensor-core bound: TFLOP/s against the measured cuBLAS bf16 peak."""
    import ctypes

    from popcorn_b200 import _lib, ops, workloads

    w = workloads.moe_bf16(scale=scale).to(device)
    x, logits = w.inputs["x"], w.inputs["router_logits"]
    experts, top_k = w.args["experts"], w.args["top_k"]
    hidden = x.shape[1]
    idx, _ = ops.moe_route(logits, top_k)
    rows, _, offsets, perm, _ = ops.moe_permute(x, idx, experts)
    tokens_x = x  # the token-order rows, for the projection that gathers them through `perm`
    del logits, idx
    gen = torch.Generator(device=device).manual_seed(5)
    gate = (torch.randn(experts, hidden, inter, device=device, generator=gen) / hidden ** 0.5).to(torch.bfloat16)
    up = (torch.randn(experts, hidden, inter, device=device, generator=gen) / hidden ** 0.5).to(torch.bfloat16)
    down = (torch.randn(experts, inter, hidden, device=device, generator=gen) / inter ** 0.5).to(torch.bfloat16)
    total = rows.shape[0]
    act = torch.empty(total, inter, device=device, dtype=torch.bfloat16)
    out = torch.empty(total, hidden, device=device, dtype=torch.bfloat16)
    lib = _lib.library()
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731

    def check(status):
        if status != 0:
            raise _lib.B200Error("b200_moe_grouped_gemm", status, lib.b200_status_string(status).decode(), lib.b200_last_error().decode())

    def gate_up(i):
        check(lib.b200_moe_grouped_gemm(p(rows), p(gate), p(up), p(offsets), p(act), total, hidden, inter, experts, hidden, inter, _lib.BF16, stream))

    def gate_up_gathered(i):
        check(lib.b200_moe_grouped_gemm_gathered(p(tokens_x), p(perm), p(gate), p(up), p(offsets), p(act), tokens_x.shape[0], total, hidden, inter,
                                                 experts, hidden, inter, _lib.BF16, stream))

    def down_proj(i):
        check(lib.b200_moe_grouped_gemm(p(act), p(down), ctypes.c_void_p(0), p(offsets), p(out), total, inter, hidden, experts, inter, hidden, _lib.BF16, stream))

    # the training launches: both pre-activations kept, then the gradients (the values of the "gradients" do not
    # matter for the timing: the finished outputs stand in for them)
    both = torch.empty(total, 2 * inter, device=device, dtype=torch.bfloat16)
    grad_act = torch.empty(total, inter, device=device, dtype=torch.bfloat16)
    grad_rows = torch.empty(total, hidden, device=device, dtype=torch.bfloat16)
    grad_down = torch.empty_like(down)
    grad_gate = torch.empty_like(gate)
    null = ctypes.c_void_p(0)
    half = ctypes.c_void_p(both.data_ptr() + inter * 2)  # the up half of `both`

    def gate_up_kept(i):
        check(lib.b200_moe_grouped_gemm_gate_up(p(rows), p(gate), p(up), p(offsets), p(both), total, hidden, inter, experts, hidden, 2 * inter, _lib.BF16, stream))

    def down_dgrad(i):
        check(lib.b200_moe_grouped_gemm_dgrad(p(out), p(down), null, null, p(offsets), p(grad_act), total, inter, hidden, experts, hidden, inter, _lib.BF16, stream))

    def down_wgrad(i):
        check(lib.b200_moe_grouped_gemm_wgrad(p(act), p(out), p(offsets), p(grad_down), total, inter, hidden, experts, inter, hidden, _lib.BF16, stream))

    def gate_up_dgrad(i):
        check(lib.b200_moe_grouped_gemm_dgrad(p(both), p(gate), half, p(up), p(offsets), p(grad_rows), total, hidden, inter, experts, 2 * inter, hidden, _lib.BF16, stream))

    def gate_wgrad(i):
        check(lib.b200_moe_grouped_gemm_wgrad(p(rows), p(both), p(offsets), p(grad_gate), total, hidden, inter, experts, hidden, 2 * inter, _lib.BF16, stream))

    burst, sustained, kind = measured_tensor_peak()
    result = {"rows": total, "hidden": hidden, "intermediate": inter, "experts": experts, "peak_kind": kind}
    for name, fn, flop in (("gate_up_swiglu", gate_up, 2.0 * total * hidden * 2 * inter),
                           ("gate_up_swiglu_rows_gathered_in_the_operand_load", gate_up_gathered, 2.0 * total * hidden * 2 * inter),
                           ("down", down_proj, 2.0 * total * inter * hidden),
                           ("gate_up_kept", gate_up_kept, 2.0 * total * hidden * 2 * inter), ("down_dgrad", down_dgrad, 2.0 * total * inter * hidden),
                           ("down_wgrad", down_wgrad, 2.0 * total * inter * hidden), ("gate_up_dgrad", gate_up_dgrad, 2.0 * total * hidden * 2 * inter),
                           ("gate_wgrad", gate_wgrad, 2.0 * total * hidden * inter)):
        t0 = time.time()
        ms = time_launches(fn, steps, warmup, device)
        if sampler is not None:
            sampler.mark(t0, time.time())
        tflops = flop / (ms * 1e-3) / 1e12
        result[name] = {"ms": round(ms, 4), "tflop_s": round(tflops, 1), "flop": flop, "frac_of_measured_burst": round(tflops / burst, 4),
                        "frac_of_measured_sustained": round(tflops / sustained, 4)}
    result["wait_timeouts"] = _lib.wait_timeouts()
    # The same flop count through this kernel and through cuBLAS, one second each, with the SM clock sampled inside each
    # window: both run under the 1 kW power cap, where the clock each settles at is part of its speed.  time x clock
    # = SM cycles per launch, the figure that compares the two kernels' use of the tensor pipe.
    if total % experts == 0:
        per = total // experts
        a3, gate_up_w = rows.view(experts, per, hidden), torch.cat((gate, up), dim=2)
        study = {}
        for name, fn in (("gate_up_swiglu", gate_up), ("cublas_bmm_gate_up", lambda i: torch.bmm(a3, gate_up_w))):
            study[name] = time_launches_with_clock(fn, 120, warmup, device)
        if all("sm_mhz" in entry for entry in study.values()):
            ours, theirs = study["gate_up_swiglu"], study["cublas_bmm_gate_up"]
            study["sm_cycles_ratio_ours_over_cublas"] = round(ours["sm_mcycles_per_launch"] / theirs["sm_mcycles_per_launch"], 4)
        result["clock_study"] = study
        del a3, gate_up_w
    # the library GEMM on the same box in the same run, same flop count: one batched cuBLAS matmul per projection over
    # equal-size experts (total / experts rows each), without the SwiGLU epilogue and writing both projections out
    if total % experts == 0:
        per = total // experts
        a3 = rows.view(experts, per, hidden)
        gate_up_w = torch.cat((gate, up), dim=2)
        act3 = act.view(experts, per, inter)
        for name, fn, flop in (("cublas_bmm_gate_up", lambda i: torch.bmm(a3, gate_up_w), 2.0 * total * hidden * 2 * inter),
                               ("cublas_bmm_down", lambda i: torch.bmm(act3, down), 2.0 * total * inter * hidden)):
            ms = time_launches(fn, steps, warmup, device)
            result[name] = {"ms": round(ms, 4), "tflop_s": round(flop / (ms * 1e-3) / 1e12, 1)}
    # the whole layer through the registered op: inference (route, permute, two launches, unpermute) and a training
    # step (forward with the pre-activations kept, then every gradient: tokens, router logits, three weight tensors)
    del both, grad_act, grad_rows, grad_down, grad_gate, act, out, rows, tokens_x, perm
    torch.cuda.empty_cache()
    from popcorn_b200 import autograd as differentiable

    w = workloads.moe_bf16(scale=scale).to(device)
    x, logits = w.inputs["x"], w.inputs["router_logits"]
    layer_flop = 3 * 2.0 * total * hidden * inter
    ms = time_launches(lambda i: ops.momoe(x, gate, up, down, logits, top_k), steps, warmup, device)
    result["layer_forward"] = {"ms": round(ms, 4), "tflop_s": round(layer_flop / (ms * 1e-3) / 1e12, 1), "flop": layer_flop}
    leaves = [t.detach().requires_grad_() for t in (x, gate, up, down, logits)]
    grad_y = torch.ones_like(x)

    def train_step(i):
        for leaf in leaves:
            leaf.grad = None
        differentiable.momoe(*leaves, top_k).backward(grad_y)

    ms = time_launches(train_step, steps, warmup, device)
    result["layer_forward_backward"] = {"ms": round(ms, 4), "tflop_s": round(3 * layer_flop / (ms * 1e-3) / 1e12, 1), "flop": 3 * layer_flop}
    return result


def bench_moe_expert_parallel(device, world: int, rank: int, dist, exchange: str, steps: int = 20, warmup: int = 3) -> dict:
    """Config 5 sharded over the ranks: 65536 / world tokens and 64 / world experts per GPU.

    One step = dispatch (route, index, permute, all-to-all, reorder) + combine (reorder, all-to-all,
    weighted unpermute); the expert MLPs between the two are not part of this path.  Strong scaling:
    the job's token count is fixed.  Time is the max over ranks of the CUDA-event time per step."""
    from popcorn_b200 import workloads
    from popcorn_b200.expert_parallel import ExpertParallel

    w = workloads.moe_bf16().shard(rank, world)
    x, logits = w.inputs["x"].to(device), w.inputs["router_logits"].to(device)
    ep = ExpertParallel(w.args["experts"], w.args["top_k"], exchange=exchange)
    state = None
    for _ in range(warmup):
        state = ep.dispatch(x, logits)
        ep.combine(state.rows if exchange == "nccl" else state.out_rows, state)
    torch.cuda.synchronize(device)
    dist.barrier()
    torch.cuda.synchronize(device)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        state = ep.dispatch(x, logits)
        ep.combine(state.rows if exchange == "nccl" else state.out_rows, state)
    end.record()
    torch.cuda.synchronize(device)
    ms = torch.tensor([start.elapsed_time(end) / steps], device=device, dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.item())
    hidden_bytes = x.shape[1] * x.element_size()
    if exchange == "p2p":
        ep.check()  # no wait ran out, nothing over capacity
        sent_remote = int(state.info[1]) * hidden_bytes  # counted by the exchange kernel on the device
    else:
        sent_remote = (sum(state.send_counts) - state.send_counts[rank]) * hidden_bytes
    link = torch.tensor([float(sent_remote)], device=device, dtype=torch.float64)
    dist.all_reduce(link, op=dist.ReduceOp.MAX)
    return {"ms": round(ms, 4), "tokens_per_s": round(65536 / (ms * 1e-3), 1), "scaling": "strong (65536 tokens over all ranks)",
            "tokens_per_rank": int(x.shape[0]), "experts_per_rank": ep.local_experts,
            "nvlink_bytes_out_per_rank_per_exchange": int(link.item()), "exchanges_per_step": 2,
            "nvlink_gb_s_per_direction": round(link.item() * 2 / (ms * 1e-3) / 1e9, 1),
            "exchange": "NCCL all_to_all_single with split sizes" if exchange == "nccl"
            else "fused: permute kernel stores into peer memory, unpermute kernel loads from peer memory"}


def bench_strong_scaling(device, world: int, rank: int, dist, peak_gbs: float, full: dict) -> dict:
    """Configurations 1-4 (and the MoE steps over all 64 experts, without an exchange) on 1 / world of the tokens per
    GPU: the job's token count is fixed, so this is strong scaling.  Every rank times its own shard; the step time is
    the max over ranks, all ranks' times are listed, and the speed-up is against the full configuration on one GPU
    timed by rank 0 in this same run (`full`).  Configuration 1 is also reported weak (the whole configuration per GPU)."""
    keys = ["rms_norm_fp32", "add_rms_norm_bf16", "rotary_bf16", "swiglu_bf16"]
    # the shards are kernels of 3-50 us: their launches are captured in a CUDA graph and replayed, so that the host's
    # launch calls (about 5 us each through ctypes) do not set the time; the full configuration 1 is timed the same way
    mine = bench_single_kernel_ops(device, peak_gbs, None, keys, scale=1.0 / world, graph=True)
    moe = bench_moe(device, peak_gbs, None, scale=1.0 / world)
    weak = bench_single_kernel_ops(device, peak_gbs, None, ["rms_norm_fp32"], graph=True)["rms_norm_fp32"]["ms"]
    full = {**full, "rms_norm_fp32": {"ms": weak}}  # config 1's one-GPU time under the same timing (this rank's own GPU)
    times = torch.tensor([mine[k]["ms"] for k in keys] + [moe["ms"], weak], device=device, dtype=torch.float64)
    gathered = [torch.empty_like(times) for _ in range(world)]
    dist.all_gather(gathered, times)
    table = torch.stack(gathered).cpu()  # [rank, entry]
    worst = table.max(0).values.tolist()
    out = {"scaling": "strong", "tokens_per_gpu": "1/%d of each configuration" % world}
    totals = {"rms_norm_fp32": 4096, "add_rms_norm_bf16": 16384, "rotary_bf16": 32768, "swiglu_bf16": 32768, "moe_bf16_token_sharded": 65536}
    for column, key in enumerate([*keys, "moe_bf16_token_sharded"]):
        one_gpu = full.get("moe_bf16" if key.startswith("moe") else key, {}).get("ms")
        out[key] = {"ms_max_over_ranks": round(worst[column], 5), "ms_per_rank": [round(v, 5) for v in table[:, column].tolist()],
                    "tokens_per_s": round(totals[key] / (worst[column] * 1e-3), 1), "ms_one_gpu_same_run": one_gpu,
                    "speedup_vs_one_gpu": round(one_gpu / worst[column], 2) if one_gpu else None}
    out["rms_norm_fp32_weak"] = {"scaling": "weak (the whole configuration on every GPU)", "ms_max_over_ranks": round(worst[-1], 5),
                                 "ms_per_rank": [round(v, 5) for v in table[:, -1].tolist()],
                                 "tokens_per_s": round(world * 4096 / (worst[-1] * 1e-3), 1)}
    out["note"] = ("configuration 1 on 1/%d of its rows is a %d KiB kernel of a few microseconds: launch latency, not HBM, "
                   "bounds its strong-scaling figure" % (world, 2 * 4096 * 4096 * 4 // world // 1024))
    return out


def expert_parallel_check(device, world: int, rank: int, dist, exchange: str) -> dict:
    """Correctness of the expert-parallel exchange at this world size, recorded in the bench line: on its own token shard
    every rank runs the single-GPU chain (route -> permute -> unpermute) and the expert-parallel one (dispatch -> combine,
    the experts passing the rows through) and the two results must be bit-equal; the per-expert row counts summed over
    ranks must equal what the owners received."""
    from popcorn_b200 import ops, workloads
    from popcorn_b200.expert_parallel import ExpertParallel

    w = workloads.moe_bf16(scale=1 / 8).shard(rank, world)
    x, logits = w.inputs["x"].to(device), w.inputs["router_logits"].to(device)
    experts, top_k = w.args["experts"], w.args["top_k"]
    indices, weights = ops.moe_route(logits, top_k)
    rows, counts, _, _, pos = ops.moe_permute(x, indices, experts)
    want = ops.moe_unpermute(rows, weights, pos)
    ep = ExpertParallel(experts, top_k, exchange=exchange)
    state = ep.dispatch(x, logits)
    if exchange == "p2p":
        state.out_rows.copy_(state.rows)
        got = ep.combine(state.out_rows, state)
    else:
        got = ep.combine(state.rows, state)
    total = counts.to(torch.int64)
    dist.all_reduce(total)
    local = ep.local_experts
    offsets = state.expert_offsets.to(device).to(torch.int64)
    received = offsets[1:] - offsets[:-1]
    in_use = int(state.info[0]) if exchange == "p2p" else state.rows.shape[0]
    if exchange == "p2p":
        ep.check()
    flags = torch.tensor([int(torch.equal(got, want)), int(torch.equal(received, total[rank * local:(rank + 1) * local])),
                          int(in_use == int(received.sum()))], device=device)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    output_equal, counts_equal, rows_equal = (bool(v) for v in flags.tolist())
    return {"pass": output_equal and counts_equal and rows_equal, "output_bit_equal_to_single_gpu_chain": output_equal,
            "per_expert_counts_equal_allreduced_bincount": counts_equal, "received_rows_equal_counts": rows_equal,
            "tokens_per_rank": int(x.shape[0]), "ranks": world}


# ------------------------------------------------------------ CPU baseline --

def cpu_reference_fn(key: str, fraction: float):
    """(fn, tokens): the CPU oracle bound to a token sample of configuration `key`, inputs built once."""
    from oracle import reference_ops as oracle
    from popcorn_b200 import workloads

    torch.set_num_threads(os.cpu_count() or 1)
    w = workloads.CONFIGS[key](scale=fraction)
    i = w.inputs
    if key == "rms_norm_fp32":
        fn = lambda: oracle.rms_norm(i["x"], i["weight"], None, w.args["eps"])  # noqa: E731
    elif key == "add_rms_norm_bf16":
        fn = lambda: oracle.add_rms_norm(i["x"], i["residual"], i["weight"], w.args["eps"], w.args["offset"])  # noqa: E731
    elif key == "rotary_bf16":
        fn = lambda: (oracle.rotary_embedding(i["q"], i["cos"], i["sin"]), oracle.rotary_embedding(i["k"], i["cos"], i["sin"]))  # noqa: E731
    elif key == "swiglu_bf16":
        c = w.args["cols"]
        fn = lambda: oracle.swiglu(i["gate_up"][:, :c], i["gate_up"][:, c:])  # noqa: E731
    else:
        def fn():
            idx, wts = oracle.moe_route(i["router_logits"], w.args["top_k"])
            rows, _, _, _, pos = oracle.moe_permute(i["x"], idx, w.args["experts"])
            return oracle.moe_unpermute(rows, wts.float(), pos)
    return fn, w.tokens


def cpu_reference_time(key: str, fraction: float, repeats: int = 5) -> tuple[float, int, str]:
    """Best-of-`repeats` seconds of the CPU oracle on a token sample of configuration `key`."""
    fn, tokens = cpu_reference_fn(key, fraction)
    best = float("inf")
    with torch.no_grad():
        fn()  # warm-up
        for _ in range(repeats):
            t0 = time.perf_counter()
            fn()
            best = min(best, time.perf_counter() - t0)
    return best, tokens, f"{tokens} tokens ({fraction:g} of the configuration), best of {repeats}"


def reference_popcorn():
    """The unmodified popcorn package: already importable, else the install under baseline/_ref; None when absent."""
    import importlib.util
    import tempfile
    import warnings

    os.environ.setdefault("POPCORN_CACHE_DIR", tempfile.mkdtemp(prefix="popcorn-cache-"))
    if importlib.util.find_spec("popcorn") is None:
        from oracle import install_reference

        if not install_reference.installed():
            return None
        package, extensions = install_reference.stable_locations()
        sys.path.insert(0, str(package))
        os.environ.setdefault("TORCH_EXTENSIONS_DIR", str(extensions))
    warnings.filterwarnings("ignore")
    import popcorn
    import popcorn.kernels  # noqa: F401

    return popcorn


def cpu_headline_baseline() -> dict:
    """The `cpu_baseline` object of the GPU arm: the headline configuration on the host cores, best of 5, through the
    unmodified popcorn package when it is installed (kind "reference"), else through the CPU restatement ("port")."""
    from popcorn_b200 import workloads

    torch.set_num_threads(os.cpu_count() or 1)
    w = workloads.add_rms_norm_bf16()
    popcorn = reference_popcorn()
    if popcorn is not None:
        reference, kind, what = popcorn.KERNELS["add_rms_norm"].reference, "reference", "popcorn's add_rms_norm reference called from the unmodified package"
    else:
        from oracle import reference_ops

        reference, kind, what = reference_ops.add_rms_norm, "port", "PyTorch CPU restatement of popcorn's add_rms_norm reference"
    i = w.inputs
    best = float("inf")
    with torch.no_grad():
        for attempt in range(6):
            t0 = time.perf_counter()
            reference(i["x"], i["residual"], i["weight"], w.args["eps"], w.args["offset"])
            if attempt:
                best = min(best, time.perf_counter() - t0)
    return {"value": round(w.tokens / best, 1), "unit": "tokens/s", "cores": os.cpu_count() or 1, "kind": kind,
            "sample": f"{w.tokens} tokens (the whole configuration), best of 5; {what}, PyTorch CPU, {torch.get_num_threads()} threads"}


def run_reference_arm(args) -> None:
    """The reference's own implementation of the headline path on the host cores: popcorn's registered PyTorch
    reference of add_rms_norm (src/popcorn/kernels/add_rms_norm.py:8-23) called from the unmodified package, all host
    threads, one full configuration (16384 tokens) per step.  Without the package the CPU restatement stands in."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from popcorn_b200 import workloads

    torch.set_num_threads(os.cpu_count() or 1)
    w = workloads.add_rms_norm_bf16(scale=args.scale)
    x, residual, weight = w.inputs["x"], w.inputs["residual"], w.inputs["weight"]
    popcorn = reference_popcorn()
    if popcorn is not None:
        reference, kind = popcorn.KERNELS["add_rms_norm"].reference, "reference"
        what = f"popcorn {getattr(popcorn, '__version__', '')} add_rms_norm reference called from the unmodified package, PyTorch CPU".replace("  ", " ")
    else:
        from oracle import reference_ops

        reference, kind = reference_ops.add_rms_norm, "port"
        what = "PyTorch CPU restatement of popcorn's add_rms_norm reference (the package is not installed)"
    fn = lambda: reference(x, residual, weight, w.args["eps"], w.args["offset"])  # noqa: E731
    with torch.no_grad():
        for _ in range(max(args.warmup, 0)):
            fn()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            fn()
        seconds = time.perf_counter() - t0
    ms = seconds * 1e3 / args.steps
    value = w.tokens / (ms * 1e-3)
    cores = os.cpu_count() or 1
    line = {
        "impl": "reference", "metric": "tokens_per_s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": 0,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": headline_config(w.tokens),
        "cpu_baseline": {"value": round(value, 1), "unit": "tokens/s", "cores": cores, "kind": kind,
                         "sample": f"each step = {w.tokens} tokens (the whole configuration); {what}, {torch.get_num_threads()} threads"},
        "e2e": {"value": round(value, 1), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# -------------------------------------------------------------------- main --

def main() -> None:
    # Libraries (NCCL among them) may print to stdout; the contract is ONE JSON line there.
    # Keep the real stdout aside and point fd 1 at stderr until the line is printed.
    real_stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    sys.stdout = real_stdout
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", choices=["b200", "reference"], default="b200")
    parser.add_argument("--skip-per-op", action="store_true", help="only the headline loop (used for profiling captures)")
    parser.add_argument("--skip-incumbents", action="store_true", help="do not time popcorn's own CUDA / Triton kernels beside the b200 ones")
    parser.add_argument("--scale", type=float, default=1.0, help="shrink the token count (profiling captures only)")
    parser.add_argument("--records", metavar="DIR", help="also write popcorn report rows (schema 3) under DIR/v3/reports")
    parser.add_argument("--only", choices=["rms_norm_fp32", "add_rms_norm_bf16", "rotary_bf16", "swiglu_bf16", "paired_rope_bf16", "moe_bf16", "extras", "grouped_gemm"],
                        help="time one configuration's kernels alone and print a short JSON (profiling captures); "
                             "`extras` = the ops beyond the five configurations, filtered by --match")
    parser.add_argument("--match", default="", help="with --only extras: run the ops whose name contains this text")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    if args.impl == "reference":
        run_reference_arm(args)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the b200 backend has no CPU path")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)

    from popcorn_b200 import _lib, build, ops, workloads

    build.build()
    peak_gbs, peak_kind = measured_peak()
    if args.only:
        if args.only == "moe_bf16":
            result = bench_moe(device, peak_gbs, None, args.scale, args.steps, args.warmup)
        elif args.only == "extras":
            result = bench_extra_ops(device, peak_gbs, None, args.scale, args.steps, args.match)
        elif args.only == "grouped_gemm":
            result = bench_grouped_gemm(device, None, args.scale, args.steps, args.warmup)
        else:
            result = bench_single_kernel_ops(device, peak_gbs, None, [args.only], args.scale, args.steps, args.warmup)[args.only]
        print(json.dumps({"only": args.only, "scale": args.scale, "steps": args.steps, **result}), flush=True)
        return
    sampler = ClockSampler(local) if rank == 0 else None

    # ---- headline: add_rms_norm bf16, device-resident inputs, exactly K timed steps
    w = workloads.add_rms_norm_bf16(scale=args.scale)
    nbytes = w.algorithmic_bytes["add_rms_norm"]
    run, nsets = make_runner(w, device)
    for i in range(args.warmup):
        run(i)
    torch.cuda.synchronize(device)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize(device)
    launches_before = _lib.launch_count()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.time()
    start.record()
    for i in range(args.steps):
        run(i)
    end.record()
    torch.cuda.synchronize(device)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize(device)
    wall1 = time.time()
    launches = _lib.launch_count() - launches_before
    elapsed_ms = torch.tensor([start.elapsed_time(end)], device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(elapsed_ms, op=dist.ReduceOp.MAX)
    elapsed_ms = float(elapsed_ms.item())
    ms_per_step = elapsed_ms / args.steps
    value = world * w.tokens / (ms_per_step * 1e-3)
    achieved = nbytes / (ms_per_step * 1e-3) / 1e9
    if sampler is not None:
        sampler.mark(wall0, wall1)

    # ---- end to end: pinned host buffers in, both results back out, through the public host-tensor op
    from popcorn_b200 import host

    host_in = {k: w.inputs[k].pin_memory() for k in ("x", "residual")}
    weight_dev = w.inputs["weight"].to(device)
    host_out = [torch.empty_like(w.inputs["x"]).pin_memory() for _ in range(2)]
    h2d = sum(t.numel() * t.element_size() for t in host_in.values())
    d2h = sum(t.numel() * t.element_size() for t in host_out)

    def e2e_step() -> None:
        host.add_rms_norm_host(host_in["x"], host_in["residual"], weight_dev, w.args["eps"], w.args["offset"],
                               y=host_out[0], s=host_out[1], device=device)

    e2e_steps = max(3, min(args.steps, 10))
    # warm-up: the link idled during the device-only headline loop and needs a few hundred milliseconds of traffic
    # to run at full speed again (measured: the first 20 steps at half the rate of the later ones)
    for _ in range(30):
        e2e_step()
    torch.cuda.synchronize(device)
    # Five timed windows of e2e_steps steps each; the reported figure is the MEDIAN window (the PCIe path is shared
    # with the machine's other tenants: about one window in four runs at 60 % of the others), all five are listed.
    t0 = time.time()
    window_ms = []
    for _ in range(5):
        if dist is not None:
            dist.barrier()
        start.record()
        for _ in range(e2e_steps):
            e2e_step()
        end.record()
        torch.cuda.synchronize(device)
        one = torch.tensor([start.elapsed_time(end) / e2e_steps], device=device, dtype=torch.float64)
        if dist is not None:
            dist.barrier()
            dist.all_reduce(one, op=dist.ReduceOp.MAX)
        window_ms.append(float(one.item()))
    if sampler is not None:
        sampler.mark(t0, time.time())
    e2e_ms = torch.tensor([sorted(window_ms)[len(window_ms) // 2]], dtype=torch.float64)
    e2e_value = world * w.tokens / (float(e2e_ms.item()) * 1e-3)
    del host_in, host_out, run
    torch.cuda.empty_cache()

    # ---- the other configurations, per op (rank 0 reports its own GPU)
    per_op = {}
    if not args.skip_per_op and rank == 0:
        per_op = bench_single_kernel_ops(device, peak_gbs, sampler, ["rms_norm_fp32", "add_rms_norm_bf16", "rotary_bf16", "swiglu_bf16", "paired_rope_bf16"])
        per_op["moe_bf16"] = bench_moe(device, peak_gbs, sampler)
        if world == 1:
            torch_eager_incumbent(device, per_op, args.records)
            if not args.skip_incumbents:
                popcorn_incumbents(device, per_op)
            per_op["beyond_the_five_configs"] = bench_extra_ops(device, peak_gbs, sampler)
            per_op["moe_expert_mlp_bf16"] = bench_grouped_gemm(device, sampler)
            # the CPU reference of every configuration on a bounded token sample, beside the GPU number
            for key, fraction in (("rms_norm_fp32", 1.0), ("rotary_bf16", 1 / 8), ("swiglu_bf16", 1 / 8), ("moe_bf16", 1 / 64)):
                seconds, cpu_tokens, note = cpu_reference_time(key, fraction, repeats=3)
                cpu_rate = cpu_tokens / seconds
                per_op[key]["cpu_reference"] = {"tokens_per_s": round(cpu_rate, 1), "cores": os.cpu_count() or 1, "sample": note,
                                                "gpu_over_cpu": round(per_op[key]["tokens_per_s"] / cpu_rate, 1)}
    strong = None
    if dist is not None:
        dist.barrier()
        if not args.skip_per_op:
            full = torch.tensor([per_op[k]["ms"] if rank == 0 else 0.0 for k in
                                 ("rms_norm_fp32", "add_rms_norm_bf16", "rotary_bf16", "swiglu_bf16", "moe_bf16")], device=device, dtype=torch.float64)
            dist.broadcast(full, 0)
            full = {k: {"ms": v} for k, v in zip(("rms_norm_fp32", "add_rms_norm_bf16", "rotary_bf16", "swiglu_bf16", "moe_bf16"), full.tolist())}
            strong = bench_strong_scaling(device, world, rank, dist, peak_gbs, full)
            for exchange in ("nccl", "p2p"):
                try:
                    ep_result = bench_moe_expert_parallel(device, world, rank, dist, exchange)
                    ep_result["ep_check"] = expert_parallel_check(device, world, rank, dist, exchange)
                except Exception as error:  # symmetric memory may be unavailable on a given box: report, do not hide
                    ep_result = {"error": f"{type(error).__name__}: {error}"}
                if rank == 0:
                    per_op[f"moe_bf16_expert_parallel_{exchange}"] = ep_result

    if rank == 0:
        clocks = sampler.finish()
        cpu = None
        if world == 1 and not args.skip_per_op:
            cpu = cpu_headline_baseline()
        traffic = profiled_traffic_bytes()
        line = {
            "metric": "tokens_per_s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 5), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": headline_config(w.tokens),
            "roofline": {"bound": "hbm", "kernel": "rms_rows_kernel<bf16,256,4,add>", "achieved": round(achieved, 1), "peak": peak_gbs,
                         "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": round(achieved / peak_gbs, 4),
                         "frac_of_8tbs": round(achieved / SPEC_HBM_GBS, 4), "algorithmic_bytes_per_launch": nbytes,
                         "traffic": None if traffic is None else int(traffic * args.scale),
                         "per_config_frac_of_measured": per_config_fractions(per_op)},
            "cpu_baseline": cpu,
            "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "windows": len(window_ms), "rule": "median window",
                    "window_values": [round(world * w.tokens / (ms * 1e-3), 1) for ms in window_ms]},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "strong_scaling": strong,
            "per_op": per_op,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

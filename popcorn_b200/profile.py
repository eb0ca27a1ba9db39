"""Nsight Compute harness for the b200 kernels.

    python -m popcorn_b200.profile <configuration> [--scale S] [--sections ...] [--kernel REGEX] [--out FILE]

builds one benchmark configuration (popcorn_b200.workloads.CONFIGS, token count scaled by --scale), warms the op
up, then runs itself again under `ncu` with the capture scoped to one annotated call, the way popcorn's own
`popcorn profile <op>` does (src/popcorn/impls/_profile.py:32-40, 98-122).  Differences that matter on shared
machines: the same worker command is first run WITHOUT ncu and the capture only starts if that run exits 0; ncu
always gets `--clock-control none` (it must not lock the clocks of a GPU somebody else uses next); the number of
captured launches is bounded; the default workload is a fraction of the configuration that still exceeds L2.

For custom scripts: run them under `ncu --profile-from-start off --clock-control none` and wrap the region of
interest in `annotate()`.
"""

from __future__ import annotations

import argparse
import contextlib
import shutil
import subprocess
import sys
from collections.abc import Iterator

import torch

from popcorn_b200 import ops, workloads


@contextlib.contextmanager
def annotate() -> Iterator[None]:
    """The region ncu captures under --profile-from-start off (cudaProfilerStart / cudaProfilerStop)."""
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    try:
        yield
    finally:
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()


def runner(key: str, scale: float, device: torch.device):
    """A zero-argument callable that launches the kernels of configuration `key` once, inputs already on the device."""
    w = workloads.CONFIGS[key](scale=scale).to(device)
    i, a = w.inputs, w.args
    if key == "rms_norm_fp32":
        return lambda: ops.rms_norm(i["x"], i["weight"], None, a["eps"])
    if key == "add_rms_norm_bf16":
        return lambda: ops.add_rms_norm(i["x"], i["residual"], i["weight"], a["eps"], a["offset"])
    if key == "rotary_bf16":
        return lambda: ops.rotary_embedding_qk_(i["q"], i["k"], i["cos"], i["sin"])
    if key == "paired_rope_bf16":
        return lambda: ops.rope(i["q"], i["k"], i["cos"], i["sin"])
    if key == "swiglu_bf16":
        cols = a["cols"]
        return lambda: ops.swiglu(i["gate_up"][:, :cols], i["gate_up"][:, cols:])
    if key == "moe_bf16":
        def moe():
            idx, wts = ops.moe_route(i["router_logits"], a["top_k"])
            rows, _, _, _, pos = ops.moe_permute(i["x"], idx, a["experts"])
            return ops.moe_unpermute(rows, wts, pos)
        return moe
    raise SystemExit(f"unknown configuration {key!r}; choose from {sorted(workloads.CONFIGS)}")


def _worker(args: argparse.Namespace) -> None:
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    run = runner(args.configuration, args.scale, device)
    for _ in range(3):  # warm-up outside the capture
        run()
    print(f"profiling {args.configuration} at scale {args.scale}", file=sys.stderr)
    with annotate():
        run()


def main() -> None:
    parser = argparse.ArgumentParser(prog="python -m popcorn_b200.profile", description="Profile one configuration under Nsight Compute.")
    parser.add_argument("configuration", choices=sorted(workloads.CONFIGS))
    parser.add_argument("--scale", type=float, default=0.25, help="fraction of the configuration's tokens (keep captures small)")
    parser.add_argument("--sections", nargs="*", default=["SpeedOfLight", "MemoryWorkloadAnalysis"], help="ncu sections to collect")
    parser.add_argument("--kernel", help="ncu kernel-name regex filter")
    parser.add_argument("--launches", type=int, default=3, help="capture at most this many launches")
    parser.add_argument("--out", help="write an .ncu-rep file instead of printing to stdout")
    parser.add_argument("--worker", action="store_true", help=argparse.SUPPRESS)
    args = parser.parse_args()
    if args.worker:
        return _worker(args)
    ncu = shutil.which("ncu")
    if not ncu:
        raise SystemExit("ncu not found on PATH (load Nsight Compute or the CUDA toolkit module)")
    worker = [sys.executable, "-m", "popcorn_b200.profile", args.configuration, "--scale", str(args.scale), "--worker"]
    plain = subprocess.run(worker)
    if plain.returncode != 0:
        raise SystemExit(f"not profiled: the plain run exited {plain.returncode}")
    command = [ncu, "--profile-from-start", "off", "--clock-control", "none", "--launch-count", str(max(1, args.launches))]
    for section in args.sections:
        command += ["--section", section]
    if args.kernel:
        command += ["--kernel-name", f"regex:{args.kernel}"]
    if args.out:
        command += ["--force-overwrite", "--export", args.out]
    raise SystemExit(subprocess.run([*command, *worker]).returncode)


if __name__ == "__main__":
    main()

"""Benchmark-record rows in popcorn's report schema (version 3) for the `b200` backend.

popcorn's tuner picks a backend without being forced only if the op's report
store holds a usable row for it: status "pass", benchmarked, same torch version,
matching backend version and code fingerprints, and both `fwd_ms` and
`ref_fwd_ms` (src/popcorn/core/tuning.py:82-116).  Rows live one JSON object per
line in `$POPCORN_CACHE_DIR/v3/reports/<op>.jsonl` (src/popcorn/bench/store.py:62-72,
358-380); the row layout is `Record.to_dict()` (src/popcorn/bench/model.py:105-131)
and the case id is a SHA-1 over the canonical case (src/popcorn/core/config.py:54-64).

With popcorn installed next to a GPU, `KERNELS[op].benchmark(*args, backend="b200")`
lets popcorn's own harness measure and write such rows.  This module produces the
same rows from measurements taken WITHOUT popcorn in the process (bench.py on a box
that has only this package), so they can be dropped into a popcorn user's cache.
"""

from __future__ import annotations

import datetime
import hashlib
import json
import os
from pathlib import Path
from typing import Any

SCHEMA = 3
BACKEND = "b200"

# Fingerprints popcorn 0.1.1 computes for the references of its four ops, for the
# three op definitions in popcorn_b200/plugin.py, and for the dispatch predicates
# `plugin.PREDICATES` (the implementation hash of a bare external source is the hash of its predicate).  A row whose
# hashes differ from the live ones is ignored by popcorn as stale;
# tests/test_records.py recomputes them whenever popcorn is importable.
REFERENCE_HASHES = {
    "rms_norm": "520d99dddf52",
    "add_rms_norm": "efa7d047c69a",
    "rotary_embedding": "54089714d061",
    "rope": "1b989955d9be",
    "swiglu": "a2768d81c5aa",
    "geglu": "1bbe631dff25",
    "rms_norm_gated": "8c982cfacaf2",
    "l2_norm": "d283c2e0ec98",
    "layer_norm": "8a52ecd56f71",
    "moe_route": "3b877b7d155e",
    "moe_permute": "2d4425c300da",
    "moe_unpermute": "96a7326d99b2",
}
IMPLEMENTATION_HASH = "1c417c864f16"  # a bare source gated by one of plugin.PREDICATES (one closure body, so one hash)
# ops registered with their own predicate hash differently
IMPLEMENTATION_HASHES: dict[str, str] = {}


def implementation_hash(op: str) -> str:
    return IMPLEMENTATION_HASHES.get(op, IMPLEMENTATION_HASH)


def make_config(dims: dict[str, int], batch: list[int], dtype: str, args: dict[str, Any], present: list[str]) -> dict[str, Any]:
    """The canonical case dictionary (config.py:37-51): sorted dims and args, dtype without the `torch.` prefix."""
    return {"dims": dict(sorted(dims.items())), "batch": list(batch), "dtype": dtype.removeprefix("torch."),
            "args": dict(sorted(args.items())), "present": sorted(present)}


def config_id(config: dict[str, Any]) -> str:
    """12 hex digits of SHA-1 over the canonical payload (config.py:54-64)."""
    dtype = config["dtype"] if str(config["dtype"]).startswith("torch.") else f"torch.{config['dtype']}"
    payload = [
        tuple(sorted(config["dims"].items())), tuple(config["batch"]), dtype,
        tuple(sorted(config["args"].items())), sorted(config["present"]),
    ]
    return hashlib.sha1(json.dumps(payload, default=str).encode()).hexdigest()[:12]


def case_label(config: dict[str, Any]) -> str:
    """Human-readable case string in the format of Case.__str__ (model.py:27-32)."""
    parts = [f"{k}={v}" for k, v in config["dims"].items()]
    parts += [f"batch={tuple(config['batch'])}", config["dtype"]]
    parts += [f"{k}={v}" for k, v in config["args"].items()]
    parts += [f"+{name}" for name in sorted(config["present"])]
    return ",".join(parts)


def make_row(
    op: str, config: dict[str, Any], *, device: str, torch_version: str, fwd_ms: float, ref_fwd_ms: float,
    gauges: dict[str, dict[str, float]], reps: int, status: str = "pass", reason: str = "",
    peak_gb: float | None = None, ref_peak_gb: float | None = None, timestamp: str | None = None,
    grad_gauges: dict[str, dict[str, float]] | None = None, bwd_ms: float | None = None, ref_bwd_ms: float | None = None,
) -> dict[str, Any]:
    """One report row for the b200 implementation of `op` on the case `config`.

    Without `grad_gauges` it is an inference row (grad = False).  With them it is the training-call row of the same case
    (model.py:75-89: `grad` is part of the row's identity): per-input gradient gauges and the time of the backward pass
    alone next to the forward time, the pair popcorn's tuner adds up (tuning.py:54-61)."""
    bench = {"fwd_ms": fwd_ms, "ref_fwd_ms": ref_fwd_ms}
    if grad_gauges is not None:
        if bwd_ms is None or ref_bwd_ms is None:
            raise ValueError("a training-call row needs bwd_ms and ref_bwd_ms")
        bench.update(bwd_ms=bwd_ms, ref_bwd_ms=ref_bwd_ms)
    if peak_gb is not None:
        bench["fwd_peak_gb"] = peak_gb
    if ref_peak_gb is not None:
        bench["ref_fwd_peak_gb"] = ref_peak_gb

    def plain(table: dict[str, dict[str, float]] | None) -> dict[str, dict[str, float]]:
        return {name: {"err": g["err"], "budget": g["budget"], "scale": g["scale"]} for name, g in (table or {}).items()}

    return {
        "schema": SCHEMA, "op": op, "impl": BACKEND, "case": case_label(config), "case_id": config_id(config), "config": config,
        "device": device, "torch": torch_version, "backend_version": None,  # undeclared backend: no version gate
        "ts": timestamp or datetime.datetime.now(datetime.timezone.utc).isoformat(timespec="seconds"),
        "ref_hash": REFERENCE_HASHES.get(op), "impl_hash": implementation_hash(op),
        "status": status, "reason": reason, "grad": grad_gauges is not None,
        "fwd": plain(gauges), "bwd": plain(grad_gauges), "bench": bench, "benchmarked": True, "bench_error": "", "reps": reps,
    }


FLOORS = {"float64": 1e-10, "float32": 2e-5, "float16": 1e-3, "bfloat16": 2e-2}  # compare.py:14


def grade(dtype: str, gauges: dict[str, dict[str, float]], grad_gauges: dict[str, dict[str, float]] | None = None) -> tuple[str, str]:
    """popcorn's verdict on a set of gauges (model.py:66-71, compare.py:279-293): an output or gradient passes when its
    error against fp64 is at most twice the reference's own error or the dtype's floor times the size of the values.
    Returns (status, reason) for `make_row`."""
    floor = FLOORS.get(dtype.removeprefix("torch."), FLOORS["float32"])
    failures = []
    for prefix, table in (("", gauges), ("grad ", grad_gauges or {})):
        for name, g in table.items():
            if not g["err"] == g["err"] or g["err"] in (float("inf"), float("-inf")):
                failures.append(f"{prefix}{name}: err is non-finite")
            elif g["err"] > max(2 * g["budget"], floor * g["scale"]):
                failures.append(f"{prefix}{name}: err {g['err']:.3e} > max(2*{g['budget']:.3e}, {floor:.0e}*{g['scale']:.1f})")
    return ("fail", "; ".join(failures)) if failures else ("pass", "")


def row_key(row: dict[str, Any]) -> tuple[Any, ...]:
    """Identity of a row in popcorn's store (model.py:152-163)."""
    return (row["op"], row["impl"], row["device"], row["case_id"], row["grad"], row["torch"], row["backend_version"])


def reports_directory(root: str | os.PathLike[str] | None = None) -> Path:
    """popcorn's per-user report cache (store.py:62-72): <root>/v3/reports."""
    if root is None:
        root = os.getenv("POPCORN_CACHE_DIR") or Path(os.getenv("XDG_CACHE_HOME", Path.home() / ".cache")) / "popcorn"
    return Path(root).expanduser() / f"v{SCHEMA}" / "reports"


def write_rows(rows: list[dict[str, Any]], root: str | os.PathLike[str] | None = None) -> list[Path]:
    """Upsert rows into <root>/v3/reports/<op>.jsonl, newest row per key winning, keys sorted."""
    directory = reports_directory(root)
    directory.mkdir(parents=True, exist_ok=True)
    written = []
    for op in sorted({row["op"] for row in rows}):
        path = directory / f"{op}.jsonl"
        merged: dict[tuple[Any, ...], dict[str, Any]] = {}
        if path.exists():
            for line in path.read_text().splitlines():
                if line.strip():
                    old = json.loads(line)
                    merged[row_key(old)] = old
        for row in rows:
            if row["op"] == op and (row_key(row) not in merged or row["ts"] >= merged[row_key(row)]["ts"]):
                merged[row_key(row)] = row
        order = sorted(merged, key=lambda key: tuple("" if v is None else str(v) for v in key))
        temporary = path.with_name(f".{path.name}.{os.getpid()}.tmp")
        temporary.write_text("\n".join(json.dumps(merged[key], sort_keys=True) for key in order) + "\n")
        os.replace(temporary, path)
        written.append(path)
    return written


def benchmark_configs() -> dict[str, tuple[str, dict[str, Any]]]:
    """The benchmark configurations as popcorn cases: name -> (op, canonical config).

    The rotary configuration (bf16 activations with fp32 cos/sin) has no entry: popcorn cannot
    represent a call with mixed float dtypes as a case (config.py:96-99), so it keeps no rows for it."""
    return {
        "rms_norm_fp32": ("rms_norm", make_config({"normalized_shape": 4096}, [4096], "float32", {"eps": 1e-6}, [])),
        "add_rms_norm_bf16": ("add_rms_norm", make_config({"hidden": 8192}, [16384], "bfloat16", {"eps": 1e-5, "offset": 0.0}, [])),
        "swiglu_bf16": ("swiglu", make_config({"hidden": 14336}, [32768], "bfloat16", {}, [])),
    }

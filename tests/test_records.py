"""Report rows written by popcorn_b200.records are rows popcorn itself reads, trusts and ranks."""

import importlib.util
import json
import os
import warnings
from pathlib import Path

import pytest
import torch

from popcorn_b200 import records

REFERENCE_SRC = Path(os.environ.get("POPCORN_SOURCE_TREE", "/root/reference/src"))
HAVE_POPCORN = importlib.util.find_spec("popcorn") is not None or (REFERENCE_SRC / "popcorn").is_dir()


def example_row(op="add_rms_norm", name="add_rms_norm_bf16", device="NVIDIA B200", fwd_ms=0.157, ref_fwd_ms=2.9):
    _, config = records.benchmark_configs()[name]
    return records.make_row(op, config, device=device, torch_version=torch.__version__, fwd_ms=fwd_ms, ref_fwd_ms=ref_fwd_ms,
                            gauges={"0": {"err": 0.0156, "budget": 0.0156, "scale": 5.5}, "1": {"err": 0.0, "budget": 0.0, "scale": 7.1}}, reps=10)


def test_rows_round_trip_and_upsert(tmp_path):
    first = example_row(fwd_ms=0.2)
    first["ts"] = "2026-01-01T00:00:00+00:00"
    second = example_row(fwd_ms=0.157)
    second["ts"] = "2026-01-02T00:00:00+00:00"
    other = example_row("swiglu", "swiglu_bf16")
    records.write_rows([first, other], tmp_path)
    (path,) = [p for p in records.write_rows([second], tmp_path) if p.name == "add_rms_norm.jsonl"]
    assert path == tmp_path / "v3" / "reports" / "add_rms_norm.jsonl"
    rows = [json.loads(line) for line in path.read_text().splitlines()]
    assert len(rows) == 1 and rows[0]["bench"]["fwd_ms"] == 0.157  # the newer measurement replaced the older one
    assert rows[0]["schema"] == 3 and rows[0]["impl"] == "b200" and rows[0]["status"] == "pass" and rows[0]["benchmarked"]
    assert rows[0]["case"] == "hidden=8192,batch=(16384,),bfloat16,eps=1e-05,offset=0.0"
    assert (tmp_path / "v3" / "reports" / "swiglu.jsonl").exists()


@pytest.mark.skipif(not HAVE_POPCORN, reason="popcorn itself is not importable on this machine")
def test_popcorn_reads_and_ranks_the_rows(tmp_path, monkeypatch):
    if importlib.util.find_spec("popcorn") is None:
        monkeypatch.syspath_prepend(str(REFERENCE_SRC))
    monkeypatch.setenv("POPCORN_CACHE_DIR", str(tmp_path))
    warnings.filterwarnings("ignore")
    import popcorn
    from popcorn.bench.model import Case, Record
    from popcorn.core.config import config_id

    from popcorn_b200 import plugin

    plugin.register()
    # the committed fingerprints are the live ones
    for op_name, want in records.REFERENCE_HASHES.items():
        assert popcorn.KERNELS[op_name].fingerprint == want, f"{op_name}: reference fingerprint changed"
        assert popcorn.KERNELS[op_name]["b200"].fingerprint == records.implementation_hash(op_name), op_name
    # case ids and labels agree with popcorn's own
    for name, (op_name, config) in records.benchmark_configs().items():
        case = Case.from_config(config)
        assert case.config() == config and case.case_id == records.config_id(config) == config_id(config)
        assert str(case) == records.case_label(config)
    # popcorn parses the rows ...
    rows = [example_row(), example_row("swiglu", "swiglu_bf16", fwd_ms=0.43, ref_fwd_ms=3.5),
            example_row("rms_norm", "rms_norm_fp32", fwd_ms=0.0215, ref_fwd_ms=0.3)]
    for row in rows:
        parsed = Record.from_dict(row)
        assert parsed.to_dict() == row
    records.write_rows(rows, tmp_path)
    # ... and its tuner accepts them as usable timing samples of the b200 backend
    monkeypatch.setattr(torch.cuda, "get_device_name", lambda *a, **k: "NVIDIA B200", raising=False)
    for op_name in ("add_rms_norm", "swiglu", "rms_norm"):
        op = popcorn.KERNELS[op_name]
        op.tuner.forget()
        samples = [s for s in op.tuner.samples if s.impl == "b200"]
        assert len(samples) == 1, f"{op_name}: popcorn did not accept the row as evidence"
        assert samples[0].fwd_ms < samples[0].ref_fwd_ms

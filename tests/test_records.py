"""Report rows written by popcorn_b200.records are rows popcorn itself reads, trusts and ranks."""

import json

import pytest
import torch

from tests import popcorn_location
from popcorn_b200 import records



def example_row(op="add_rms_norm", name="add_rms_norm_bf16", device="NVIDIA B200", fwd_ms=0.157, ref_fwd_ms=2.9, training=False):
    _, config = records.benchmark_configs()[name]
    extra = {}
    if training:
        extra = dict(grad_gauges={"x": {"err": 0.03, "budget": 0.03, "scale": 9.0}, "weight": {"err": 0.5, "budget": 1.0, "scale": 300.0}},
                     bwd_ms=2 * fwd_ms, ref_bwd_ms=3 * ref_fwd_ms)
    return records.make_row(op, config, device=device, torch_version=torch.__version__, fwd_ms=fwd_ms, ref_fwd_ms=ref_fwd_ms,
                            gauges={"0": {"err": 0.0156, "budget": 0.0156, "scale": 5.5}, "1": {"err": 0.0, "budget": 0.0, "scale": 7.1}}, reps=10,
                            **extra)


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
    # the training-call row of the same case is a row of its own (grad is part of the key)
    training = example_row(training=True)
    assert training["grad"] and set(training["bwd"]) == {"x", "weight"} and training["bench"]["bwd_ms"] == 2 * 0.157
    records.write_rows([training], tmp_path)
    rows = [json.loads(line) for line in path.read_text().splitlines()]
    assert sorted(row["grad"] for row in rows) == [False, True]
    with pytest.raises(ValueError, match="bwd_ms"):
        records.make_row("swiglu", records.benchmark_configs()["swiglu_bf16"][1], device="d", torch_version="t", fwd_ms=1, ref_fwd_ms=2,
                         gauges={}, reps=1, grad_gauges={})


def test_grade_follows_popcorns_verdict():
    good = {"0": {"err": 0.03, "budget": 0.0156, "scale": 1.0}}       # within twice the reference's own error
    floor = {"x": {"err": 0.05, "budget": 0.0, "scale": 4.0}}        # within the bf16 floor (2e-2) times the scale
    bad = {"x": {"err": 0.2, "budget": 0.01, "scale": 4.0}}
    assert records.grade("bfloat16", good) == ("pass", "") and records.grade("torch.bfloat16", good, floor) == ("pass", "")
    status, reason = records.grade("bfloat16", good, bad)
    assert status == "fail" and reason.startswith("grad x: err 2.000e-01")
    assert records.grade("float32", floor)[0] == "fail" and records.grade("float32", {"0": {"err": float("nan"), "budget": 0, "scale": 1}})[0] == "fail"


@pytest.mark.skipif(not popcorn_location.available(), reason=popcorn_location.MISSING)
def test_popcorn_reads_and_ranks_the_rows(tmp_path, monkeypatch):
    popcorn = popcorn_location.import_popcorn(tmp_path, monkeypatch)
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
            example_row("rms_norm", "rms_norm_fp32", fwd_ms=0.0215, ref_fwd_ms=0.3), example_row(training=True)]
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
        assert len(samples) == (2 if op_name == "add_rms_norm" else 1), f"{op_name}: popcorn did not accept the row as evidence"
        assert all(s.fwd_ms < s.ref_fwd_ms for s in samples)
        if op_name == "add_rms_norm":  # the training-call sample carries the backward times too
            (training,) = [s for s in samples if s.grad]
            assert training.bwd_ms == 2 * 0.157 and training.ref_bwd_ms == 3 * 2.9

"""Host-side helpers of bench.py: column split per scaling mode, the recorded ncu traffic tied to the
kernel sources, the scaled error of the parity field."""
import json
import types

import pytest
import torch

import bench


def test_columns_per_gpu():
    args = types.SimpleNamespace(width=0, workload="propagation", scaling="strong")
    assert bench.widths_for(args, 1) == (256, 256)
    assert bench.widths_for(args, 4) == (256, 64)
    args.scaling = "weak"
    assert bench.widths_for(args, 4) == (1024, 256)
    args.scaling, args.width = "strong", 96
    assert bench.widths_for(args, 2) == (96, 48)
    with pytest.raises(AssertionError):
        bench.widths_for(args, 5)


def test_recorded_traffic_follows_the_kernel_sources(tmp_path, monkeypatch):
    record = tmp_path / "ncu_traffic.json"
    current = bench.kernel_source_hash()
    record.write_text(json.dumps({"captures": [
        {"workload": "propagation", "feature_width": 256, "dram_bytes_per_launch": 123, "captured": "then",
         "kernel_source_sha256": current},
        {"workload": "propagation", "feature_width": 128, "dram_bytes_per_launch": 456, "captured": "earlier",
         "kernel_source_sha256": "0" * 64}]}))
    monkeypatch.setattr(bench, "TRAFFIC_RECORD", record)
    assert bench.recorded_traffic("propagation", 256, 1)[0] == 123
    value, why = bench.recorded_traffic("propagation", 128, 1)          # captured from other sources
    assert value is None and "changed" in why
    assert bench.recorded_traffic("propagation", 64, 1)[0] is None      # never captured
    assert bench.recorded_traffic("propagation", 256, 2)[0] is None     # captures are single-GPU
    monkeypatch.setattr(bench, "TRAFFIC_RECORD", tmp_path / "absent.json")
    assert bench.recorded_traffic("propagation", 256, 1)[0] is None


def test_committed_traffic_record_is_well_formed():
    captures = json.loads(bench.TRAFFIC_RECORD.read_text())["captures"]
    assert {c["feature_width"] for c in captures} >= {256}
    for c in captures:
        assert c["dram_bytes_per_launch"] == c["dram_bytes_read"] + c["dram_bytes_write"]
        assert len(c["kernel_source_sha256"]) == 64


def test_scaled_error():
    ref = torch.tensor([[1.0, -2.0, 0.0], [100.0, 0.0, 0.0]])
    assert bench.scaled_error(ref.clone(), ref) == 0.0
    off = ref.clone()
    off[0, 2] += 1e-3      # a small entry is measured against the rms of its row, not against itself
    assert 0 < bench.scaled_error(off, ref) < 1e-3

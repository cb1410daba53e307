"""bench.py's reference arm runs anywhere (it is the CPU path) and prints the contract's JSON line."""

import json
import os
import subprocess
import sys

import conftest


def test_reference_arm_prints_one_json_line(tmp_path):
    cmd = [sys.executable, os.path.join(conftest.REPO_ROOT, "bench.py"), "--impl", "reference", "--layers", "1",
           "--steps", "1", "--warmup", "2", "--cpu-sample-gb", "0.05", "--ref-budget-s", "20", "--workdir", str(tmp_path / "w")]
    run = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    lines = [l for l in run.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["unit"] == "GB/s" and line["higher_is_better"] is True
    assert line["metric"] == "checkpoint_save_throughput" and line["value"] > 0
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    import ref_arm

    # the reference's own saver from oracle/_ref where that build exists, its restatement otherwise
    want_kind = "reference" if ref_arm.unavailable_reason() is None else "port"
    assert line["cpu_baseline"]["kind"] == want_kind and line["cpu_baseline"]["cores"] >= 1
    if want_kind == "reference":
        assert "buffer pool" in line["cpu_baseline"]["sample"] and line["cpu_baseline"]["ranks"] == 1
    assert "workload" in line["config"] and "model" not in line["config"]
    for key in ("n_gpus", "steps", "warmup", "ms_per_step", "scaling", "vs_baseline", "dtype", "data", "gpu_launches"):
        assert key in line


import pytest


@pytest.mark.gpu
def test_native_arm_prints_the_contract_line_with_every_leg():
    """The default single-GPU run on a small shard: save, restore, overlap probe and CPU baseline all
    run, and the line carries the roofline, end-to-end, baseline and clock keys."""
    cmd = [sys.executable, os.path.join(conftest.REPO_ROOT, "bench.py"), "--layers", "1", "--steps", "2", "--warmup", "3",
           "--cpu-sample-gb", "0.2"]
    run = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert run.returncode == 0, (run.stdout[-1500:], run.stderr[-3000:])
    lines = [l for l in run.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert "impl" not in line and line["n_gpus"] == 1 and line["steps"] == 2 and line["warmup"] == 3
    assert line["metric"] == "checkpoint_save_throughput" and line["unit"] == "GB/s" and line["value"] > 0
    assert line["gpu_launches"] == 2 and line["dtype"] == "u8" and line["scaling"] == "weak"
    roofline = line["roofline"]
    assert roofline["bound"] == "hbm" and roofline["unit"] == "GB/s" and 0 < roofline["frac"] < 1.2
    assert abs(roofline["frac"] - roofline["achieved"] / roofline["peak"]) < 1e-9
    assert line["e2e"]["value"] > 0 and line["e2e"]["d2h_bytes_per_step"] > line["config"]["payload_bytes_per_rank"] - 1
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["value"] > 0 and line["cpu_baseline"]["cores"] >= 1
    assert line["restore"]["bit_exact"] is True and line["parity_vs_oracle_prefix"] is True
    assert line["parity_vs_oracle"]["whole_object_sha256_equal"] is True
    if line["cpu_baseline"]["kind"] == "reference" and line["cpu_baseline"]["whole_shard"]:
        assert line["parity_vs_oracle"]["equal_to_reference_object"] is True
    assert line["restore"]["roofline"]["bound"] == "host_link" and 0 < line["restore"]["roofline"]["frac"] < 1.3
    assert line["hbm_held_bytes"] >= line["config"]["payload_bytes_per_rank"]
    assert 0 < line["host_link"]["frac_of_pinned_peak"] < 1.3
    assert line["overlap"]["gemm_batch_ms_alone"] > 0
    assert set(line["clocks"]) >= {"sm_mhz", "sm_max_mhz", "reasons"}

"""bench.py's reference arm runs anywhere (it is the CPU path) and prints the contract's JSON line."""

import json
import os
import subprocess
import sys

import conftest


def test_reference_arm_prints_one_json_line(tmp_path):
    cmd = [sys.executable, os.path.join(conftest.REPO_ROOT, "bench.py"), "--impl", "reference", "--layers", "1",
           "--steps", "1", "--warmup", "1", "--cpu-sample-gb", "0.05", "--workdir", str(tmp_path / "w")]
    run = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    lines = [l for l in run.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["unit"] == "GB/s" and line["higher_is_better"] is True
    assert line["metric"] == "checkpoint_save_throughput" and line["value"] > 0
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert "workload" in line["config"] and "model" not in line["config"]
    for key in ("n_gpus", "steps", "warmup", "ms_per_step", "scaling", "vs_baseline", "dtype", "data", "gpu_launches"):
        assert key in line

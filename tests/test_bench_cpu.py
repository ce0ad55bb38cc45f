"""The reference arm of bench.py runs on the host cores: its JSON line carries the keys the
bench contract names, on a sample small enough for the CPU suite."""
import json
import os
import subprocess
import sys

from conftest import ROOT


def test_reference_arm_prints_one_contract_line(reference):
    env = dict(os.environ, OMP_NUM_THREADS="2")
    result = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                             "--steps", "2", "--warmup", "1", "--rows", "4096"],
                            capture_output=True, text=True, env=env, timeout=300, cwd=ROOT)
    assert result.returncode == 0, result.stderr[-2000:]
    lines = [line for line in result.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step",
                "higher_is_better", "scaling", "vs_baseline", "dtype", "data", "config",
                "cpu_baseline", "e2e", "gpu_launches"):
        assert key in line, key
    assert line["metric"] == "q8_0_gemv_weight_bandwidth" and line["unit"] == "GB/s"
    assert line["steps"] == 2 and line["warmup"] == 1 and line["higher_is_better"] is True
    assert line["value"] > 0 and line["vs_baseline"] is None
    assert line["cpu_baseline"]["kind"] in ("reference", "port")
    assert line["cpu_baseline"]["value"] == line["value"]
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}
    assert "workload" in line["config"]


def test_gpu_arm_refuses_to_run_without_a_device():
    import torch
    if torch.cuda.is_available():
        return
    result = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "1",
                             "--warmup", "1"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert result.returncode != 0
    assert "no CPU fallback" in (result.stderr + result.stdout)

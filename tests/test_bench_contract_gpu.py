"""bench.py on one GPU (one layer, two steps) prints the JSON line of the benchmark contract."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_gpu_arm_prints_the_contract_line():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--layers", "wo", "--steps", "2", "--warmup", "3",
                          "--quick"],
                         capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches", "roofline", "cpu_baseline"):
        assert key in line, key
    assert line["n_gpus"] == 1 and line["steps"] == 2 and line["warmup"] == 3 and line["scaling"] == "weak"
    assert line["value"] > 0 and line["vs_baseline"] is None and line["data"] == "synthetic"
    assert line["gpu_launches"] == 2 * 9  # per step and layer: 3 amax, 3 casts, 3 GEMMs
    roof = line["roofline"]
    assert roof["bound"] == "tensor" and roof["unit"] == "TFLOP/s" and 0 < roof["frac"] < 1.5
    assert abs(roof["frac"] - roof["achieved"] / roof["peak"]) < 1e-9 and roof["traffic"] > 0
    assert roof["traffic"] >= 0.9 * roof["traffic_algorithmic"]
    e2e = line["e2e"]
    assert e2e["value"] > 0 and e2e["h2d_bytes_per_step"] == 2 * 2 * 16384 * 8192 and e2e["d2h_bytes_per_step"] > 0
    assert e2e["value"] < line["value"]  # the copies are inside its timed region
    cpu = line["cpu_baseline"]
    assert cpu["kind"] in ("port", "reference") and cpu["cores"] >= 1 and cpu["value"] > 0 and "sample" in cpu
    assert set(line["clocks"]) >= {"sm_mhz", "sm_max_mhz", "reasons"}
    assert "workload" in line["config"]

"""CPU test of the benchmark's reference arm: `bench.py --impl reference` times the reference engine's own CPU path on the
host cores and must print one JSON line with the keys the comparison needs (same metric, unit and workload as the CUDA arm)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "2", "--warmup", "1"], cwd=ROOT,
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    line = json.loads(p.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    if "unavailable" in line:  # the compiled reference is not in the tree (it is built where the reference sources are)
        assert isinstance(line["unavailable"], str) and line["unavailable"]
        return
    assert line["metric"] == "attention TFLOP/s" and line["unit"] == "TFLOP/s" and line["higher_is_better"] is True
    assert line["n_gpus"] == 1 and line["steps"] == 2 and line["warmup"] == 1 and line["ms_per_step"] > 0
    assert line["value"] > 0 and line["vs_baseline"] is None and line["data"] == "synthetic"
    assert line["config"]["workload"].startswith("config 4")
    cb = line["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["value"] == line["value"] and cb["sample"]
    e2e = line["e2e"]
    assert e2e["value"] == line["value"] and e2e["unit"] == line["unit"]
    assert e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0


import pytest


@pytest.mark.gpu
def test_cuda_arm_prints_the_contract_line():
    """The CUDA arm on one GPU, shortened (three steps, no extra legs, no two-second sustained run): every key the line must
    carry is there and means what it says."""
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "3", "--warmup", "3", "--no-extra", "--sustained", "0"], cwd=ROOT,
                       capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    line = json.loads(p.stdout.strip().splitlines()[-1])
    assert "impl" not in line or line["impl"] != "reference"
    assert line["metric"] == "attention TFLOP/s" and line["unit"] == "TFLOP/s" and line["higher_is_better"] is True
    assert line["n_gpus"] == 1 and line["steps"] == 3 and line["warmup"] == 3 and line["dtype"] == "bf16" and line["data"] == "synthetic"
    assert line["config"]["workload"].startswith("config 4") and "l2" in line["config"]
    assert line["gpu_launches"] >= 3
    flops = 4 * 4 * 16 * 8192 * 8192 * 128
    assert abs(line["value"] - flops / (line["ms_per_step"] * 1e-3) / 1e12) < 1e-6 * line["value"]
    roof = line["roofline"]
    assert roof["bound"] == "tensor" and roof["unit"] == "TFLOP/s" and 0.3 < roof["frac"] < 1.1
    assert abs(roof["frac"] - roof["achieved"] / roof["peak"]) < 1e-9 and roof["traffic"] > 0
    e2e = line["e2e"]
    assert 0 < e2e["value"] < line["value"]  # host buffers and both copies inside the timed region
    assert e2e["h2d_bytes_per_step"] == 3 * 4 * 16 * 8192 * 128 * 2 and e2e["d2h_bytes_per_step"] == 4 * 16 * 8192 * 128 * 2
    cb = line["cpu_baseline"]
    assert cb["value"] > 0 and cb["unit"] == "TFLOP/s" and cb["cores"] >= 1 and cb["kind"] in ("reference", "port")
    ck = line["clocks"]
    assert "sm_mhz" in ck and "sm_max_mhz" in ck and isinstance(ck["reasons"], list)

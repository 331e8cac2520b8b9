"""The one JSON line bench.py prints: keys and basic consistency, for the CPU arm (runs anywhere)
and for the device arm (needs a GPU)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASE_KEYS = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline", "dtype",
             "data", "config", "e2e", "cpu_baseline"}


def run_bench(*args, timeout=600):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], cwd=ROOT, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.strip().splitlines() if l.startswith("{")]
    assert len(lines) == 1, "exactly one JSON line on stdout"
    return json.loads(lines[0])


def test_reference_arm_line():
    d = run_bench("--impl", "reference", "--steps", "1", "--warmup", "1")
    assert BASE_KEYS <= set(d), BASE_KEYS - set(d)
    assert d["impl"] == "reference" and d["higher_is_better"] is True and d["unit"] == "samples/s"
    assert d["value"] > 0 and "workload" in d["config"]
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("port", "reference") and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


@pytest.mark.gpu
def test_device_arm_line():
    d = run_bench("--steps", "10", "--warmup", "3", "--no-configs")
    assert BASE_KEYS | {"roofline", "clocks", "gpu_launches", "value_spread", "kernels_per_step"} <= set(d)
    assert d["n_gpus"] == 1 and d["steps"] == 10 and d["warmup"] == 3 and d["dtype"] == "f32" and d["vs_baseline"] is None
    assert abs(d["value"] - 8192 / (d["ms_per_step"] * 1e-3)) <= 1e-6 * d["value"]
    assert d["gpu_launches"] == d["kernels_per_step"] * d["steps"] > 0
    sp = d["value_spread"]
    assert sp["ms_per_step_min"] <= d["ms_per_step"] <= sp["ms_per_step_max"]
    r = d["roofline"]
    assert r["bound"] in ("hbm", "tensor") and r["unit"] in ("GB/s", "TFLOP/s")
    assert abs(r["frac"] - r["achieved"] / r["peak"]) <= 1e-9 and 0 < r["frac"] < 1.5
    e = d["e2e"]
    assert e["h2d_bytes_per_step"] == 8192 * 784 * 4 + 8192 * 8 and e["d2h_bytes_per_step"] == 4
    assert 0 < e["value"] < d["value"]  # the host-fed run cannot beat the device-resident one
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["value"] > 0 and cb["cores"] >= 1
    assert d["clocks"]["sm_max_mhz"] >= d["clocks"]["sm_mhz"] > 0

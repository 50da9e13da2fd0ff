"""bench.py prints one JSON line with the agreed keys: the CPU reference arm here, the GPU arm on a B200."""
import json
import os
import subprocess
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run_bench(*flags):
    proc = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), *flags], cwd=REPO, capture_output=True,
                          text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, proc.stdout[-2000:]
    return json.loads(lines[0])


COMMON = ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
          "vs_baseline", "dtype", "data", "config", "e2e", "cpu_baseline")


def test_reference_arm_line():
    d = _run_bench("--impl", "reference", "--steps", "2", "--warmup", "1")
    assert d["steps"] == 2 and d["warmup"] == 1  # both honoured as given
    assert set(d["config"]) == {"workload", "B_per_gpu", "H", "N", "D", "mask", "keep_prob", "step", "l2", "sharding"}
    for key in COMMON + ("impl",):
        assert key in d, key
    assert d["impl"] == "reference" and d["n_gpus"] == 1 and d["vs_baseline"] is None
    assert d["metric"] == "effective_tflops_dense_equiv" and d["unit"] == "TFLOP/s" and d["higher_is_better"] is True
    assert d["config"]["workload"].startswith("cfg2_headline")
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["sample"] and cb["value"] == d["value"] > 0
    e2e = d["e2e"]
    assert e2e["value"] == d["value"] and e2e["unit"] == d["unit"]
    assert e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0


@pytest.mark.gpu
def test_gpu_arm_line():
    d = _run_bench("--steps", "3", "--warmup", "3", "--repeats", "4", "--no-cpu-baseline", "--no-extras")
    for key in COMMON[:-1] + ("gpu_launches", "clocks", "roofline", "roofline_pack"):
        assert key in d, key
    assert "impl" not in d or d["impl"] != "reference"
    assert d["n_gpus"] == 1 and d["steps"] == 3 and d["scaling"] == "weak" and d["vs_baseline"] is None
    assert d["dtype"] == "f16" and d["data"] == "synthetic"
    assert d["repeats"] == 4 and len(d["timing"]["step_us_per_rank"]) == 1
    assert d["gpu_launches"] == 2 * d["steps"] * d["repeats"]  # one pack and one attention launch per step
    assert d["value"] > 0 and d["ms_per_step"] > 0
    e2e = d["e2e"]
    assert e2e["value"] > 0 and e2e["unit"] == d["unit"]
    assert e2e["h2d_bytes_per_step"] == 16 * 12 * 512 * (3 * 64 * 2 + 512)  # q, k, v (fp16) and the bool mask
    assert e2e["d2h_bytes_per_step"] == 16 * 12 * 512 * 64 * 2
    assert e2e["value"] < d["value"]  # the copies over PCIe dominate the end-to-end call
    for name, bound, unit in (("roofline", "tensor", "TFLOP/s"), ("roofline_pack", "hbm", "GB/s")):
        r = d[name]
        assert r["bound"] == bound and r["unit"] == unit and r["peak"] > 0
        assert abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-9
        assert 0 < r["frac"] < 1.2 and r["traffic"] > 0 and r["traffic_source"].startswith("profiles/")
        b2b = r["back_to_back"]
        assert 0 < b2b["ms_per_launch"] and abs(b2b["frac"] - b2b["achieved"] / r["peak"]) < 1e-9
    clocks = d["clocks"]
    assert clocks["sm_max_mhz"] >= clocks["sm_mhz"] > 0 and isinstance(clocks["reasons"], list)

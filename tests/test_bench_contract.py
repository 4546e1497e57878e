"""bench.py's reference arm (the reference's CPU GEMM on the host cores) runs without a GPU: its one JSON line must
carry the keys the benchmark contract names.  The GPU arm's line is checked on the GPU box."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, timeout=600):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                       timeout=timeout, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, r.stdout[-2000:]
    return json.loads(lines[0])


def test_reference_arm_line():
    d = _run("--impl", "reference", "--workload", "c4:192x160x128", "--steps", "2", "--warmup", "1")
    assert d["impl"] == "reference" and d["metric"] == "sgemm_tflops" and d["unit"] == "TFLOP/s"
    assert d["n_gpus"] == 1 and d["steps"] == 2 and d["warmup"] == 1 and d["higher_is_better"] is True
    assert d["value"] > 0 and d["ms_per_step"] > 0 and d["vs_baseline"] is None and d["dtype"] == "f32"
    assert d["config"]["workload"] == "c4:192x160x128"
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["gpu_launches"] == 0


@pytest.mark.gpu
def test_gpu_arm_line():
    d = _run("--workload", "c4:1024x1024x1024", "--steps", "5", "--warmup", "3")
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "roofline", "cpu_baseline", "clocks", "e2e", "gpu_launches"):
        assert key in d, key
    assert d["value"] > 1.0 and d["gpu_launches"] >= 5 and d["config"]["workload"] == "c4:1024x1024x1024"
    r = d["roofline"]
    assert set(("bound", "achieved", "peak", "unit", "frac", "traffic")) <= set(r) and 0 < r["frac"] < 1.2
    e = d["e2e"]
    assert e["value"] > 0 and e["h2d_bytes_per_step"] == 2 * 1024 * 1024 * 4 and e["d2h_bytes_per_step"] == 1024 * 1024 * 4
    assert d["cpu_baseline"]["value"] > 0 and d["tf32x3"]["status"] == 0

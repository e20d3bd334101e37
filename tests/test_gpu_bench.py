"""The benchmark's output line: every key the measurement contract names, on a cut-down run."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _line(*args):
    res = subprocess.run([sys.executable, "bench.py", *args], capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert res.returncode == 0, res.stdout + res.stderr
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, res.stdout                     # exactly one JSON line
    return json.loads(lines[0])


def test_bench_line_has_the_contract_keys():
    d = _line("--layers", "2", "--steps", "3", "--warmup", "3", "--cpu-seconds", "1")
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "roofline", "cpu_baseline", "e2e", "gpu_launches", "clocks"):
        assert key in d, key
    assert d["n_gpus"] == 1 and d["steps"] == 3 and d["warmup"] == 3 and d["higher_is_better"] is True
    assert d["scaling"] == "weak" and d["vs_baseline"] is None and d["data"] == "synthetic" and "workload" in d["config"]
    r = d["roofline"]
    assert r["bound"] == "hbm" and r["unit"] == "GB/s" and r["achieved"] > 1000 and abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-9
    assert r["traffic"] >= r["algorithmic_bytes_per_launch"] and r["launches_timed"] == 3 * 2
    e = d["e2e"]
    assert e["value"] > 0 and e["h2d_bytes_per_step"] == 2 * (2 * 64 * 8 * 128 * 2 + 64 * 32 * 128 * 2)
    assert e["d2h_bytes_per_step"] == 2 * 64 * 32 * 128 * 2
    c = d["cpu_baseline"]
    assert c["kind"] == "port" and c["cores"] >= 1 and c["value"] > 0
    assert 3 * 2 <= d["gpu_launches"] <= 3 * (2 + 1)       # per step: one fused kernel per layer (+ the table patch)
    assert d["clocks"]["sm_max_mhz"] > 0

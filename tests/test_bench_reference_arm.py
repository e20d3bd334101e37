"""`bench.py --impl reference`: the CPU arm's output line (needs no GPU)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _line(*args, env=None):
    res = subprocess.run([sys.executable, "bench.py", *args], capture_output=True, text=True, timeout=900, cwd=ROOT,
                         env=dict(os.environ, **(env or {})))
    assert res.returncode == 0, res.stdout + res.stderr
    return [l for l in res.stdout.splitlines() if l.startswith("{")]


def test_reference_arm_line():
    lines = _line("--impl", "reference", "--steps", "1", "--warmup", "0")
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["value"] > 0 and d["cpu_baseline"]["kind"] == "port"
    assert d["metric"] == "paged_decode_steps_per_s" and d["higher_is_better"] is True and d["steps"] == 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0 and d["e2e"]["value"] == d["value"]


def test_reference_arm_uses_the_host_cores_under_a_launcher_that_pins_one_thread():
    """torchrun exports OMP_NUM_THREADS=1 to every rank; the CPU arm must still use the cores it may run on."""
    lines = _line("--impl", "reference", "--steps", "1", "--warmup", "0",
                  env={"OMP_NUM_THREADS": "1", "RANK": "0", "WORLD_SIZE": "2", "LOCAL_RANK": "0"})
    d = json.loads(lines[0])
    assert d["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))


def test_reference_arm_is_silent_on_other_ranks():
    assert _line("--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0",
                 env={"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}) == []

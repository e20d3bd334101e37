"""Multi-GPU runs (skipped unless at least 2 GPUs are visible): the long-context split with the
NCCL exchange of partials, and the benchmark's by-sequence sharding."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(n, script, *args):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29517", script, *args]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env, cwd=ROOT)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_long_context_split_over_two_gpus():
    res = _torchrun(2, "tests/multi_gpu/long_context_worker.py", "--tokens", "32768", "--layers", "2", "--steps", "3")
    assert res.returncode == 0, res.stdout + res.stderr
    line = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    assert line["ok"] and line["n_gpus"] == 2


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_long_context_peer_exchange_over_two_gpus():
    """The exchange as one kernel over peer memory (CUDA IPC mailboxes): same bytes as the all-gather route."""
    res = _torchrun(2, "tests/multi_gpu/long_context_worker.py", "--tokens", "32768", "--layers", "2", "--steps", "3",
                    "--exchange", "peer")
    assert res.returncode == 0, res.stdout + res.stderr
    line = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    assert line["ok"] and line["n_gpus"] == 2 and line["exchange"] == "peer" and line["same_bytes_as_all_gather_route"]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_long_context_peer_exchange_mixed_routes_over_two_gpus():
    """Rank 0: attention kernel carries the exchange (one launch); rank 1: rows, then the exchange kernel."""
    res = _torchrun(2, "tests/multi_gpu/long_context_worker.py", "--tokens", "32768", "--layers", "2", "--steps", "3",
                    "--exchange", "peer", "--mixed")
    assert res.returncode == 0, res.stdout + res.stderr
    line = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    assert line["ok"] and line["exchange"] == "peer" and line["same_bytes_as_all_gather_route"]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_long_context_with_cold_tier_over_two_gpus():
    # hot window of 16384 over 32768 tokens: rank 0's pages live in pinned host memory
    res = _torchrun(2, "tests/multi_gpu/long_context_worker.py", "--tokens", "32768", "--layers", "3", "--steps", "3",
                    "--hot-window", "16384")
    assert res.returncode == 0, res.stdout + res.stderr
    line = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    assert line["ok"] and line["rank0_stats"]["pages_cold"] == 1024 and line["rank0_stats"]["prefetch_hits"] > 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_long_context_peer_exchange_with_cold_tier_over_two_gpus():
    """Rank 0 reads its pages through the cold tier (milliseconds per layer) while rank 1's merging CTAs wait
    for its rows inside their attention kernel: the bounded wait must simply be long enough."""
    res = _torchrun(2, "tests/multi_gpu/long_context_worker.py", "--tokens", "32768", "--layers", "3", "--steps", "3",
                    "--hot-window", "16384", "--exchange", "peer")
    assert res.returncode == 0, res.stdout + res.stderr
    line = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    assert line["ok"] and line["rank0_stats"]["pages_cold"] == 1024 and line["same_bytes_as_all_gather_route"]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_bench_shards_by_sequence_over_two_gpus():
    res = _torchrun(2, "bench.py", "--gpus", "2", "--steps", "3", "--warmup", "3", "--layers", "4", "--no-cpu")
    assert res.returncode == 0, res.stdout + res.stderr
    line = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    assert line["n_gpus"] == 2 and line["value"] > 0 and line["scaling"] == "weak"

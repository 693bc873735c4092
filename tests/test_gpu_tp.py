"""Tensor-parallel decode against the single-GPU engine (bit-identical token streams and logits).
The worker runs in child processes: alone (world 1: the sharding code with one shard) and, when two GPUs are
visible, as two NCCL ranks (kernel runs between collectives replayed as CUDA graphs)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def run_worker(n_ranks, graph):
    env = dict(os.environ, TP_GRAPH=str(graph), NCCL_NVLS_ENABLE="0")
    if n_ranks == 1:
        cmd = [sys.executable, str(ROOT / "tests" / "tp_worker.py")]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n_ranks}", "--master-addr", "127.0.0.1",
               "--master-port", "29533", str(ROOT / "tests" / "tp_worker.py")]
    r = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0 and "TP_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-3000:])


@pytest.mark.parametrize("graph", [0, 1])
def test_one_shard_equals_engine(graph):
    run_worker(1, graph)


def test_two_ranks_equal_engine():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    run_worker(2, 1)

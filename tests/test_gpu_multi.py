"""GPU, 2 ranks over NCCL: split-N and expert-parallel shards joined by the
package's collectives equal the one-GPU result bit for bit, eagerly and inside a
CUDA graph.  Needs two GPUs in the box; on a one-GPU box the same partitions are
covered by test_sharding_cpu.py (gloo ranks, oracle arithmetic)."""
from __future__ import annotations

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.timeout(600)
def test_shards_join_bit_exact_over_nccl():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip(f"needs 2 GPUs, this box has {n}")
    env = dict(os.environ, NCCL_DEBUG="WARN")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29617",
           os.path.join(HERE, "multi_gpu_worker.py")]
    run = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=540)
    tail = (run.stdout + run.stderr)[-4000:]
    assert run.returncode == 0, tail
    assert "MULTI_GPU_OK 0" in run.stdout and "MULTI_GPU_OK 1" in run.stdout, tail

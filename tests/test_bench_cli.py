"""CPU: the benchmark's reference arm runs here (it is the CPU port) and prints the
contract's JSON line; the GPU arm refuses to run without a device instead of falling
back.  Keeps bench.py importable and its argument handling honest between GPU runs."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, timeout=300):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True,
                          text=True, timeout=timeout, cwd=ROOT)


@pytest.mark.timeout(400)
def test_reference_arm_prints_the_contract_line():
    run = _run("--impl", "reference", "--steps", "1", "--warmup", "1")
    assert run.returncode == 0, run.stderr[-2000:]
    line = json.loads([l for l in run.stdout.splitlines() if l.startswith("{")][-1])
    assert line["impl"] == "reference" and line["unit"] == "GB/s" and line["higher_is_better"] is True
    assert line["metric"] == "coded GEMV compressed-weight GB/s"
    assert line["config"]["workload"] == "dense27b_layer_decode_b1"
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}
    assert line["value"] > 0 and line["steps"] == 1 and line["gpu_launches"] == 0


def test_gpu_arm_refuses_to_run_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    run = _run("--steps", "1")
    assert run.returncode != 0
    assert "needs a CUDA device" in (run.stderr + run.stdout)

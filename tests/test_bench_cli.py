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


def test_clock_sampler_reads_a_fake_nvidia_smi(tmp_path, monkeypatch):
    """The sampler starts the timed region only after the first sample, takes rows of every
    GPU of the job from one process, reports the median SM clock and the throttle reasons
    it saw, and an inactive sampler (ranks other than 0) starts nothing."""
    import importlib.util
    fake = tmp_path / "nvidia-smi"
    fake.write_text(
        "#!/bin/sh\n"
        "while true; do\n"
        "  echo '0, 1965, 1965, 412.5, Not Active, Not Active, Not Active, Not Active'\n"
        "  echo '1, 1935, 1965, 988.0, Not Active, Not Active, Not Active, Active'\n"
        "  sleep 0.02\n"
        "done\n")
    fake.chmod(0o755)
    monkeypatch.setenv("PATH", f"{tmp_path}{os.pathsep}{os.environ['PATH']}")
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    with bench.ClockSampler([0, 1]) as clocks:
        assert clocks.rows, "the region must not start before the first sample"
    got = clocks.summary()
    assert got["samples"] >= 2 and got["sm_max_mhz"] == 1965.0
    assert 1935.0 <= got["sm_mhz"] <= 1965.0
    assert got["reasons"] == ["sw_power_cap"]
    with bench.ClockSampler([0, 1], active=False) as idle:
        pass
    assert idle.summary() == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}

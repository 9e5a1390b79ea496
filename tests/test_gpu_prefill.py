"""GPU parity of the prefill coded GEMM (channel-major decode into tensor memory, or into
shared memory with ESCHA_B200_TC_WEIGHTS=smem; tcgen05.mma with fp32 accumulators in
tensor memory) against the CPU oracle's float64 product of
reference-decoded weights, against the register-fragment tensor-core kernel, and
through the dense module.  Mirrors the reference's tests/test_gemm_mat.py bar:
tolerance-equal to the per-row kernel, deterministic run to run."""
from __future__ import annotations

import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from cases import rel_err
from escha_mlx_b200 import dense, msl, synth
from escha_mlx_b200._lib import lib

pytestmark = pytest.mark.gpu

GEMV_TOL = 1e-3      # max rel error vs f64 product of reference-decoded weights


def dev(a, device):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def host(t):
    return t.detach().cpu().numpy()


@pytest.mark.parametrize("K,IC,OC,M,splits", [
    (2, 128, 128, 1, 1),        # one chunk pair, one row
    (2, 256, 128, 48, 1),
    (3, 512, 256, 128, 1),      # exactly one row tile
    (3, 512, 256, 129, 2),      # ragged second row tile, two planes
    (2, 1024, 384, 256, None),  # policy split
    (3, 768, 128, 300, 3),      # more than 256 rows: second pass over the weights
    (2, 4096, 256, 64, 4),
    (3, 256, 128, 20, 3),       # more splits than 128-channel stages: shared-memory-operand kernel
    (3, 1280, 256, 256, 1),     # ten stages: every ring wraps
])
def test_prefill_gemm_vs_oracle(cuda, oracle, K, IC, OC, M, splits):
    rng = np.random.default_rng(K * 1000 + IC + M)
    code, _, _ = synth.coded_projection(rng, IC, OC, K)
    xh = (rng.standard_normal((M, IC)) * 0.25).astype(np.float16)
    c, xd = msl.code_tensor(code, cuda), dev(xh, cuda)
    mid = msl.dense_gemm_tc(xd, c, K, IC, OC, splits=splits)
    torch.cuda.synchronize()
    assert lib.escha_coded_gemm_tc_status() == 0
    want = oracle.gemv_f64(xh, code, None, K, IC, OC)
    assert rel_err(host(mid), want) < GEMV_TOL
    # bit-reproducible, and tolerance-equal to the register-fragment kernel
    assert torch.equal(msl.dense_gemm_tc(xd, c, K, IC, OC, splits=splits), mid)
    assert rel_err(host(mid), host(msl.dense_gemv(xd, c, K, IC, OC))) < 2e-5


def test_prefill_rejects_bad_arguments(cuda):
    xh = torch.zeros((4, 256), dtype=torch.float16, device=cuda)
    code = torch.zeros((16, 8, 16), dtype=torch.int32, device=cuda)
    with pytest.raises(ValueError, match="splits=9 exceeds"):
        msl.dense_gemm_tc(xh, code, 2, 256, 128, splits=9)
    with pytest.raises(ValueError, match="at least one row"):
        msl.dense_gemm_tc(xh[:0], code, 2, 256, 128)


@pytest.mark.parametrize("M", [16, 48, 200])
def test_dense_linear_prefill_path(cuda, oracle, monkeypatch, M):
    """EschaLinear at prefill row counts (input transform, tcgen05 product, output
    transform) against the oracle's full linear."""
    monkeypatch.delenv("ESCHA_MLX_GEMV", raising=False)
    rng = np.random.default_rng(M)
    K, IC, OC = 3, 512, 384
    code, rin, rout = synth.coded_projection(rng, IC, OC, K)
    x = synth.activations(rng, M, IC)
    lin = dense.EschaLinear(dense.EschaWeight(code, rin, rout, device=cuda))
    assert msl.use_prefill_kernel(M)
    y = lin(dev(x, cuda))
    ri, ro = oracle.fold_scales(rin, rout)
    want = oracle.dense_linear(x, code, ri, ro, K)
    assert rel_err(host(y), want) < 2e-3
    assert torch.equal(lin(dev(x, cuda)), y)
    a, b = dense.project_pair(lin, lin, dev(x, cuda))
    assert torch.equal(a, y) and torch.equal(b, y)


@pytest.mark.parametrize("splits", [1, 3])
def test_prefill_fused_output_equals_separate_transform(cuda, splits):
    rng = np.random.default_rng(splits)
    K, IC, OC, M = 3, 768, 256, 100
    code, _, rout = synth.coded_projection(rng, IC, OC, K)
    xh = (rng.standard_normal((M, IC)) * 0.25).astype(np.float16)
    c, xd = msl.code_tensor(code, cuda), dev(xh, cuda)
    ro = dev(rout.astype(np.float32), cuda)
    fused = msl.dense_gemm_tc(xd, c, K, IC, OC, splits=splits, rout=ro)
    separate = msl.dense_scaled_had_out(msl.dense_gemm_tc(xd, c, K, IC, OC, splits=splits), ro, msl.RS)
    assert torch.equal(fused, separate)


ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SMEM_CHILD = r"""
import sys
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + "/tests")
import numpy as np, torch
from escha_mlx_b200 import msl, synth
from escha_mlx_b200._lib import lib
from oracle import escha_oracle as oracle
dev = torch.device("cuda", 0)
worst = 0.0
for K, IC, OC, M, S in ((2, 1024, 256, 200, 1), (3, 768, 128, 300, 3)):
    rng = np.random.default_rng(K + M)
    code, rin, rout = synth.coded_projection(rng, IC, OC, K)
    xh = (rng.standard_normal((M, IC)) * 0.25).astype(np.float16)
    mid = msl.dense_gemm_tc(torch.from_numpy(xh).to(dev), msl.code_tensor(code, dev), K, IC, OC, splits=S)
    torch.cuda.synchronize()
    assert lib.escha_coded_gemm_tc_status() == 0
    want = oracle.gemv_f64(xh, code, None, K, IC, OC)
    worst = max(worst, float(np.abs(mid.cpu().numpy() - want).max() / np.abs(want).max()))
print("WORST", worst)
"""


@pytest.mark.timeout(300)
def test_shared_memory_operand_kernel_still_matches(cuda):
    """The earlier kernel (weights as a shared-memory operand) stays selectable and correct;
    the switch is read once per process, hence the child process."""
    env = dict(os.environ, ESCHA_B200_TC_WEIGHTS="smem")
    run = subprocess.run([sys.executable, "-c", SMEM_CHILD, ROOT], env=env, capture_output=True,
                         text=True, timeout=240)
    assert run.returncode == 0, run.stderr[-2000:]
    assert float(run.stdout.split("WORST")[1]) < GEMV_TOL


PDL_OFF_CHILD = r"""
import sys
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + "/tests")
import numpy as np, torch
from escha_mlx_b200 import dense, synth
from oracle import escha_oracle as oracle
dev = torch.device("cuda", 0)
rng = np.random.default_rng(5)
K, IC, OC, M = 3, 512, 384, 100
code, rin, rout = synth.coded_projection(rng, IC, OC, K)
x = synth.activations(rng, M, IC)
lin = dense.EschaLinear(dense.EschaWeight(code, rin, rout, device=dev))
y = lin(torch.from_numpy(x).to(dev)).cpu().numpy()
ri, ro = oracle.fold_scales(rin, rout)
want = oracle.dense_linear(x, code, ri, ro, K)
print("WORST", float(np.abs(y.astype(np.float64) - want).max() / np.abs(want).max()))
"""


@pytest.mark.timeout(300)
def test_unchained_launches_give_the_same_linear(cuda):
    """ESCHA_B200_PDL=off: transforms and the prefill GEMM launched without programmatic
    dependent launch (the in-kernel waits become no-ops); ESCHA_B200_TC_CLUSTER_SUM=0: the split
    launch writes f32 planes and a second kernel sums and transforms them."""
    env = dict(os.environ, ESCHA_B200_PDL="off", ESCHA_B200_TC_CLUSTER_SUM="0")
    run = subprocess.run([sys.executable, "-c", PDL_OFF_CHILD, ROOT], env=env, capture_output=True,
                         text=True, timeout=240)
    assert run.returncode == 0, run.stderr[-2000:]
    assert float(run.stdout.split("WORST")[1]) < 2e-3


@pytest.mark.parametrize("M,ocs,splits", [(100, (384, 128, 128), None), (200, (256, 128), 1),
                                          (40, (128, 128, 256), 3), (130, (256,), 2)])
def test_prefill_projections_sharing_one_launch(cuda, oracle, M, ocs, splits):
    """Up to three projections of equal IC and K in one tcgen05 launch: every output within
    tolerance of the oracle and of its own separate launch."""
    rng = np.random.default_rng(M + len(ocs))
    K, IC = 2, 1024
    xhs, codes, routs, raw = [], [], [], []
    for oc in ocs:
        code, _, rout = synth.coded_projection(rng, IC, oc, K)
        xh = (rng.standard_normal((M, IC)) * 0.25).astype(np.float16)
        raw.append((code, xh, rout))
        xhs.append(dev(xh, cuda))
        codes.append(msl.code_tensor(code, cuda))
        routs.append(dev(rout.astype(np.float32), cuda))
    got = msl.dense_gemm_tc_many(xhs, codes, K, IC, list(ocs), routs, msl.RS, splits=splits)
    torch.cuda.synchronize()
    assert lib.escha_coded_gemm_tc_status() == 0
    again = msl.dense_gemm_tc_many(xhs, codes, K, IC, list(ocs), routs, msl.RS, splits=splits)
    for y, y2, (code, xh, rout), xd, c, ro, oc in zip(got, again, raw, xhs, codes, routs, ocs):
        assert y.shape == (M, oc) and torch.equal(y, y2)       # deterministic
        want = oracle.output_transform(oracle.gemv_f64(xh, code, None, K, IC, oc).astype(np.float32),
                                       rout.astype(np.float32))
        assert rel_err(host(y), want) < 2e-3
        alone = msl.dense_gemm_tc(xd, c, K, IC, oc, rout=ro)
        assert rel_err(host(y), host(alone)) < 2e-3
    with pytest.raises(ValueError):
        msl.dense_gemm_tc_many(xhs, codes, K, IC, list(ocs) + [128], routs)

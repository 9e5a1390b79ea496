"""GPU: the shared-memory codebook table inside the coded GEMV.

The reference gives every GEMV/GEMM kernel a ``_lut`` twin that looks decoded weights up in a
65536-entry fp16 table instead of hashing (escha_mlx/msl.py:17-22, :114-115, selection
:1070-1076).  Here ``ESCHA_MLX_LUT=1`` makes the persistent GEMV look all of a lane's states up
in a table it keeps in shared memory, ``ESCHA_B200_LUT_STATES=2`` two of eight.  A table entry
is the hash decode of its index, so every mode must produce the same bits as the hash kernels.
The switches are read once per process, hence the child processes.
"""
from __future__ import annotations

import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import hashlib, sys
sys.path.insert(0, sys.argv[1])
import numpy as np, torch
from escha_mlx_b200 import msl, synth
from escha_mlx_b200._lib import lib
dev = torch.device("cuda", 0)
h = hashlib.sha256()
for K, IC, OC, M, splits in ((2, 1280, 384, 1, 2), (3, 1024, 256, 1, 1), (3, 1536, 384, 5, 3),
                             (2, 2048, 256, 13, 4)):
    rng = np.random.default_rng(K * 1000 + IC + M)
    code, rin, rout = synth.coded_projection(rng, IC, OC, K)
    x = synth.activations(rng, M, IC)
    c = msl.code_tensor(code, dev)
    xd = torch.from_numpy(x).to(dev)
    ro = torch.from_numpy(rout.astype(np.float32)).to(dev)
    mid = msl.dense_gemv(xd, c, K, IC, OC, splits=splits)
    y = msl._gemv_mma_dense(xd, c, ro, K, IC, OC, splits)
    torch.cuda.synchronize()
    h.update(mid.cpu().numpy().tobytes()); h.update(y.cpu().numpy().tobytes())
assert lib.escha_coded_gemv_status() == 0
print("DIGEST", h.hexdigest())
"""


def _digest(env_extra: dict) -> str:
    env = dict(os.environ)
    for k in ("ESCHA_MLX_LUT", "ESCHA_B200_LUT_STATES", "ESCHA_B200_GEMV_KERNEL"):
        env.pop(k, None)
    env.update(env_extra)
    run = subprocess.run([sys.executable, "-c", CHILD, ROOT], env=env, capture_output=True,
                         text=True, timeout=300)
    assert run.returncode == 0, run.stderr[-2000:]
    return run.stdout.split("DIGEST")[1].strip()


@pytest.mark.gpu
def test_table_modes_equal_hash_bits():
    want = _digest({})                                           # hash, one CTA per block
    assert _digest({"ESCHA_B200_GEMV_KERNEL": "stream"}) == want  # hash, persistent kernel
    assert _digest({"ESCHA_MLX_LUT": "1"}) == want                # all eight states from the table
    assert _digest({"ESCHA_B200_LUT_STATES": "2"}) == want        # two from the table, six hashed

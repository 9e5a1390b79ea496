"""GPU: bounded waits that run out return a status instead of hanging.

Nothing here faults, traps or spins without a limit: a test hook makes the GEMV's producers
announce their weight copies without issuing them, so the decode warps' waits run out after a
short, host-set number of tries; the peer barrier is pointed at a "peer" whose arrival word is
a local buffer that nobody writes; the tcgen05 prefill kernel has the same hook as the GEMV.  In
every case the kernel must return, raise its status word and leave the GPU usable (the same
launch, with the hook off, then gives the right answer).
"""
from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch



def dev(a, device):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def host(t):
    return t.detach().cpu().numpy()

pytestmark = pytest.mark.gpu


def test_gemv_wait_gives_up_and_reports(cuda, oracle):
    from escha_mlx_b200 import msl, synth
    from escha_mlx_b200._lib import lib
    rng = np.random.default_rng(5)
    K, IC, OC, M = 2, 1536, 256, 3
    code, _, _ = synth.coded_projection(rng, IC, OC, K)
    xh = synth.activations(rng, M, IC)
    c, x = msl.code_tensor(code, cuda), dev(xh, cuda)
    good = msl.dense_gemv(x, c, K, IC, OC, splits=3)
    torch.cuda.synchronize()
    assert lib.escha_coded_gemv_status() == 0
    lib.escha_debug_gemv_stall(1, 64)
    try:
        msl.dense_gemv(x, c, K, IC, OC, splits=3)      # returns: every wait is bounded
        torch.cuda.synchronize()
        assert lib.escha_coded_gemv_status() != 0       # ... and says that it gave up
        assert lib.escha_coded_gemv_status() == 0       # reading clears the word
    finally:
        lib.escha_debug_gemv_stall(0, 0)
    # the device is usable and the split counters were left clean: same bits as before
    again = msl.dense_gemv(x, c, K, IC, OC, splits=3)
    torch.cuda.synchronize()
    assert lib.escha_coded_gemv_status() == 0
    assert torch.equal(again, good)
    exact = oracle.gemv_f64(xh, code, None, K, IC, OC)
    assert np.abs(host(again) - exact).max() / np.abs(exact).max() < 1e-3


def test_peer_barrier_gives_up_on_a_silent_peer(cuda):
    from escha_mlx_b200._lib import check, lib, stream
    nranks = 2
    # this rank's words: [nranks] arrivals, epoch, status; the "peer" is just more local
    # memory, so nobody ever announces an epoch to us
    mine = torch.zeros(nranks + 2, dtype=torch.int32, device=cuda)
    silent = torch.zeros(nranks + 2, dtype=torch.int32, device=cuda)
    peers = (ctypes.c_void_p * nranks)(mine.data_ptr(), silent.data_ptr())
    lib.escha_debug_peer_poll_limit(2000)               # about 0.2 ms
    try:
        check(lib.escha_peer_barrier(ctypes.c_void_p(mine.data_ptr()), peers, 0, nranks, stream()))
        torch.cuda.synchronize()
    finally:
        lib.escha_debug_peer_poll_limit(0)
    words = mine.cpu().tolist()
    assert words[nranks] == 1                           # our epoch advanced
    assert words[nranks + 1] == 1                       # the wait gave up and said so
    assert silent.cpu().tolist()[0] == 1                # our announcement reached the "peer"
    # the GPU still answers
    assert float(torch.ones(8, device=cuda).sum().item()) == 8.0


TC_CHILD = r"""
import sys
sys.path.insert(0, sys.argv[1])
import numpy as np, torch
from escha_mlx_b200 import msl, synth
from escha_mlx_b200._lib import lib
dev = torch.device("cuda", 0)
rng = np.random.default_rng(11)
K, IC, OC, M = 3, 1024, 256, 64
code, _, rout = synth.coded_projection(rng, IC, OC, K)
c = msl.code_tensor(code, dev)
xh = torch.from_numpy(synth.activations(rng, M, IC)).to(dev)
ro = torch.from_numpy(rout.astype(np.float32)).to(dev)
good_mid = msl.dense_gemm_tc(xh, c, K, IC, OC, splits=1)
good_y = msl.dense_gemm_tc(xh, c, K, IC, OC, splits=1, rout=ro)
torch.cuda.synchronize()
assert lib.escha_coded_gemm_tc_status() == 0
lib.escha_debug_gemm_tc_stall(1, 2000)      # about 2 ms of patience per wait
msl.dense_gemm_tc(xh, c, K, IC, OC, splits=1)           # f32 plane epilogue
msl.dense_gemm_tc(xh, c, K, IC, OC, splits=1, rout=ro)  # fused output transform
msl.dense_gemm_tc(xh, c, K, IC, OC, splits=2, rout=ro)  # the cluster-sum form: both CTAs give up
torch.cuda.synchronize()                                  # returns: every wait is bounded
assert lib.escha_coded_gemm_tc_status() != 0              # ... and the kernels said so
lib.escha_debug_gemm_tc_stall(0, 0)
again_mid = msl.dense_gemm_tc(xh, c, K, IC, OC, splits=1)
again_y = msl.dense_gemm_tc(xh, c, K, IC, OC, splits=1, rout=ro)
torch.cuda.synchronize()
assert torch.equal(again_mid, good_mid) and torch.equal(again_y, good_y)
print("TC STALL OK")
"""


def test_prefill_gemm_waits_give_up_and_report():
    """The tcgen05 kernel's rings (code, weights in tensor memory, activations): with the
    weight copies withheld, the decode warps, the issuing warp and the activation loader each
    run out of patience, meet at the CTA barrier, free their tensor memory and return; the
    status word reports it and the next launches give the same bits as before.  In a process
    of its own: that status word is not cleared by reading."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    run = subprocess.run([sys.executable, "-c", TC_CHILD, root], capture_output=True, text=True,
                         timeout=600)
    assert run.returncode == 0, (run.stdout + run.stderr)[-3000:]
    assert "TC STALL OK" in run.stdout

"""GPU: the GEMV entry point that brings its own scratch (escha_coded_gemv_static).

Some callers of this library cannot allocate device memory -- a plugin inside a
server that owns the whole device arena, a callback that must not re-enter the
host allocator -- so they cannot provide the split-K workspace the regular entry
point takes.  For them the library carries a static device array.  This test
calls that entry point straight through the C ABI, twice in a row (the second
call sees whatever the first left in the shared array), and checks both results
against the regular entry point given a caller workspace (equal split factors
mean equal summation order, so that comparison is exact) and against the CPU
oracle (an fp64 product of oracle-decoded weights, then the oracle's output
transform where the launch fuses it) within the path's 1e-3 bar.

Collected last on purpose: if it fails, `pytest -x` has already run everything else.
"""
from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from escha_mlx_b200 import msl, synth
from escha_mlx_b200._lib import check, lib, ptr

pytestmark = pytest.mark.gpu


def _regular(xh, code, rout, K, IC, OC, splits):
    m = xh.shape[0]
    nbytes = int(lib.escha_coded_gemv_workspace_bytes(1, OC, splits, 8 if m <= 8 else 16))
    ws = torch.zeros(max(nbytes, 16), dtype=torch.uint8, device=xh.device)
    out = torch.empty((m, OC), dtype=torch.float16 if rout is not None else torch.float32,
                      device=xh.device)
    check(lib.escha_coded_gemv(ptr(xh), ptr(code), ptr(rout), m, IC, OC, K, splits, msl.RS,
                               ptr(ws), ctypes.c_size_t(ws.numel()), ptr(out), None))
    return out


def _static(xh, code, rout, K, IC, OC, splits):
    m = xh.shape[0]
    out = torch.empty((m, OC), dtype=torch.float16 if rout is not None else torch.float32,
                      device=xh.device)
    check(lib.escha_coded_gemv_static(ptr(xh), ptr(code), ptr(rout), m, IC, OC, K, splits, msl.RS,
                                      ptr(out), None))
    return out


@pytest.mark.parametrize("K,IC,OC,M,splits,fused", [(2, 1024, 384, 1, 4, True),
                                                    (3, 1536, 256, 7, 3, False),
                                                    (2, 512, 128, 12, 2, True)])
def test_static_scratch_matches_caller_workspace_twice(cuda, oracle, K, IC, OC, M, splits, fused):
    rng = np.random.default_rng(K * 100 + M)
    code, _, rout = synth.coded_projection(rng, IC, OC, K)
    c = msl.code_tensor(code, cuda)
    ro = torch.from_numpy(rout.astype(np.float32)).to(cuda) if fused else None
    xs = [torch.from_numpy((rng.standard_normal((M, IC)) * 0.05).astype(np.float16)).to(cuda)
          for _ in range(2)]
    want = [_regular(x, c, ro, K, IC, OC, splits) for x in xs]
    got = [_static(x, c, ro, K, IC, OC, splits) for x in xs]   # two calls in a row, shared array
    torch.cuda.synchronize()
    for g, w in zip(got, want):
        assert torch.equal(g, w)
    for g, x in zip(got, xs):
        exact = oracle.gemv_f64(x.cpu().numpy(), code, None, K, IC, OC)
        if fused:   # y = f16((H128(mid) * RS) * rout): the oracle's transform of the exact product
            exact = oracle.output_transform(exact.astype(np.float32), rout.astype(np.float32)).astype(np.float64)
        err = np.abs(g.float().cpu().numpy().astype(np.float64) - exact).max() / np.abs(exact).max()
        assert err < 1e-3, err
    assert not torch.equal(got[0], got[1])   # different inputs really produced different outputs


def test_static_scratch_rejects_sizes_beyond_its_array(cuda):
    fake = ctypes.c_void_p(0x1000)   # validation fails before anything is dereferenced
    with pytest.raises(ValueError, match=r"M must be in \[1, 16\]"):
        check(lib.escha_coded_gemv_static(fake, fake, None, 17, 1024, 1024, 2, 2, msl.RS, fake, None))
    with pytest.raises(ValueError, match="static array holds"):
        # 64 splits x 1024 output blocks x 8 rows x 512 B = 256 MiB of partials
        check(lib.escha_coded_gemv_static(fake, fake, None, 1, 8192, 131072, 2, 64, msl.RS, fake, None))

"""ctypes binding of ``libescha_b200.so`` (the C ABI in ``include/escha_b200.h``).

There is no fallback: if the shared library is missing or a symbol cannot be
resolved, importing this module raises.  Contract violations reported by the
library (``ESCHA_EINVAL``) surface as ``ValueError`` -- the exception type the
reference raises for the same mistakes (escha_mlx/dense.py:172-242) -- and CUDA
failures as ``RuntimeError``.
"""
from __future__ import annotations

import ctypes
import os

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
# ESCHA_B200_LIBRARY points at another build of the same library (kernel experiments)
LIB_PATH = os.environ.get("ESCHA_B200_LIBRARY") or os.path.join(_PKG, "libescha_b200.so")

ESCHA_OK, ESCHA_EINVAL, ESCHA_ECUDA = 0, -1, -2

_vp, _i, _f, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t

# name -> (restype, argtypes); must list every symbol the header declares
SIGNATURES = {
    "escha_version": (_i, []),
    "escha_last_error": (ctypes.c_char_p, []),
    "escha_lut_init": (_i, [_vp, _vp]),
    "escha_decode_tiles": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp]),
    "escha_scaled_had": (_i, [_vp, _vp, _vp, _i, _i, _f, _vp, _vp]),
    "escha_scaled_had_out": (_i, [_vp, _vp, _vp, _i, _i, _f, _vp, _vp]),
    "escha_scaled_had_pair": (_i, [_vp, _vp, _vp, _i, _i, _f, _vp, _vp, _vp]),
    "escha_coded_gemm_tc_many": (_i, [_i, _vp, _vp, _vp, _i, _i, _vp, _i, _i, _f, _vp, _vp, _vp]),
    "escha_scaled_had_many": (_i, [_vp, _vp, _i, _vp, _vp, _i, _i, _f, _vp]),
    "escha_scaled_had_out_pair": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp, _vp, _vp]),
    "escha_had128": (_i, [_vp, ctypes.c_long, _vp, _vp]),
    "escha_w8a16": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp]),
    "escha_w8a16_many": (_i, [_vp, _i, _vp, _vp, _vp, _i, _i, _vp, _vp]),
    "escha_q8_embed": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp]),
    "escha_gemv_ref": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp]),
    "escha_coded_gemv_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "escha_coded_gemv_splits": (_i, [_i, _i, _i, _i]),
    "escha_coded_gemv": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _vp, _sz, _vp, _vp]),
    "escha_coded_gemv_static": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _vp, _vp]),
    "escha_coded_projections": (_i, [_vp, _vp, _vp, ctypes.c_long, _i, _i, _i, _vp, _vp, _vp, _vp, _vp,
                                     _vp, _i, _i, _i, _i, _i, _i, _vp, _f, _vp, _sz, _vp]),
    "escha_coded_projections_gather": (_i, [_vp, _vp, _vp, ctypes.c_long, _i, _i, _i, _vp, _vp, _vp,
                                           _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _f, _vp,
                                           _sz, _vp, _i, _vp, _vp, _vp]),
    "escha_coded_projections_mixed": (_i, [_vp, _vp, _vp, ctypes.c_long, _i, _i, _i, _vp, _vp, _vp,
                                          _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _f, _vp,
                                          _sz, _vp, _i, _vp, _vp, _vp]),
    "escha_peer_barrier": (_i, [_vp, _vp, _i, _i, _vp]),
    "escha_moe_jobs_bound": (_i, [_i, _i, _i]),
    "escha_moe_group_rows": (_i, [_vp, _i, _i, _i, _vp, _i, _vp, _vp]),
    "escha_jobs_from_groups": (_i, [_vp, _vp, _i, _i, _i, _i, _vp, _vp]),
    "escha_coded_gemv_jobs": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp,
                                   _sz, _vp, _vp]),
    "escha_swiglu": (_i, [_vp, _vp, _i, _i, ctypes.c_long, _vp, _vp]),
    "escha_moe_combine": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp]),
    "escha_coded_gemm_tc": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp]),
    "escha_coded_gemm_tc_splits": (_i, [_i, _i, _i]),
    "escha_coded_gemm_tc_needs_planes": (_i, [_i, _i, _i]),
    "escha_coded_gemm_tc_status": (_i, []),
    "escha_coded_gemv_status": (_i, []),
    "escha_debug_gemv_stall": (None, [_i, ctypes.c_uint]),
    "escha_debug_peer_poll_limit": (None, [ctypes.c_uint]),
    "escha_debug_gemm_tc_stall": (None, [_i, ctypes.c_uint]),
    "escha_moe_route": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp,
                            _vp, _i, _vp, _sz, _vp]),
    "escha_moe_shared_finish": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _i, _vp, _vp]),
}


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m escha_mlx_b200.csrc.build` "
            "(needs nvcc). This package has no CPU or eager fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = stale library: rebuild
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()


def check(rc: int) -> None:
    if rc == ESCHA_OK:
        return
    msg = (lib.escha_last_error() or b"").decode()
    if rc == ESCHA_EINVAL:
        raise ValueError(msg)
    raise RuntimeError(msg)


def ptr(t: torch.Tensor | None, dtype: torch.dtype | None = None) -> ctypes.c_void_p | None:
    """Device pointer of a contiguous CUDA tensor (None passes through as NULL)."""
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("escha kernels take CUDA tensors; got a CPU tensor "
                         "(there is no CPU path in this package)")
    if not t.is_contiguous():
        raise ValueError("escha kernels take contiguous tensors")
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"expected a {dtype} tensor, got {t.dtype}")
    return ctypes.c_void_p(t.data_ptr())


def stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class _Workspaces:
    """Zero-initialised scratch for the split-K kernels, one buffer per
    (device, stream).  Kernels leave the counter region zero on exit, so a buffer
    is reused by every launch on its stream without clearing; two launches that
    may overlap on the GPU must not share one (hence the per-stream key)."""

    def __init__(self) -> None:
        self._bufs: dict[tuple[int, int], torch.Tensor] = {}

    def get(self, nbytes: int, device: torch.device) -> torch.Tensor:
        key = (device.index if device.index is not None else torch.cuda.current_device(),
               torch.cuda.current_stream().cuda_stream)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < nbytes:
            buf = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
            self._bufs[key] = buf
        return buf


workspaces = _Workspaces()

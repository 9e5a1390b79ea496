"""Kernel layer of the coded-projection path on B200.

Mirrors the function surface of the reference's ``escha_mlx/msl.py`` (the
module whose functions each launch one Metal kernel) with the same names,
argument order and error behaviour, taking contiguous CUDA ``torch.Tensor``s in
place of ``mx.array``s and calling hand-written sm_100a kernels through the C
ABI in ``include/escha_b200.h``.  Wrappers are pure: inputs are borrowed, a
freshly allocated output is returned, nothing synchronises.

Two GEMV kernel families exist (``ESCHA_MLX_GEMV``):

* ``mma`` (default) -- the tensor-core kernel: decoded tile fragments feed
  ``mma.sync`` directly, 8 or 16 rows share one decode, split-K over 128-channel
  input blocks with a fixed-order reduction, optional fused output transform.
  Deterministic: bit-reproducible run to run, and a row's result does not
  depend on which other rows are in the batch.
* ``reforder`` -- a scalar kernel in the reference kernels' exact accumulation
  order (bit-identical to them and to the CPU oracle).

Reference citations are to ``escha_mlx/msl.py`` unless stated otherwise.
"""
from __future__ import annotations

import ctypes
import os
from functools import lru_cache

import numpy as np
import torch

from . import envs
from ._lib import check, lib, ptr, stream, workspaces

RS = 0.088388347648  # escha_mlx/ref.py:30

#: Rows that share one decode in the tensor-core kernel (one or two mma column blocks).
MMA_ROWS = (8, 16)

#: Largest rows-per-group the reference's dense row-blocked GEMM chooses (:1548);
#: kept for API compatibility -- here 16 rows always share a decode.
DENSE_R_MAX = 16
DENSE_MAT_R = 16


# ---------------------------------------------------------------------------
# knobs (reference: :1024-1026, :1070, :1140-1242, :1551-1601, :1729-1759)
# ---------------------------------------------------------------------------

def use_fused_had() -> bool:
    return bool(envs.ESCHA_MLX_FUSED_HAD.get())


def use_lut() -> bool:
    return bool(envs.ESCHA_MLX_LUT.get())


def gemv_family() -> str:
    return envs.ESCHA_MLX_GEMV.get()


def use_dense_mat() -> bool:
    """The reference gates its reassociated matrix-unit GEMM behind a flag
    (:1729-1759); here the tensor-core kernel IS the default family."""
    return gemv_family() == "mma"


def wave_splits(IC: int, OCs, njobs: int = 1) -> list[int]:
    """Split factors for projections that share ONE launch, chosen for the launch as a whole:
    the launch's CTAs (output blocks x splits, summed over the projections) should fill the
    GPU's resident slots once, where ``split_k_for`` fills them once per projection.  The sums
    of a projection then differ in their last bits from those of a launch of its own (each
    composition is still bit-reproducible); measured on the 27B-class layer at one row, q/k/v/o
    in one launch take 1192 CTAs of 2 to 4 input blocks with per-projection factors and 416
    CTAs of 10 blocks this way, 119 against 126 us per layer step.  A launch too wide for one
    wave gets the fewest waves it can fill (with a single, underfilled wave for gate/up the
    step took 144 us)."""
    blocks = sum(oc // 128 for oc in OCs) * max(1, njobs)
    smax = max(1, (IC // 128) // 2)
    slots = 3 * sm_count()
    # the fewest waves whose slots the launch can fill to 85%: one wave for q/k/v/o of the
    # 27B-class layer (104 blocks x 4 = 416 of 444 slots), two for gate/up (272 x 3 = 816 of 888)
    s = smax
    for waves in range(1, 9):
        cand = min(smax, (waves * slots) // max(1, blocks))
        if cand >= 1 and blocks * cand >= 0.85 * waves * slots:
            s = cand
            break
        if cand == smax:
            break
    return [s] * len(OCs)


def kt_block() -> int:
    """kt tiles per pipeline stage of the tensor-core kernel (fixed at 8 = one
    128-channel block; the reference stages a configurable count, :1229-1242)."""
    return 8


def dense_block_r_pin() -> int | None:
    return envs.ESCHA_MLX_DENSE_BLOCK_R.get()


def dense_block_r(m: int, pin: int | None = None) -> int:
    """Rows per decode the reference's policy would pick (:1562-1601): min(m, 16)
    snapped down to a power of two.  Informational here -- the tensor-core kernel
    shares every decode across up to 16 rows regardless."""
    if pin is not None:
        return pin
    r = min(m, DENSE_R_MAX)
    while r & (r - 1):
        r &= r - 1
    return max(1, r)


def split_k_for(m: int, oc: int, tk: int, njobs: int = 1) -> int:
    """Split factor for an [m, tk*16] x [tk*16, oc] coded product (:1191-1226).

    ``ESCHA_MLX_SPLITK``: an integer pins it, ``auto`` (default) fills the GPU:
    as many splits as fit the three resident CTAs per SM without exceeding them,
    at least two 128-channel blocks per split.  Depends on the shape only -- never on the data and, for a dense
    stream, not on m -- so results are reproducible and batch-invariant.
    """
    setting = envs.ESCHA_MLX_SPLITK.get()
    nblk = tk // 8
    if setting != "auto":
        s = int(setting)
        return s if 1 < s <= nblk else 1
    return int(lib.escha_coded_gemv_splits(tk * 16, oc, njobs, 0))


# ---------------------------------------------------------------------------
# helpers
# ---------------------------------------------------------------------------

def code_to_u32(code_i16: np.ndarray) -> np.ndarray:
    """View an int16 code tensor [..., 16K] as little-endian uint32 [..., 8K] (:1398-1401)."""
    a = np.ascontiguousarray(code_i16).view(np.uint16)
    return a.view(np.uint32)


def code_tensor(code_i16: np.ndarray, device=None) -> torch.Tensor:
    """Host int16 export -> device code stream (stored as int32 words; torch has
    no arithmetic on uint32 and the kernels only read the bits)."""
    words = code_to_u32(code_i16).view(np.int32)
    return torch.from_numpy(words).to(device or "cuda")


_LUTS: dict[int, torch.Tensor] = {}


def _lut_tensor(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _LUTS.get(idx)
    if t is None:
        t = torch.empty(65536, dtype=torch.float16, device=device)
        check(lib.escha_lut_init(ptr(t), stream()))
        _LUTS[idx] = t
    return t


def _maybe_lut(device) -> torch.Tensor | None:
    return _lut_tensor(device) if use_lut() else None


def _check_code(code: torch.Tensor) -> None:
    if code.dtype not in (torch.int32, torch.uint32):
        raise ValueError(f"code stream must be 32-bit words, got {code.dtype}")


def _i32(t: torch.Tensor | None) -> torch.Tensor | None:
    if t is None:
        return None
    if t.dtype != torch.int32:
        raise ValueError(f"index tensors must be int32, got {t.dtype}")
    return t


# ---------------------------------------------------------------------------
# decode
# ---------------------------------------------------------------------------

def decode_tiles(code_u32: torch.Tensor, K: int, IC: int, OC: int) -> torch.Tensor:
    """Decode one projection's packed stream -> fp16 bare weight [IC, OC] (:1404-1421)."""
    _check_code(code_u32)
    w = torch.empty((IC, OC), dtype=torch.float16, device=code_u32.device)
    check(lib.escha_decode_tiles(ptr(code_u32), K, IC, OC, ptr(_maybe_lut(code_u32.device)),
                                 ptr(w), stream()))
    return w


# ---------------------------------------------------------------------------
# scaled Hadamard transforms
# ---------------------------------------------------------------------------

def scaled_had(rows: torch.Tensor, rin: torch.Tensor, row_expert: torch.Tensor | None,
               rs: float) -> torch.Tensor:
    """rows [m, IC] f16, rin [E, IC] f32 (or [IC] with row_expert=None) -> [m, IC] f16 (:1029-1047)."""
    m, ic = rows.shape
    out = torch.empty((m, ic), dtype=torch.float16, device=rows.device)
    check(lib.escha_scaled_had(ptr(rows, torch.float16), ptr(rin, torch.float32),
                               ptr(_i32(row_expert)), m, ic, float(rs), ptr(out), stream()))
    return out


def scaled_had_out(mid: torch.Tensor, rout: torch.Tensor, row_expert: torch.Tensor | None,
                   rs: float) -> torch.Tensor:
    """mid [m, OC] f32, rout [E, OC] f32 -> transformed [m, OC] f16 (:1050-1067)."""
    m, oc = mid.shape
    out = torch.empty((m, oc), dtype=torch.float16, device=mid.device)
    check(lib.escha_scaled_had_out(ptr(mid, torch.float32), ptr(rout, torch.float32),
                                   ptr(_i32(row_expert)), m, oc, float(rs), ptr(out), stream()))
    return out


def dense_scaled_had(rows: torch.Tensor, rin: torch.Tensor, rs: float) -> torch.Tensor:
    return scaled_had(rows, rin, None, rs)


def dense_scaled_had_out(mid: torch.Tensor, rout: torch.Tensor, rs: float) -> torch.Tensor:
    return scaled_had_out(mid, rout, None, rs)


def dense_scaled_had_pair(rows: torch.Tensor, rin0: torch.Tensor, rin1: torch.Tensor, rs: float):
    """Two dense input transforms in one launch (:1491-1504)."""
    m, ic = rows.shape
    out0 = torch.empty((m, ic), dtype=torch.float16, device=rows.device)
    out1 = torch.empty_like(out0)
    check(lib.escha_scaled_had_pair(ptr(rows, torch.float16), ptr(rin0, torch.float32),
                                    ptr(rin1, torch.float32), m, ic, float(rs), ptr(out0),
                                    ptr(out1), stream()))
    return out0, out1


def dense_scaled_had_many(rows: torch.Tensor, rins, rs: float, up: torch.Tensor | None = None):
    """One to four dense input transforms of the same rows in one launch (the pair dispatch of
    :1491-1504 widened to Q/K/V); with ``up`` the rows are a SwiGLU gate and the input is
    ``f16(f16(silu(rows)) * up)`` (the SwiGLU-into-down-input fusion of
    models/qwen3_5.py:63-198).  Bit-identical to the separate launches."""
    m, ic = rows.shape
    rins = list(rins)
    if not 1 <= len(rins) <= 4:
        raise ValueError(f"one to four transforms per launch, got {len(rins)}")
    if up is not None and up.shape != rows.shape:
        raise ValueError("SwiGLU input needs gate and up of equal shape")
    outs = [torch.empty((m, ic), dtype=torch.float16, device=rows.device) for _ in rins]
    rin_ptrs = (ctypes.c_void_p * len(rins))(*[r.data_ptr() for r in rins])
    out_ptrs = (ctypes.c_void_p * len(rins))(*[o.data_ptr() for o in outs])
    for r in rins:
        if r.dtype != torch.float32 or r.numel() != ic or not r.is_contiguous():
            raise ValueError("scale vectors must be contiguous f32 [IC]")
    check(lib.escha_scaled_had_many(ptr(rows, torch.float16),
                                    ptr(up, torch.float16) if up is not None else None,
                                    len(rins), rin_ptrs, out_ptrs, m, ic, float(rs), stream()))
    return outs


def dense_scaled_had_out_pair(mid0: torch.Tensor, mid1: torch.Tensor, rout0: torch.Tensor,
                              rout1: torch.Tensor, rs: float):
    """Two dense output transforms in one launch (:1507-1527)."""
    m, oc0 = mid0.shape
    if mid1.shape[0] != m:
        raise ValueError("output transform pair requires equal row counts")
    oc1 = mid1.shape[1]
    out0 = torch.empty((m, oc0), dtype=torch.float16, device=mid0.device)
    out1 = torch.empty((m, oc1), dtype=torch.float16, device=mid0.device)
    check(lib.escha_scaled_had_out_pair(ptr(mid0, torch.float32), ptr(mid1, torch.float32),
                                        ptr(rout0, torch.float32), ptr(rout1, torch.float32), m,
                                        oc0, oc1, float(rs), ptr(out0), ptr(out1), stream()))
    return out0, out1


# ---------------------------------------------------------------------------
# row jobs (device-side grouping for E-stacked streams)
# ---------------------------------------------------------------------------

JOB_INTS = 18


def jobs_bound(m: int, E: int, R: int = 8) -> int:
    return int(lib.escha_moe_jobs_bound(m, E, R))


def group_rows(row_expert: torch.Tensor, E: int, R: int = 8) -> torch.Tensor:
    """row_expert [m] i32 -> row jobs [jobs_bound(m, E, R), 18] i32, device-resident
    (replaces moe.build_groups for the tensor-core kernel; no host sync)."""
    m = row_expert.shape[0]
    cap = jobs_bound(m, E, R)
    jobs = torch.empty((cap, JOB_INTS), dtype=torch.int32, device=row_expert.device)
    check(lib.escha_moe_group_rows(ptr(_i32(row_expert)), m, E, R, ptr(jobs), cap, None, stream()))
    return jobs


def expected_jobs(m: int, E: int) -> int:
    """Expected number of distinct experts hit by m uniformly routed rows; the
    data-independent job count the split policy is evaluated at."""
    return max(1, int(round(E * (1.0 - (1.0 - 1.0 / E) ** m))))


# ---------------------------------------------------------------------------
# coded GEMV / small-batch GEMM
# ---------------------------------------------------------------------------

def _gemv_reforder(xh, code, row_expert, K, IC, OC, splits, row_map=None, n_out=None):
    m = xh.shape[0] if n_out is None else n_out
    s = splits if splits and splits > 1 and (IC // 16) % splits == 0 else 1
    mid = torch.zeros((m, OC), dtype=torch.float32, device=xh.device) if row_map is not None \
        else torch.empty((m, OC), dtype=torch.float32, device=xh.device)
    part = torch.empty((s, m, OC), dtype=torch.float32, device=xh.device) if s > 1 else None
    slots = 0 if row_map is None else row_map.shape[0]
    check(lib.escha_gemv_ref(ptr(xh, torch.float16), ptr(code), ptr(_i32(row_expert)),
                             ptr(_i32(row_map)), slots, ptr(_maybe_lut(xh.device)), m, IC, OC, K,
                             s, ptr(part), ptr(mid), stream()))
    return mid


def _gemv_mma_dense(xh, code, rout, K, IC, OC, splits, rs=RS):
    m = xh.shape[0]
    s = split_k_for(m, OC, IC // 16) if splits is None else max(1, min(int(splits), IC // 128))
    rows_per_job = 8 if m <= 8 else 16
    njobs = (m + rows_per_job - 1) // rows_per_job
    out = torch.empty((m, OC), dtype=torch.float32 if rout is None else torch.float16,
                      device=xh.device)
    # always a workspace: besides the split-K scratch it holds the counter the persistent
    # kernel hands its work items out through
    nbytes = int(lib.escha_coded_gemv_workspace_bytes(njobs, OC, s, rows_per_job))
    ws = workspaces.get(nbytes, xh.device)
    nbytes = ws.numel()
    check(lib.escha_coded_gemv(ptr(xh, torch.float16), ptr(code),
                               ptr(rout, torch.float32) if rout is not None else None, m, IC, OC,
                               K, s, float(rs), ptr(ws), ctypes.c_size_t(nbytes), ptr(out),
                               stream()))
    return out


INPUT_TRANSFORMED, INPUT_RAW, INPUT_SWIGLU = 0, 1, 2

#: Projections one launch of the tensor-core kernel can hold.
MAX_PROJECTIONS = 8


def mixed_rates_supported() -> bool:
    """Whether projections of different rates should share a launch: they can (the
    persistent kernel takes any mix), but by default a mixed group is split by rate and
    each part runs on the one-CTA-per-block kernel, which measures faster per launch;
    ``ESCHA_B200_GEMV_KERNEL=stream`` keeps the group together."""
    return os.environ.get("ESCHA_B200_GEMV_KERNEL") == "stream"


#: Up to this many rows the dense modules fuse the input transform into the GEMV
#: launch (every output block's CTA redoes it for its slice of the input, which is
#: noise at decode batch sizes and a real cost beyond them: measured on the 27B-class
#: layer, fusing at 8 rows is 10% slower than separate transform launches, at 16 rows 20%).
FUSE_INPUT_MAX_ROWS = 4


def coded_projections(x: torch.Tensor, codes, rins, routs, K: int, IC: int, OCs,
                      input_mode: int = INPUT_TRANSFORMED, x_up: torch.Tensor | None = None,
                      jobs: torch.Tensor | None = None, E: int = 1, splits: int | None = None,
                      rs: float = RS, rows_per_job: int = 8, outs=None,
                      policy_rows: int | None = None, xs=None, rows: int | None = None,
                      x_stride: int | None = None, x_row_div: int = 1, gather=None):
    """One launch of the tensor-core kernel for 1..8 projections of the same rows.

    ``K`` is the rate of all of them, or a sequence with one rate per projection.
    ``codes``/``rins``/``routs``/``OCs`` are equal-length sequences (rins may be
    None for ``INPUT_TRANSFORMED``; a rout of None yields that projection's f32
    mid instead of its f16 output).  ``input_mode`` selects what ``x`` is: the
    transformed rows, the raw activation (input transform fused), or the gate
    half of a SwiGLU whose up half is ``x_up``.  Returns the list of outputs.
    Bit-identical to running the stages as separate launches.

    ``rows`` (default: the rows of ``x``) is the number of output rows; output row
    r reads input row ``r // x_row_div`` at ``x_stride`` elements per row, which
    lets the first expert leg read token rows directly and the second read the
    gate/up halves of one merged tensor.

    ``gather``: a sequence with one ``(peer_tensor, col0)`` per projection,
    ``peer_tensor`` a ``peer.PeerTensor`` of shape [rows, row_width].  The kernel stores
    this rank's columns at ``col0`` of the local copy and of every other GPU's copy
    (split-N tensor parallelism: row_width = OC_total; expert parallelism with row
    jobs: row_width = OC, col0 = 0, rows disjoint across ranks); the caller runs
    ``PeerGroup.barrier()`` before reading.  Returns the local gathered tensors.
    """
    n = len(codes)
    m = x.shape[0] if rows is None else rows
    if rins is None:
        rins = [None] * n
    Ks = [int(k) for k in K] if isinstance(K, (list, tuple)) else [int(K)] * n
    if len(Ks) != n:
        raise ValueError(f"{len(Ks)} rates for {n} projections")
    mixed = len(set(Ks)) > 1
    K = Ks[0]
    dense = jobs is None
    pr = m if policy_rows is None else policy_rows
    total_oc = sum(OCs)
    # every projection keeps the split factor it has when launched alone, so a
    # joint launch changes no output bit
    if splits is None:
        est = 1 if dense else expected_jobs(pr, E)
        per = [split_k_for(pr, oc, IC // 16, est) for oc in OCs]
    elif isinstance(splits, (list, tuple)):
        per = [max(1, min(int(v), IC // 128)) for v in splits]
        if len(per) != n:
            raise ValueError(f"{len(per)} split factors for {n} projections")
    else:
        per = [max(1, min(int(splits), IC // 128))] * n
    s = max(per)
    if dense:
        rows_per_job = 8 if m <= 8 else 16
        njobs = (m + rows_per_job - 1) // rows_per_job
    else:
        njobs = jobs.shape[0]
    if outs is None and gather is None:
        outs = [torch.empty((m, oc), dtype=torch.float32 if ro is None else torch.float16,
                            device=x.device) for oc, ro in zip(OCs, routs)]
    nbytes = int(lib.escha_coded_gemv_workspace_bytes(njobs, total_oc, s, rows_per_job))
    ws = workspaces.get(nbytes, x.device)
    nbytes = ws.numel()
    vp = ctypes.c_void_p * n

    def table(ts, dtype=None):
        return vp(*[None if t is None else ptr(t, dtype).value for t in ts])

    for c in codes:
        _check_code(c)
    if x.dtype != torch.float16 or not x.is_cuda:
        raise ValueError("coded_projections takes a CUDA float16 activation tensor")
    # x / x_up may be column slices of one row-major tensor (merged gate/up)
    x_ptr = ctypes.c_void_p(x.data_ptr())
    up_ptr = None if x_up is None else ctypes.c_void_p(x_up.data_ptr())
    if x_stride is None:
        x_stride = IC if x.shape[0] == 1 else x.stride(0)
    if x.stride(-1) != 1 or (x_up is not None and x_up.stride(-1) != 1):
        raise ValueError("activation rows must be contiguous along the channel axis")
    if mixed:
        locs, npeers, flat = None, 0, []
        if gather is not None:
            locs = [g[0].local for g in gather]
            npeers = len(gather[0][0].peer_ptrs())
            flat = [p for g in gather for p in g[0].peer_ptrs()]
        dst = outs if gather is None else locs
        check(lib.escha_coded_projections_mixed(
            x_ptr, None if xs is None else table(xs, torch.float16), up_ptr,
            x_stride, x_row_div, input_mode, n, table(codes), table(rins, torch.float32),
            table(routs, torch.float32), table(dst), (ctypes.c_int * n)(*OCs),
            (ctypes.c_int * n)(*Ks),
            None if dense else ptr(jobs, torch.int32), njobs, rows_per_job, m, E, IC,
            (ctypes.c_int * n)(*per), float(rs), ptr(ws), ctypes.c_size_t(nbytes),
            (ctypes.c_void_p * len(flat))(*flat) if flat else None, npeers,
            None if gather is None else (ctypes.c_int * n)(*[t.shape[-1] for t in locs]),
            None if gather is None else (ctypes.c_int * n)(*[int(g[1]) for g in gather]),
            stream()))
        return dst
    if gather is not None:
        locs = [g[0].local for g in gather]
        npeers = len(gather[0][0].peer_ptrs())
        flat = [p for g in gather for p in g[0].peer_ptrs()]
        check(lib.escha_coded_projections_gather(
            x_ptr, None if xs is None else table(xs, torch.float16), up_ptr,
            x_stride, x_row_div, input_mode, n, table(codes), table(rins, torch.float32),
            table(routs, torch.float32), table(locs), (ctypes.c_int * n)(*OCs),
            None if dense else ptr(jobs, torch.int32), njobs, rows_per_job, m, E, IC, K,
            (ctypes.c_int * n)(*per), float(rs), ptr(ws), ctypes.c_size_t(nbytes),
            (ctypes.c_void_p * len(flat))(*flat), npeers,
            (ctypes.c_int * n)(*[t.shape[-1] for t in locs]),
            (ctypes.c_int * n)(*[int(g[1]) for g in gather]), stream()))
        return locs
    check(lib.escha_coded_projections(
        x_ptr, None if xs is None else table(xs, torch.float16), up_ptr,
        x_stride, x_row_div, input_mode, n, table(codes), table(rins, torch.float32),
        table(routs, torch.float32), table(outs), (ctypes.c_int * n)(*OCs),
        None if dense else ptr(jobs, torch.int32), njobs, rows_per_job, m, E, IC, K,
        (ctypes.c_int * n)(*per), float(rs), ptr(ws), ctypes.c_size_t(nbytes), stream()))
    return outs


def coded_gemv_jobs(xh: torch.Tensor, code_u32: torch.Tensor, jobs: torch.Tensor,
                    rout: torch.Tensor | None, K: int, IC: int, OC: int, E: int,
                    splits: int | None = None, rs: float = RS, rows_per_job: int = 8,
                    out: torch.Tensor | None = None, policy_rows: int | None = None) -> torch.Tensor:
    """Tensor-core expert GEMV over row jobs (see ``group_rows``).  Returns f32
    mid [m, OC], or f16 y [m, OC] with the output transform fused when ``rout``
    ([E, OC] f32) is given.  ``policy_rows`` is the row count the split policy is
    evaluated at (default: the rows of ``xh``)."""
    m = xh.shape[0]
    njobs = jobs.shape[0]
    pr = m if policy_rows is None else policy_rows
    s = split_k_for(pr, OC, IC // 16, expected_jobs(pr, E)) if splits is None \
        else max(1, min(int(splits), IC // 128))
    if out is None:
        out = torch.empty((m, OC), dtype=torch.float32 if rout is None else torch.float16,
                          device=xh.device)
    # always a workspace: besides the split-K scratch it holds the counter the persistent
    # kernel hands its work items out through
    nbytes = int(lib.escha_coded_gemv_workspace_bytes(njobs, OC, s, rows_per_job))
    ws = workspaces.get(nbytes, xh.device)
    nbytes = ws.numel()
    check(lib.escha_coded_gemv_jobs(ptr(xh, torch.float16), ptr(code_u32),
                                    ptr(rout, torch.float32) if rout is not None else None,
                                    ptr(jobs, torch.int32), njobs, rows_per_job, m, E, IC, OC, K, s,
                                    float(rs), ptr(ws), ctypes.c_size_t(nbytes), ptr(out), stream()))
    return out


def moe_gemv(xh: torch.Tensor, code_u32: torch.Tensor, row_expert: torch.Tensor | None,
             K: int, IC: int, OC: int, splits: int | None = None,
             jobs: torch.Tensor | None = None) -> torch.Tensor:
    """Fused expert GEMV: mid[r, :] = xh[r, :] @ decode(code[row_expert[r]]) (:1424-1478).

    xh [M, IC] f16; code_u32 [E, TK, TN, 8K] (E-stacked) or [TK, TN, 8K] with
    ``row_expert=None`` for a dense linear; returns mid [M, OC] f32.
    ``splits``: None = the size policy, 1 = no split.  ``jobs`` lets a caller
    that runs several projections over the same rows group them once.
    """
    _check_code(code_u32)
    if xh.shape[0] < 1:
        raise ValueError("moe_gemv needs at least one row")
    if gemv_family() == "reforder":
        return _gemv_reforder(xh, code_u32, row_expert, K, IC, OC, splits)
    if row_expert is None:
        return _gemv_mma_dense(xh, code_u32, None, K, IC, OC, splits)
    E = code_u32.shape[0]
    if jobs is None:
        jobs = group_rows(row_expert, E)
    return coded_gemv_jobs(xh, code_u32, jobs, None, K, IC, OC, E, splits)


def dense_gemv(xh: torch.Tensor, code_u32: torch.Tensor, K: int, IC: int, OC: int,
               splits: int | None = None) -> torch.Tensor:
    """Fused dense GEMV: mid = xh @ decode(code), code_u32 [TK, TN, 8K] (:1530-1538)."""
    return moe_gemv(xh, code_u32, None, K, IC, OC, splits)


def dense_gemm_rows(xh: torch.Tensor, code_u32: torch.Tensor, K: int, IC: int, OC: int,
                    R: int) -> torch.Tensor:
    """Row-blocked dense GEMM: mid = xh @ decode(code) (:1785-1812).  Bit-identical
    to ``dense_gemv`` on the same rows, as in the reference (same kernel, same
    per-row summation order; R only reports the reference's blocking)."""
    if xh.shape[0] < 1:
        raise ValueError("dense_gemm_rows needs at least one row")
    return dense_gemv(xh, code_u32, K, IC, OC)


def dense_gemm_rows_direct(xh: torch.Tensor, code_u32: torch.Tensor, K: int, IC: int, OC: int,
                           R: int) -> torch.Tensor:
    """Small-row dense GEMM (:1815-1841); same kernel as ``dense_gemm_rows``."""
    if xh.shape[0] < 1:
        raise ValueError("dense_gemm_rows_direct needs at least one row")
    return dense_gemv(xh, code_u32, K, IC, OC)


#: From this many rows on the dense modules run the product on tcgen05 (decode once per 256
#: rows into tensor memory) instead of the register-fragment kernel, which decodes once per 16
#: rows.  Measured on the 27B-class layer (us per layer step, tcgen05 vs register-fragment):
#: 9 rows 202 vs 170, 12 rows 203 vs 176, 16 rows 172 vs 186, 24 rows 175 vs 306, 32 rows 178 vs
#: 323, 48 rows 193 vs 457.
PREFILL_MIN_ROWS = int(os.environ.get("ESCHA_B200_PREFILL_MIN_ROWS", "16"))


def use_prefill_kernel(m: int) -> bool:
    return gemv_family() == "mma" and m >= PREFILL_MIN_ROWS


def dense_gemm_mat(xh: torch.Tensor, code_u32: torch.Tensor, K: int, IC: int,
                   OC: int) -> torch.Tensor:
    """Matrix-unit dense GEMM (:1762-1782): the tcgen05 kernel at prefill row counts,
    the register-fragment tensor-core kernel below them."""
    _check_code(code_u32)
    # up to one 16-row block (the reference's DENSE_MAT_R) the register-fragment kernel, whose
    # rows are bit-identical to the per-row GEMV
    if xh.shape[0] > DENSE_MAT_R and use_prefill_kernel(xh.shape[0]):
        return dense_gemm_tc(xh, code_u32, K, IC, OC)
    return _gemv_mma_dense(xh, code_u32, None, K, IC, OC, None)


def dense_gemm_rows_direct_out(xh: torch.Tensor, code: torch.Tensor, rout: torch.Tensor, K: int,
                               IC: int, OC: int, R: int, rs: float) -> torch.Tensor:
    """Small-row GEMM with its output transform fused (:1844-1870) -> f16 [M, OC]."""
    _check_code(code)
    if xh.shape[0] < 1:
        raise ValueError("dense_gemm_rows_direct_out needs at least one row")
    if gemv_family() == "reforder":
        return scaled_had_out(_gemv_reforder(xh, code, None, K, IC, OC, None), rout, None, rs)
    return _gemv_mma_dense(xh, code, rout, K, IC, OC, None, rs)


def dense_gemm_pair(xh0, xh1, code0, code1, K0: int, K1: int, IC: int, OC0: int, OC1: int,
                    R: int):
    """Two coded projections with the same input geometry (:1909-1950)."""
    if xh0.shape != xh1.shape or xh0.shape[0] < 1:
        raise ValueError("dense_gemm_pair requires matching non-empty input rows")
    if K0 == K1 and gemv_family() == "mma":   # one launch; a mixed-rate pair takes two
        return tuple(coded_projections(xh0, [code0, code1], None, [None, None], K0, IC,
                                       [OC0, OC1], xs=[xh0, xh1]))
    return (dense_gemv(xh0, code0, K0, IC, OC0), dense_gemv(xh1, code1, K1, IC, OC1))


def dense_gemm_pair_out(xh0, xh1, code0, code1, rout0, rout1, K0: int, K1: int, IC: int,
                        OC0: int, OC1: int, R: int, rs: float):
    """Mixed-K projection pair with both output transforms fused (:1873-1906)."""
    if xh0.shape != xh1.shape or xh0.shape[0] < 1:
        raise ValueError("dense_gemm_pair_out requires matching non-empty input rows")
    if K0 == K1 and gemv_family() == "mma":
        return tuple(coded_projections(xh0, [code0, code1], None, [rout0, rout1], K0, IC,
                                       [OC0, OC1], rs=rs, xs=[xh0, xh1]))
    return (dense_gemm_rows_direct_out(xh0, code0, rout0, K0, IC, OC0, R, rs),
            dense_gemm_rows_direct_out(xh1, code1, rout1, K1, IC, OC1, R, rs))


def moe_gemm_rows(xh: torch.Tensor, code_u32: torch.Tensor, rows_idx: torch.Tensor,
                  group_expert: torch.Tensor, K: int, IC: int, OC: int, R: int, n_rows: int,
                  sort_idx=None) -> torch.Tensor:
    """Row-blocked expert GEMM over ``moe.build_groups`` output (:1366-1395).

    xh [n_rows + 1, IC] f16 (row n_rows is the zero padding sink), rows_idx
    [n_groups * R] i32 with padding == n_rows, group_expert [n_groups] i32 with -1
    past the end.  Returns mid [n_rows + 1, OC] f32 whose padding row is zero.
    ``sort_idx`` (the reference's sorted-x addressing) is accepted and ignored:
    the kernel gathers rows by index either way.
    """
    _check_code(code_u32)
    n_groups = group_expert.shape[0]
    if gemv_family() == "reforder":
        row_expert = torch.zeros(n_rows + 1, dtype=torch.int32, device=xh.device)
        ge = group_expert.clamp(min=0).repeat_interleave(R)
        row_expert.scatter_(0, rows_idx.long(), ge)
        # padding slots point at the zero sink row n_rows and yield a zero row
        return _gemv_reforder(xh, code_u32, row_expert, K, IC, OC, 1, row_map=rows_idx,
                              n_out=n_rows + 1)
    rows_per_job = 8 if R <= 8 else 16
    per_group = (R + rows_per_job - 1) // rows_per_job
    jobs = torch.empty((n_groups * per_group, JOB_INTS), dtype=torch.int32, device=xh.device)
    check(lib.escha_jobs_from_groups(ptr(_i32(rows_idx)), ptr(_i32(group_expert)), n_groups, R,
                                     n_rows, rows_per_job, ptr(jobs), stream()))
    E = code_u32.shape[0]
    out = torch.zeros((n_rows + 1, OC), dtype=torch.float32, device=xh.device)
    coded_gemv_jobs(xh, code_u32, jobs, None, K, IC, OC, E, None, rows_per_job=rows_per_job,
                    out=out, policy_rows=n_rows)
    return out


# ---------------------------------------------------------------------------
# elementwise stages of the routed-expert path
# ---------------------------------------------------------------------------

def swiglu(gu16: torch.Tensor) -> torch.Tensor:
    """gu16 [m, 2I] f16 (gate first) -> f16(f16(silu(g)) * u) [m, I]
    (models/qwen3_5_moe.py:221-223 of the reference)."""
    m, two_i = gu16.shape
    inter = two_i // 2
    h = torch.empty((m, inter), dtype=torch.float16, device=gu16.device)
    base = ptr(gu16, torch.float16)
    check(lib.escha_swiglu(base, ctypes.c_void_p(base.value + 2 * inter), m, inter, two_i, ptr(h),
                           stream()))
    return h


def swiglu_pair(gate16: torch.Tensor, up16: torch.Tensor) -> torch.Tensor:
    """Same stage for gate and up held in two [m, I] f16 tensors (a dense MLP)."""
    m, inter = gate16.shape
    if up16.shape != gate16.shape:
        raise ValueError("swiglu_pair needs gate and up of equal shape")
    h = torch.empty((m, inter), dtype=torch.float16, device=gate16.device)
    check(lib.escha_swiglu(ptr(gate16, torch.float16), ptr(up16, torch.float16), m, inter, inter,
                           ptr(h), stream()))
    return h


def moe_combine(d16: torch.Tensor, scores: torch.Tensor, T: int, top_k: int) -> torch.Tensor:
    """Fixed slot-order combine -> f16 [T, H] (models/qwen3_5_moe.py:227-253)."""
    H = d16.shape[1]
    y = torch.empty((T, H), dtype=torch.float16, device=d16.device)
    check(lib.escha_moe_combine(ptr(d16, torch.float16), ptr(scores, torch.float32), T, top_k, H,
                                ptr(y), stream()))
    return y


ROUTE_MAX_EXPERTS, ROUTE_MAX_TOP_K = 1024, 16


def moe_route(x: torch.Tensor, gate_w: torch.Tensor | None, shg_w: torch.Tensor | None, top_k: int,
              E: int, ids: torch.Tensor | None = None, expert_range: tuple[int, int] | None = None,
              R: int = 8, group: bool = True):
    """Router, shared-gate logit and row grouping in one launch
    (models/qwen3_5_moe.py:255-268 + moe.py:30-83).

    x [T, H] f16.  With ``ids`` None the routing is computed from ``gate_w`` [E, H]:
    returns ``(ids [T, k] i32, scores [T, k] f32, shared_gate_logit [T] f32 | None,
    jobs | None)``; with ``ids`` given only the logit and the jobs are produced and
    ``scores`` comes back None.  ``expert_range`` restricts the jobs to this rank's
    experts (local indices)."""
    T, H = x.shape
    dev = x.device
    lo, hi = expert_range or (0, E)
    ids_in = None
    if ids is not None:
        ids_in = ids.to(torch.int32).contiguous()
        out_ids = out_scores = scratch = None
    else:
        out_ids = torch.empty((T, top_k), dtype=torch.int32, device=dev)
        out_scores = torch.empty((T, top_k), dtype=torch.float32, device=dev)
        scratch = torch.empty((T, E), dtype=torch.float32, device=dev)
    slog = torch.empty((T,), dtype=torch.float32, device=dev) if shg_w is not None else None
    jobs, cap = None, 0
    if group:
        cap = jobs_bound(T * top_k, hi - lo, R)
        jobs = torch.empty((cap, JOB_INTS), dtype=torch.int32, device=dev)
    ws = workspaces.get(1 << 20, dev)
    check(lib.escha_moe_route(ptr(x, torch.float16),
                              ptr(gate_w, torch.float16) if gate_w is not None else None,
                              ptr(shg_w, torch.float16) if shg_w is not None else None,
                              ptr(ids_in), T, H, E, top_k, lo, hi, R, ptr(out_ids), ptr(out_scores),
                              ptr(slog), ptr(scratch), ptr(jobs), cap, ptr(ws),
                              ctypes.c_size_t(ws.numel()), stream()))
    return (ids_in if ids is not None else out_ids), out_scores, slog, jobs


def moe_shared_finish(gu: torch.Tensor, w8: torch.Tensor, scale: torch.Tensor, d16: torch.Tensor,
                      scores: torch.Tensor, shared_gate_logit: torch.Tensor, top_k: int,
                      ids: torch.Tensor | None = None, experts_per_rank: int = 0) -> torch.Tensor:
    """Shared expert's SwiGLU + down linear, routed-expert combine and the gated add
    in one launch -> out f16 [T, H] (models/qwen3_5_moe.py:227-273).  Expert
    parallel: ``d16`` is the all-gathered [ranks * T * top_k, H] buffer and ``ids``
    [T, top_k] selects each row from the copy of the rank that owns its expert."""
    T, two_i = gu.shape
    H, inter = w8.shape
    m = T * top_k
    ranks = d16.shape[0] // m if ids is not None else 1
    if two_i != 2 * inter or d16.shape != (ranks * m, H):
        raise ValueError(f"shapes do not form a shared-expert tail: gu {tuple(gu.shape)}, "
                         f"w8 {tuple(w8.shape)}, d16 {tuple(d16.shape)}, top_k {top_k}")
    out = torch.empty((T, H), dtype=torch.float16, device=gu.device)
    check(lib.escha_moe_shared_finish(ptr(gu, torch.float16), ptr(w8, torch.int8),
                                      ptr(scale, torch.float16), ptr(d16, torch.float16),
                                      ptr(ids, torch.int32) if ids is not None else None,
                                      int(experts_per_rank), ptr(scores, torch.float32),
                                      ptr(shared_gate_logit, torch.float32),
                                      T, top_k, H, inter, ptr(out), stream()))
    return out


def dense_gemm_tc(xh: torch.Tensor, code_u32: torch.Tensor, K: int, IC: int, OC: int,
                  splits: int | None = None, rout: torch.Tensor | None = None,
                  rs: float = RS) -> torch.Tensor:
    """Prefill coded GEMM on the tcgen05 tensor cores (the product of dense_gemm_mat,
    msl.py:1608-1782, decoded once per 256 rows).  Returns mid f32 [M, OC], or with
    ``rout`` the transformed output f16 [M, OC] (split-order sum and output transform
    as one second kernel)."""
    _check_code(code_u32)
    m = xh.shape[0]
    if m < 1:
        raise ValueError("dense_gemm_tc needs at least one row")
    s = int(lib.escha_coded_gemm_tc_splits(IC, OC, 0)) if splits is None else int(splits)
    out = torch.empty((m, OC), dtype=torch.float32 if rout is None else torch.float16,
                      device=xh.device)
    # scratch only when the library will use it (split sums inside the kernel need none)
    need = lib.escha_coded_gemm_tc_needs_planes(IC, s, 1 if rout is not None else 0)
    planes = torch.empty((s, m, OC), dtype=torch.float32, device=xh.device) if need else None
    check(lib.escha_coded_gemm_tc(ptr(xh, torch.float16), ptr(code_u32),
                                  ptr(rout, torch.float32) if rout is not None else None,
                                  m, IC, OC, K, s, float(rs), ptr(planes), ptr(out), stream()))
    return out


@lru_cache(maxsize=None)
def _sm_count(device_index: int) -> int:
    return int(torch.cuda.get_device_properties(device_index).multi_processor_count)


def sm_count() -> int:
    """Streaming multiprocessors of the current device."""
    return _sm_count(torch.cuda.current_device())


def dense_gemm_tc_many(xhs, codes, K: int, IC: int, OCs, routs, rs: float = RS,
                       splits: int | None = None):
    """One to three prefill projections of equal IC and K in one tcgen05 launch (Q/K/V; the
    launch-sharing of dense_gemm_pair_out, msl.py:1880-1950, widened).  ``xhs[i]`` f16 [M, IC]
    are the transformed activations of projection i; returns the transformed outputs f16
    [M, OCs[i]].  The split factor is chosen for the summed width, so outputs are
    tolerance-equal, not bit-equal, to separate ``dense_gemm_tc`` calls."""
    n = len(codes)
    if not (1 <= n <= 3 and len(xhs) == n and len(OCs) == n and len(routs) == n):
        raise ValueError("dense_gemm_tc_many takes one to three projections with matching lists")
    m = xhs[0].shape[0]
    if m < 1 or any(x.shape != (m, IC) for x in xhs):
        raise ValueError("dense_gemm_tc_many needs equal [M, IC] activations for every projection")
    for c in codes:
        _check_code(c)
    s = int(lib.escha_coded_gemm_tc_splits(IC, int(sum(OCs)), 0)) if splits is None else int(splits)
    dev = xhs[0].device
    outs = [torch.empty((m, oc), dtype=torch.float16, device=dev) for oc in OCs]
    need = lib.escha_coded_gemm_tc_needs_planes(IC, s, 1)   # the joint launch always has routs
    planes = [torch.empty((s, m, oc), dtype=torch.float32, device=dev) for oc in OCs] if need else None
    arr = ctypes.c_void_p * n
    check(lib.escha_coded_gemm_tc_many(
        n, arr(*[ptr(x, torch.float16) for x in xhs]), arr(*[ptr(c) for c in codes]),
        arr(*[ptr(r, torch.float32) for r in routs]), m, IC, (ctypes.c_int * n)(*[int(o) for o in OCs]),
        K, s, float(rs), arr(*[ptr(t) for t in planes]) if planes else None,
        arr(*[ptr(o) for o in outs]), stream()))
    return outs

"""NumPy-facing wrapper around the CPU oracle (``libescha_oracle.so``).

TEST INFRASTRUCTURE ONLY: the checker for the CUDA kernels and the CPU baseline
leg of the benchmark.  The product package never imports this module.

Function names and argument meaning follow the reference's NumPy module
``escha_mlx/ref.py`` (cited per function in ``escha_oracle.c``), so a parity test
written against this module reads like the reference's own tests.  All arrays
are NumPy; half-precision arrays are ``np.float16``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libescha_oracle.so")

RS = 0.088388347648  # escha_mlx/ref.py:30


def build(force: bool = False) -> str:
    """Compile the C restatement with the Makefile beside it; returns the .so path."""
    src = os.path.join(_HERE, "escha_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True,
                       stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.esc_num_threads.restype = ctypes.c_int
    return _lib


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def _h(a) -> np.ndarray:
    """float16 array -> contiguous uint16 view of its bits."""
    return np.ascontiguousarray(np.asarray(a, dtype=np.float16)).view(np.uint16)


def code_to_u32(code_i16: np.ndarray) -> np.ndarray:
    """int16 [..., 16K] -> little-endian uint32 [..., 8K] (escha_mlx/msl.py:1398-1401)."""
    a = np.ascontiguousarray(code_i16)
    if a.dtype == np.uint32:
        return a
    return a.view(np.uint16).view(np.uint32)


def num_threads() -> int:
    return int(lib().esc_num_threads())


def set_num_threads(n: int) -> None:
    lib().esc_set_num_threads(ctypes.c_int(n))


def cba_lut() -> np.ndarray:
    out = np.empty(65536, dtype=np.uint16)
    lib().esc_cba_lut(_p(out))
    return out.view(np.float16)


def tile_states(code: np.ndarray, K: int) -> np.ndarray:
    """code [..., 8K] u32 (or int16 [..., 16K]) -> states [tiles, 32, 8] uint16."""
    c = code_to_u32(code).reshape(-1, 8 * K)
    out = np.empty((c.shape[0], 32, 8), dtype=np.uint16)
    lib().esc_tile_states(_p(c), ctypes.c_long(c.shape[0]), ctypes.c_int(K), _p(out))
    return out


def reconstruct(code: np.ndarray, in_features: int, out_features: int, K: int) -> np.ndarray:
    """packed (in/16, out/16, 16K) int16 or (.., 8K) uint32 -> (in, out) float16."""
    c = code_to_u32(code).reshape(-1)
    assert c.size == (in_features // 16) * (out_features // 16) * 8 * K, c.size
    out = np.empty((in_features, out_features), dtype=np.uint16)
    lib().esc_reconstruct(_p(c), ctypes.c_int(in_features), ctypes.c_int(out_features),
                          ctypes.c_int(K), _p(out))
    return out.view(np.float16)


reconstruct_fast = reconstruct


def h128(x: np.ndarray) -> np.ndarray:
    shape = x.shape
    assert shape[-1] % 128 == 0, shape
    y = np.array(x, dtype=np.float32, order="C", copy=True).reshape(-1, shape[-1])
    lib().esc_h128(_p(y), ctypes.c_long(y.shape[0]), ctypes.c_int(y.shape[1]))
    return y.reshape(shape)


def _re(row_expert):
    return None if row_expert is None else _c(row_expert, np.int32)


def input_transform(x: np.ndarray, rin: np.ndarray, row_expert=None) -> np.ndarray:
    """xh = f16(H128(x*rin)*RS).  rin [IC], or [E, IC] gathered by row_expert."""
    x2 = np.asarray(x, dtype=np.float16)
    m, ic = x2.reshape(-1, x2.shape[-1]).shape
    xb = _h(x2)
    r = _c(rin, np.float32)
    re = _re(row_expert)
    assert (r.ndim == 2) == (re is not None)
    out = np.empty((m, ic), dtype=np.uint16)
    lib().esc_input_transform(_p(xb), _p(r), _p(re), ctypes.c_int(m), ctypes.c_int(ic), _p(out))
    return out.view(np.float16).reshape(x2.shape)


def output_transform(mid: np.ndarray, rout: np.ndarray, row_expert=None) -> np.ndarray:
    """y = f16(H128(mid)*RS*rout).  mid [..., OC] f32."""
    md = _c(mid, np.float32)
    m, oc = md.reshape(-1, md.shape[-1]).shape
    r = _c(rout, np.float32)
    re = _re(row_expert)
    assert (r.ndim == 2) == (re is not None)
    out = np.empty((m, oc), dtype=np.uint16)
    lib().esc_output_transform(_p(md), _p(r), _p(re), ctypes.c_int(m), ctypes.c_int(oc), _p(out))
    return out.view(np.float16).reshape(md.shape)


def gemv_ref_order(xh: np.ndarray, code: np.ndarray, row_expert, K: int, IC: int,
                   OC: int) -> np.ndarray:
    """mid [M, OC] f32 in the reference kernels' accumulation order."""
    xb = _h(xh).reshape(-1, IC)
    c = code_to_u32(code).reshape(-1)
    re = _re(row_expert)
    out = np.empty((xb.shape[0], OC), dtype=np.float32)
    lib().esc_gemv_ref_order(_p(xb), _p(c), _p(re), ctypes.c_int(xb.shape[0]), ctypes.c_int(IC),
                             ctypes.c_int(OC), ctypes.c_int(K), _p(out))
    return out


def gemv_f64(xh: np.ndarray, code: np.ndarray, row_expert, K: int, IC: int, OC: int) -> np.ndarray:
    """Exact-product tolerance oracle: float64 accumulate of reference-decoded weights."""
    xb = _h(xh).reshape(-1, IC)
    c = code_to_u32(code).reshape(-1)
    re = _re(row_expert)
    out = np.empty((xb.shape[0], OC), dtype=np.float64)
    lib().esc_gemv_f64(_p(xb), _p(c), _p(re), ctypes.c_int(xb.shape[0]), ctypes.c_int(IC),
                       ctypes.c_int(OC), ctypes.c_int(K), _p(out))
    return out


def fold_scales(rin, rout, s_in=None, s_out=None):
    """escha_mlx/ref.py:242-277: rin_eff = f32(rin)*f32(s_in), rout likewise."""
    ri = np.asarray(rin).astype(np.float32)
    ro = np.asarray(rout).astype(np.float32)
    if s_in is not None:
        ri = ri * np.asarray(s_in).astype(np.float32)
    if s_out is not None:
        ro = ro * np.asarray(s_out).astype(np.float32)
    return ri, ro


def expert_linear(x, code, rin, rout, K: int, row_expert=None, bias=None) -> np.ndarray:
    """Full coded linear x [M, IC] -> [M, OC] float16 (escha_mlx/ref.py:231-293)."""
    r_in = _c(rin, np.float32)
    r_out = _c(rout, np.float32)
    ic, oc = r_in.shape[-1], r_out.shape[-1]
    xb = _h(x).reshape(-1, ic)
    c = code_to_u32(code).reshape(-1)
    re = _re(row_expert)
    b = None if bias is None else _h(bias)
    out = np.empty((xb.shape[0], oc), dtype=np.uint16)
    rc = lib().esc_linear(_p(xb), _p(c), _p(r_in), _p(r_out), _p(re), _p(b),
                          ctypes.c_int(xb.shape[0]), ctypes.c_int(ic), ctypes.c_int(oc),
                          ctypes.c_int(K), _p(out))
    assert rc == 0
    return out.view(np.float16)


def dense_linear(x, code, rin, rout, K: int, bias=None) -> np.ndarray:
    return expert_linear(x, code, rin, rout, K, None, bias)


def swiglu(gate_up_f16: np.ndarray) -> np.ndarray:
    g = _h(gate_up_f16)
    m, two_i = g.reshape(-1, g.shape[-1]).shape
    out = np.empty((m, two_i // 2), dtype=np.uint16)
    lib().esc_swiglu(_p(g), ctypes.c_int(m), ctypes.c_int(two_i // 2), _p(out))
    return out.view(np.float16)


def w8a16(x, w8, scale) -> np.ndarray:
    xb = _h(x)
    w = _c(w8, np.int8)
    n, kd = w.shape
    xb = xb.reshape(-1, kd)
    sc = np.asarray(scale).astype(np.float32)
    out = np.empty((xb.shape[0], n), dtype=np.uint16)
    lib().esc_w8a16(_p(xb), _p(w), _p(sc), ctypes.c_int(xb.shape[0]), ctypes.c_int(n),
                    ctypes.c_int(kd), _p(out))
    return out.view(np.float16)


def moe_routed(x, ids, scores, gu_code, gu_rin, gu_rout, Kg, dn_code, dn_rin, dn_rout, Kd):
    """Routed-expert path (token-major rows, fixed slot-order combine) -> float16 [T, H]."""
    xb = _h(x)
    t, hdim = xb.shape
    idv = _c(ids, np.int32)
    top_k = idv.shape[1]
    sc = _c(scores, np.float32)
    gr, go = _c(gu_rin, np.float32), _c(gu_rout, np.float32)
    dr, do = _c(dn_rin, np.float32), _c(dn_rout, np.float32)
    inter = go.shape[-1] // 2
    gc = code_to_u32(gu_code).reshape(-1)
    dc = code_to_u32(dn_code).reshape(-1)
    out = np.empty((t, hdim), dtype=np.uint16)
    rc = lib().esc_moe_routed(_p(xb), _p(idv), _p(sc), ctypes.c_int(t), ctypes.c_int(top_k),
                              ctypes.c_int(hdim), ctypes.c_int(inter), _p(gc), _p(gr), _p(go),
                              ctypes.c_int(Kg), _p(dc), _p(dr), _p(do), ctypes.c_int(Kd), _p(out))
    assert rc == 0
    return out.view(np.float16)


def moe_shared_add(x, y16, shared: dict, shg_w) -> np.ndarray:
    """out = f16(f32(y16) + shared_expert(x) * sigmoid(x @ shg_w^T))."""
    xb = _h(x)
    t, hdim = xb.shape
    yb = _h(y16)
    gw, uw, dw = (_c(shared[k], np.int8) for k in ("gate_w8", "up_w8", "down_w8"))
    gs, us, ds = (np.asarray(shared[k]).astype(np.float32)
                  for k in ("gate_scale", "up_scale", "down_scale"))
    inter = gw.shape[0]
    sg = _h(np.asarray(shg_w).reshape(-1))
    out = np.empty((t, hdim), dtype=np.uint16)
    rc = lib().esc_moe_shared_add(_p(xb), _p(yb), ctypes.c_int(t), ctypes.c_int(hdim),
                                  ctypes.c_int(inter), _p(gw), _p(gs), _p(uw), _p(us), _p(dw),
                                  _p(ds), _p(sg), _p(out))
    assert rc == 0
    return out.view(np.float16)


def router(x, gate_w, top_k: int):
    """fp32 logits rounded through f16, stable top-k, softmax over the k values
    (escha_mlx/ref.py:326-331).  Returns (ids int32 [T, k], scores f32 [T, k])."""
    logits = (np.asarray(x, np.float16).astype(np.float32)
              @ np.asarray(gate_w, np.float16).astype(np.float32).T
              ).astype(np.float16).astype(np.float32)
    ids = np.argsort(-logits, axis=-1, kind="stable")[:, :top_k]
    top = np.take_along_axis(logits, ids, axis=-1)
    e = np.exp(top - top.max(axis=-1, keepdims=True))
    return ids.astype(np.int32), (e / e.sum(axis=-1, keepdims=True)).astype(np.float32)


def build_groups(row_expert, E: int, R: int, n_groups: int):
    re = _c(row_expert, np.int32)
    rows_idx = np.empty(n_groups * R, dtype=np.int32)
    group_expert = np.empty(n_groups, dtype=np.int32)
    lib().esc_build_groups(_p(re), ctypes.c_int(re.shape[0]), ctypes.c_int(E), ctypes.c_int(R),
                           ctypes.c_int(n_groups), _p(rows_idx), _p(group_expert))
    return rows_idx, group_expert


def n_groups_bound(m: int, E: int, R: int) -> int:
    return (m + E * (R - 1) + R - 1) // R

"""Seeded synthetic tensors in the reference's checkpoint formats (NumPy only).

The reference's own benches and tests feed the coded path uniform-random code
streams, because the trellis is tail-biting and every bit string decodes to a
valid weight (tests/test_dense_linear.py:263-268, bench/p0_gates.py:86-96,
bench/roofline.py:126-131 in the reference).  These generators reproduce that
recipe with one ``numpy.random.default_rng(seed)`` per case and a fixed draw
order, so tests, fixtures and the benchmark all see identical inputs.

Draw order for one coded projection: code, scale_in, sign_in, scale_out, sign_out.
"""
from __future__ import annotations

import numpy as np


def signed_scale(rng: np.random.Generator, shape) -> np.ndarray:
    """(|N(0, 0.02)| + 1e-3) * random sign, as float16 -- the folded per-channel
    scale-and-sign vector form the reference stores as ``escha_rin``/``escha_rout``."""
    scale = np.abs(rng.normal(0.0, 0.02, size=shape)) + 1e-3
    sign = rng.choice(np.array([-1.0, 1.0]), size=shape)
    return (scale * sign).astype(np.float16)


def coded_projection(rng: np.random.Generator, IC: int, OC: int, K: int, E: int | None = None):
    """-> (code int16 [E?, IC/16, OC/16, 16K], rin f16 [E?, IC], rout f16 [E?, OC])."""
    lead = () if E is None else (E,)
    code = rng.integers(-32768, 32768, size=lead + (IC // 16, OC // 16, 16 * K), dtype=np.int16)
    rin = signed_scale(rng, lead + (IC,))
    rout = signed_scale(rng, lead + (OC,))
    return code, rin, rout


def activations(rng: np.random.Generator, M: int, IC: int) -> np.ndarray:
    return rng.standard_normal((M, IC)).astype(np.float16)


def router_logits(rng: np.random.Generator, T: int, E: int) -> np.ndarray:
    return rng.standard_normal((T, E)).astype(np.float32)


def topk_softmax(logits: np.ndarray, top_k: int):
    """Stable top-k of f32 logits and softmax over the k values
    (escha_mlx/ref.py:328-331) -> (ids int32 [T, k], scores f32 [T, k])."""
    ids = np.argsort(-logits, axis=-1, kind="stable")[:, :top_k]
    top = np.take_along_axis(logits, ids, axis=-1)
    e = np.exp(top - top.max(axis=-1, keepdims=True))
    return ids.astype(np.int32), (e / e.sum(axis=-1, keepdims=True)).astype(np.float32)


def int8_linear(rng: np.random.Generator, N: int, Kd: int):
    """-> (w8 int8 [N, Kd], scale f16 [N]) as tests/test_models.py:62-64 draws them."""
    w8 = rng.integers(-128, 128, size=(N, Kd), dtype=np.int8)
    scale = (rng.random(N) * 0.01 + 1e-3).astype(np.float16)
    return w8, scale


def moe_weights(rng: np.random.Generator, E: int, H: int, I: int, Kg: int = 2, Kd: int = 2):
    """Weights of one MoE block in the key layout ``ref.moe_block`` documents
    (escha_mlx/ref.py:318-320)."""
    gu_code, gu_rin, gu_rout = coded_projection(rng, H, 2 * I, Kg, E)
    dn_code, dn_rin, dn_rout = coded_projection(rng, I, H, Kd, E)
    w = {
        "gate_w": (rng.standard_normal((E, H)) * 0.05).astype(np.float16),
        "gu_code": gu_code, "gu_rin": gu_rin, "gu_rout": gu_rout,
        "dn_code": dn_code, "dn_rin": dn_rin, "dn_rout": dn_rout,
        "shg_w": (rng.standard_normal((1, H)) * 0.05).astype(np.float16),
    }
    for name, (n, kd) in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I))):
        w8, sc = int8_linear(rng, n, kd)
        w[f"sh_{name}_w8"], w[f"sh_{name}_scale"] = w8, sc
    return w


# Shapes of the published benchmark configurations.
DENSE_LAYER_27B = (
    # name, IC, OC, K
    ("q_proj", 5120, 6144, 2),
    ("k_proj", 5120, 1024, 2),
    ("v_proj", 5120, 1024, 2),
    ("o_proj", 5120, 5120, 2),
    ("gate_proj", 5120, 17408, 3),
    ("up_proj", 5120, 17408, 3),
    ("down_proj", 17408, 5120, 3),
)

MOE_35B = dict(E=256, top_k=8, H=2048, I=512, Kg=2, Kd=2)


def coded_bytes(IC: int, OC: int, K: int) -> int:
    """Bytes of one projection's code stream: IC*OC*K/8."""
    return IC * OC * K // 8

"""Regenerates the fixtures in this directory from the reference checkout.

Run where the reference tree is available (it is not on the GPU machine):

    python tests/golden/make_golden.py [/path/to/escha-mlx]

Two kinds of fixture are written:

* ``ref_*.npz`` -- the reference's own committed golden vectors for this path
  (tests/data/codec, tests/data/qwen3_5 of the reference), reduced where they
  are large: the packed code streams are kept whole, the 6 MB of expected
  decoded weights are kept as SHA-256 digests plus corner blocks, and the 4 MB
  int8 matrix is cut to its first 128 output rows.
* ``seeded_*.npz`` -- outputs of the reference's NumPy module
  ``escha_mlx/ref.py`` (imported by file path; the package ``__init__`` needs
  mlx, which is not installable here) on seeded synthetic inputs drawn by
  ``escha_mlx_b200.synth``.  Inputs are regenerated from the seed at test time;
  only the reference outputs are stored.
"""
from __future__ import annotations

import hashlib
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from escha_mlx_b200 import synth  # noqa: E402


def load_ref(root: str):
    spec = importlib.util.spec_from_file_location(
        "escha_ref", os.path.join(root, "escha_mlx", "ref.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


# (name, seed, K, IC, OC): decode cases, rectangular and multi-block on purpose
DECODE_CASES = (
    ("k2_64x160", 11, 2, 64, 160),
    ("k3_160x64", 12, 3, 160, 64),
    ("k2_256x384", 13, 2, 256, 384),
    ("k3_384x256", 14, 3, 384, 256),
)

# (name, seed, K, IC, OC, M, E): full linears; E=None is the dense form
LINEAR_CASES = (
    ("dense_k2", 21, 2, 256, 384, 3, None),
    ("dense_k3", 22, 3, 384, 256, 5, None),
    ("expert_k2", 23, 2, 256, 128, 6, 4),
    ("expert_k3", 24, 3, 128, 256, 6, 4),
)

MOE_CASE = dict(seed=31, E=8, H=256, I=128, top_k=2, T=4)


def linear_inputs(seed, K, IC, OC, M, E):
    rng = np.random.default_rng(seed)
    code, rin, rout = synth.coded_projection(rng, IC, OC, K, E)
    x = synth.activations(rng, M, IC)
    row_expert = None if E is None else rng.integers(0, E, size=M).astype(np.int32)
    return code, rin, rout, x, row_expert


def moe_inputs():
    c = MOE_CASE
    rng = np.random.default_rng(c["seed"])
    # ref.moe_block decodes gate_up at K=2 and down at K=3 (escha_mlx/ref.py:336-340)
    w = synth.moe_weights(rng, c["E"], c["H"], c["I"], Kg=2, Kd=3)
    x = synth.activations(rng, c["T"], c["H"])
    return w, x


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to an escha-mlx checkout>")
    root = sys.argv[1]
    ref = load_ref(root)
    data = os.path.join(root, "tests", "data")

    # ---- reference goldens: codec -------------------------------------------
    p2 = np.fromfile(os.path.join(data, "codec/packed_gu_e0_k2.i16"), np.int16).reshape(128, 64, 32)
    e2 = np.fromfile(os.path.join(data, "codec/expected_gu_e0_k2.f16"), np.float16).reshape(2048, 1024)
    p3 = np.fromfile(os.path.join(data, "codec/packed_down_e0_k3.i16"), np.int16).reshape(32, 128, 48)
    e3 = np.fromfile(os.path.join(data, "codec/expected_down_e0_k3.f16"), np.float16).reshape(512, 2048)
    np.savez_compressed(
        os.path.join(HERE, "ref_codec.npz"),
        k2_packed=p2, k2_sha256=np.array(sha(e2)), k2_corner=e2[:64, :64], k2_tail=e2[-32:, -48:],
        k3_packed=p3, k3_sha256=np.array(sha(e3)), k3_corner=e3[:64, :64], k3_tail=e3[-32:, -48:],
        lut_sha256=np.array(sha(ref.cba_lut())),
    )

    # ---- reference goldens: full dense linear (128x128 corner of a shipped one)
    lin = {}
    for k in (2, 3):
        q = os.path.join(data, "qwen3_5", f"lin_k{k}_")
        lin[f"k{k}_code"] = np.fromfile(q + "code.i16", np.int16).reshape(8, 8, 16 * k)
        for leaf, dt in (("rin", np.float16), ("rout", np.float16), ("s_in", np.float32),
                         ("s_out", np.float32), ("bias", np.float16)):
            lin[f"k{k}_{leaf}"] = np.fromfile(q + leaf + "." + ("f16" if dt == np.float16 else "f32"), dt)
        lin[f"k{k}_x"] = np.fromfile(q + "x.f16", np.float16).reshape(8, 128)
        lin[f"k{k}_deploy"] = np.fromfile(q + "deploy.f16", np.float16).reshape(8, 128)
    np.savez_compressed(os.path.join(HERE, "ref_dense_linear.npz"), **lin)

    # ---- reference goldens: int8 linear (first 128 of 2048 output rows) -------
    w8 = np.fromfile(os.path.join(data, "codec/w8a16_w8_2048x2048.i8"), np.int8).reshape(2048, 2048)
    sc = np.fromfile(os.path.join(data, "codec/w8a16_scale_2048.f32"), np.float32)
    x8 = np.fromfile(os.path.join(data, "codec/w8a16_x_8x2048.f16"), np.float16).reshape(8, 2048)
    ex = np.fromfile(os.path.join(data, "codec/w8a16_expected_8x2048.f16"), np.float16).reshape(8, 2048)
    np.savez_compressed(os.path.join(HERE, "ref_w8a16.npz"),
                        w8=w8[:128], scale=sc[:128], x=x8, expected=ex[:, :128])

    # ---- seeded: decode -------------------------------------------------------
    dec = {}
    for name, seed, K, IC, OC in DECODE_CASES:
        rng = np.random.default_rng(seed)
        code, _, _ = synth.coded_projection(rng, IC, OC, K)
        w = ref.reconstruct_fast(code, IC, OC, K)
        assert np.array_equal(w.view(np.uint16), ref.reconstruct(code, IC, OC, K).view(np.uint16))
        if w.size <= 16384:
            dec[name] = w
        else:
            dec[name + "_sha256"] = np.array(sha(w))
            dec[name + "_corner"] = w[:48, :80]
    np.savez_compressed(os.path.join(HERE, "seeded_decode.npz"), **dec)

    # ---- seeded: transforms + full linears ------------------------------------
    out = {}
    for name, seed, K, IC, OC, M, E in LINEAR_CASES:
        code, rin, rout, x, re = linear_inputs(seed, K, IC, OC, M, E)
        ri, ro = ref.fold_scales(rin, rout, None, None)
        if E is None:
            xh = ref.input_transform(x, ri)
            w = ref.reconstruct_fast(code, IC, OC, K).astype(np.float32)
            mid = xh.astype(np.float32) @ w
            y = ref.expert_linear(x, code, ri, ro, K)
            yt = ref.output_transform(mid, ro)
        else:
            xh = np.stack([ref.input_transform(x[r], ri[re[r]]) for r in range(M)])
            mid = np.stack([xh[r].astype(np.float32)
                            @ ref.reconstruct_fast(code[re[r]], IC, OC, K).astype(np.float32)
                            for r in range(M)])
            y = np.concatenate([ref.expert_linear(x[r:r + 1], code[re[r]], ri[re[r]], ro[re[r]], K)
                                for r in range(M)])
            yt = np.stack([ref.output_transform(mid[r], ro[re[r]]) for r in range(M)])
        out[name + "_xh"] = xh
        out[name + "_mid"] = mid.astype(np.float32)
        out[name + "_y_from_mid"] = yt
        out[name + "_y"] = y
    rng = np.random.default_rng(41)
    gu = (rng.standard_normal((7, 192)) * 2.0).astype(np.float16)
    out["swiglu_in"] = gu
    out["swiglu_out"] = ref.swiglu(gu)
    np.savez_compressed(os.path.join(HERE, "seeded_linear.npz"), **out)

    # ---- seeded: whole MoE block ----------------------------------------------
    w, x = moe_inputs()
    full = ref.moe_block(x, w, top_k=MOE_CASE["top_k"])
    logits = (x.astype(np.float32) @ w["gate_w"].astype(np.float32).T).astype(np.float16).astype(np.float32)
    ids, scores = synth.topk_softmax(logits, MOE_CASE["top_k"])
    injected = ref.moe_block(x, w, top_k=MOE_CASE["top_k"], ids=ids, scores=scores)
    assert np.array_equal(full.view(np.uint16), injected.view(np.uint16))
    np.savez_compressed(os.path.join(HERE, "seeded_moe_block.npz"),
                        out=full, ids=ids, scores=scores)

    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()

"""CPU: the oracle (C restatement of escha_mlx/ref.py and of the reference
kernels' accumulation order) against the reference's golden vectors and against
reference outputs on seeded inputs.  Mirrors tests/test_ref_decode.py,
tests/test_dense_linear.py:43-111 and tests/test_mlx_cpu.py:55-132 of the
reference."""
from __future__ import annotations

import numpy as np
import pytest

from cases import (DECODE_CASES, LINEAR_CASES, MOE_CASE, bits, linear_inputs, moe_inputs,
                   rel_err, sha)
from escha_mlx_b200 import synth


def test_lut_matches_reference(oracle, ref_codec):
    lut = oracle.cba_lut()
    assert sha(lut) == str(ref_codec["lut_sha256"])
    # the two addends can cancel to exactly zero, but never to an fp16 subnormal
    b = bits(lut)
    assert not np.any((((b >> 10) & 0x1F) == 0) & ((b & 0x3FF) != 0))


def test_lane_positions_bijection(oracle):
    """Every (row, col) of the 16x16 tile is owned by exactly one (lane, j):
    decode a stream whose states are all distinct per tile position."""
    rng = np.random.default_rng(5)
    code = rng.integers(-32768, 32768, size=(1, 1, 32), dtype=np.int16)
    w = oracle.reconstruct(code, 16, 16, 2)
    states = oracle.tile_states(code, 2)[0]  # [32, 8]
    lut = oracle.cba_lut()
    # the multiset of decoded values equals the multiset of lut[state]
    assert sorted(bits(w).ravel().tolist()) == sorted(bits(lut[states.ravel()]).tolist())


@pytest.mark.parametrize("k", [2, 3])
def test_golden_decode_bit_exact(oracle, ref_codec, k):
    packed = ref_codec[f"k{k}_packed"]
    ic, oc = packed.shape[0] * 16, packed.shape[1] * 16
    got = oracle.reconstruct(packed, ic, oc, k)
    assert sha(got) == str(ref_codec[f"k{k}_sha256"])
    assert np.array_equal(bits(got[:64, :64]), bits(ref_codec[f"k{k}_corner"]))
    assert np.array_equal(bits(got[-32:, -48:]), bits(ref_codec[f"k{k}_tail"]))


@pytest.mark.parametrize("name,seed,K,IC,OC", DECODE_CASES)
def test_seeded_decode_bit_exact(oracle, seeded_decode, name, seed, K, IC, OC):
    rng = np.random.default_rng(seed)
    code, _, _ = synth.coded_projection(rng, IC, OC, K)
    got = oracle.reconstruct(code, IC, OC, K)
    if name in seeded_decode:
        assert np.array_equal(bits(got), bits(seeded_decode[name]))
    else:
        assert sha(got) == str(seeded_decode[name + "_sha256"])
        assert np.array_equal(bits(got[:48, :80]), bits(seeded_decode[name + "_corner"]))


def test_h128_involution(oracle):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((4, 256)).astype(np.float32)
    y = oracle.h128(oracle.h128(x)) / 128.0
    assert np.allclose(y, x, atol=1e-4)


@pytest.mark.parametrize("name,seed,K,IC,OC,M,E", LINEAR_CASES)
def test_seeded_transforms_bit_exact(oracle, seeded_linear, name, seed, K, IC, OC, M, E):
    code, rin, rout, x, re = linear_inputs(seed, K, IC, OC, M, E)
    ri, ro = oracle.fold_scales(rin, rout)
    xh = oracle.input_transform(x, ri, re)
    assert np.array_equal(bits(xh), bits(seeded_linear[name + "_xh"]))
    y = oracle.output_transform(seeded_linear[name + "_mid"], ro, re)
    assert np.array_equal(bits(y), bits(seeded_linear[name + "_y_from_mid"]))


@pytest.mark.parametrize("name,seed,K,IC,OC,M,E", LINEAR_CASES)
def test_seeded_linear_within_tolerance(oracle, seeded_linear, name, seed, K, IC, OC, M, E):
    """The product's summation order differs from NumPy's matmul, so the full
    linear is tolerance-gated: mid within 1e-5 relative, y within one f16 ulp-ish."""
    code, rin, rout, x, re = linear_inputs(seed, K, IC, OC, M, E)
    ri, ro = oracle.fold_scales(rin, rout)
    xh = seeded_linear[name + "_xh"]
    mid = oracle.gemv_ref_order(xh, code, re, K, IC, OC)
    assert rel_err(mid, seeded_linear[name + "_mid"]) < 1e-5
    exact = oracle.gemv_f64(xh, code, re, K, IC, OC)
    assert rel_err(mid, exact) < 1e-5
    y = oracle.expert_linear(x, code, ri, ro, K, re)
    assert rel_err(y, seeded_linear[name + "_y"]) < 2e-3


@pytest.mark.parametrize("k", [2, 3])
def test_golden_dense_linear(oracle, ref_dense_linear, k):
    """Full linear incl. fold_scales and bias against the shipped cross-runtime
    output; mean relative error < 3e-3 as tests/test_dense_linear.py:32,68-78."""
    g = ref_dense_linear
    ri, ro = oracle.fold_scales(g[f"k{k}_rin"], g[f"k{k}_rout"], g[f"k{k}_s_in"], g[f"k{k}_s_out"])
    y = oracle.dense_linear(g[f"k{k}_x"], g[f"k{k}_code"], ri, ro, k, g[f"k{k}_bias"])
    dep = g[f"k{k}_deploy"].astype(np.float64)
    rel = np.abs(y.astype(np.float64) - dep).mean() / np.abs(dep).mean()
    assert rel < 3e-3, rel
    assert np.corrcoef(y.astype(np.float64).ravel(), dep.ravel())[0, 1] > 0.99999


def test_fold_scales_algebra(oracle):
    rng = np.random.default_rng(9)
    rin = synth.signed_scale(rng, 128)
    rout = synth.signed_scale(rng, 256)
    s_in = rng.random(128).astype(np.float32) + 0.5
    ri, ro = oracle.fold_scales(rin, rout, s_in, None)
    assert ri.dtype == np.float32 and ro.dtype == np.float32
    assert np.array_equal(ri, rin.astype(np.float32) * s_in)
    assert np.array_equal(ro, rout.astype(np.float32))


def test_swiglu_bit_exact(oracle, seeded_linear):
    got = oracle.swiglu(seeded_linear["swiglu_in"])
    want = seeded_linear["swiglu_out"]
    # expf differs between libraries by an ulp: allow one f16 ulp on rare elements
    diff = np.abs(bits(got).astype(np.int32) - bits(want).astype(np.int32))
    assert diff.max() <= 1 and (diff > 0).mean() < 0.01


def test_golden_w8a16(oracle, ref_w8a16):
    """2e-3 relative, the reference's own bar (tests/test_mlx_cpu.py:55-65)."""
    g = ref_w8a16
    y = oracle.w8a16(g["x"], g["w8"], g["scale"])
    assert rel_err(y, g["expected"]) < 2e-3


def test_moe_block_vs_reference(oracle, seeded_moe_block):
    """Whole block (router, routed experts, shared expert) against ref.moe_block
    on synthetic weights; 5e-2 is the reference's bar for its own fused path
    (tests/test_mlx_cpu.py:129-132), the oracle is far inside it."""
    w, x = moe_inputs()
    ids, scores = oracle.router(x, w["gate_w"], MOE_CASE["top_k"])
    assert np.array_equal(ids, seeded_moe_block["ids"])
    assert np.allclose(scores, seeded_moe_block["scores"], rtol=1e-6)
    y16 = oracle.moe_routed(x, ids, scores, w["gu_code"], w["gu_rin"], w["gu_rout"], 2,
                            w["dn_code"], w["dn_rin"], w["dn_rout"], 3)
    shared = {k[3:]: v for k, v in w.items() if k.startswith("sh_")}
    out = oracle.moe_shared_add(x, y16, shared, w["shg_w"])
    assert rel_err(out, seeded_moe_block["out"]) < 5e-3


def test_build_groups_model(oracle):
    """Grouping against an independent NumPy model (tests/test_blocked.py:25-66)."""
    rng = np.random.default_rng(17)
    E, R, m = 16, 4, 37
    row_expert = rng.integers(0, E, size=m).astype(np.int32)
    ng = oracle.n_groups_bound(m, E, R)
    rows_idx, group_expert = oracle.build_groups(row_expert, E, R, ng)
    seen = []
    for g in range(ng):
        e = group_expert[g]
        slots = rows_idx[g * R:(g + 1) * R]
        if e < 0:
            assert np.all(slots == m)
            continue
        real = slots[slots < m]
        assert np.all(row_expert[real] == e)
        assert np.all(np.diff(real) > 0)
        seen.extend(real.tolist())
    assert sorted(seen) == list(range(m))
    # experts appear in ascending order (stable sort by expert)
    ge = group_expert[group_expert >= 0]
    assert np.all(np.diff(ge) >= 0)

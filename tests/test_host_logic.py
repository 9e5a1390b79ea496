"""CPU: host-side logic of the coded-module layer -- policies, metadata guards,
scale folding.  Mirrors tests/test_dense_linear.py:176-249, :667-744 of the
reference; the guards fire before anything touches a device."""
from __future__ import annotations

import numpy as np
import pytest

from escha_mlx_b200 import dense, msl, synth


def _leaves(K=2, IC=128, OC=256, seed=1):
    rng = np.random.default_rng(seed)
    code, rin, rout = synth.coded_projection(rng, IC, OC, K)
    return code, rin, rout


def test_dense_block_r_policy():
    assert [msl.dense_block_r(m) for m in (1, 2, 3, 4, 7, 8, 15, 16, 17, 256)] == \
        [1, 2, 2, 4, 4, 8, 8, 16, 16, 16]
    assert msl.dense_block_r(5, pin=3) == 3
    assert msl.DENSE_R_MAX == 16


def test_code_to_u32_is_a_view_not_a_permutation():
    code = np.arange(64, dtype=np.int16).reshape(1, 1, 64) - 7
    u = msl.code_to_u32(code)
    assert u.shape == (1, 1, 32) and u.dtype == np.uint32
    lo = code.view(np.uint16)[..., 0::2].astype(np.uint32)
    hi = code.view(np.uint16)[..., 1::2].astype(np.uint32)
    assert np.array_equal(u, lo | (hi << 16))


def test_rejects_unsupported_rate():
    code, rin, rout = _leaves()
    bad = np.zeros((8, 16, 64), dtype=np.int16)  # 16*K with K=4
    with pytest.raises(ValueError, match="K=4"):
        dense.EschaWeight(bad, rin, rout)
    with pytest.raises(ValueError, match="16\\*K"):
        dense.EschaWeight(np.zeros((8, 16, 40), dtype=np.int16), rin, rout)


def test_rejects_mismatched_vectors_and_non_128_dims():
    code, rin, rout = _leaves()
    with pytest.raises(ValueError, match="do not match"):
        dense.EschaWeight(code, rin[:-1], rout)
    with pytest.raises(ValueError, match="do not match"):
        dense.EschaWeight(code, np.stack([rin, rin]), rout)   # E-stacked layout
    c16 = np.zeros((9, 16, 32), dtype=np.int16)               # IC = 144
    with pytest.raises(ValueError, match="multiples of 128"):
        dense.EschaWeight(c16, np.zeros(144, np.float16), rout)


def test_config_cross_check_and_codebook_gate():
    code, rin, rout = _leaves()
    with pytest.raises(ValueError, match="expected 6"):
        dense.EschaWeight(code, rin, rout, config=np.array([16, 2, 1, 1, 128]))
    with pytest.raises(ValueError, match="disagrees"):
        dense.EschaWeight(code, rin, rout, config=np.array([16, 3, 1, 1, 128, 256]))
    with pytest.raises(ValueError, match="codebook id 2"):
        dense.EschaWeight(code, rin, rout, config=np.array([16, 2, 1, 2, 128, 256]))


def test_scale_shape_guards():
    code, rin, rout = _leaves()
    with pytest.raises(ValueError, match="escha_s_in"):
        dense.EschaWeight(code, rin, rout, s_in=np.ones((2, 128), np.float32))
    with pytest.raises(ValueError, match="escha_s_out"):
        dense.EschaWeight(code, rin, rout, s_out=np.float32(1.0))


def test_build_requires_the_three_leaves():
    code, rin, rout = _leaves()
    with pytest.raises(ValueError, match="missing"):
        dense.build({"escha_code": code, "escha_rin": rin})
    assert dense.REQUIRED <= dense.LEAVES and "bias" in dense.LEAVES


def test_fold_scales_matches_reference_algebra():
    rng = np.random.default_rng(4)
    rin, rout = synth.signed_scale(rng, 128), synth.signed_scale(rng, 256)
    s_in = (rng.random(128) + 0.5).astype(np.float32)
    s_out = (rng.random(256) + 0.5).astype(np.float32)
    ri, ro = dense.fold_scales(rin, rout, s_in, s_out)
    assert np.array_equal(ri, rin.astype(np.float32) * s_in)
    assert np.array_equal(ro, rout.astype(np.float32) * s_out)
    ri2, ro2 = dense.fold_scales(rin, rout, None, None)
    assert np.array_equal(ri2, rin.astype(np.float32)) and ri2.dtype == np.float32


def test_bias_default_off(monkeypatch):
    monkeypatch.delenv("ESCHA_MLX_BIAS", raising=False)
    assert dense.apply_bias() is False
    monkeypatch.setenv("ESCHA_MLX_BIAS", "1")
    assert dense.apply_bias() is True
    monkeypatch.setenv("ESCHA_MLX_BIAS", "maybe")
    with pytest.raises(ValueError, match="ESCHA_MLX_BIAS"):
        dense.apply_bias()


def test_cpu_tensors_are_refused_not_silently_computed():
    """There is no CPU path: handing the kernel layer a CPU tensor is an error."""
    import torch
    x = torch.zeros((1, 128), dtype=torch.float16)
    rin = torch.ones(128, dtype=torch.float32)
    with pytest.raises(ValueError, match="CUDA tensors"):
        msl.dense_scaled_had(x, rin, msl.RS)


def test_synth_coded_bytes():
    assert synth.coded_bytes(4096, 4096, 2) == 4_194_304
    total = sum(synth.coded_bytes(ic, oc, k) for _, ic, oc, k in synth.DENSE_LAYER_27B)
    assert total == 117_309_440


def test_wave_splits_policy_is_shape_only(monkeypatch):
    """Launch-wide split factors on a 148-SM part (444 resident CTA slots): the fewest waves
    the launch fills to 85%, never fewer than two input blocks per split, same factor for
    every projection of the launch, and nothing but shapes goes in."""
    from escha_mlx_b200 import msl
    monkeypatch.setattr(msl, "sm_count", lambda: 148)
    # q/k/v/o of the 27B-class layer: 104 output blocks x 4 = 416 CTAs, one wave
    assert msl.wave_splits(5120, [6144, 1024, 1024, 5120]) == [4, 4, 4, 4]
    # gate/up: 272 blocks do not fill one wave to 85% at any factor; x 3 = 816 of 888 (two waves)
    assert msl.wave_splits(5120, [17408, 17408]) == [3, 3]
    # down: 40 blocks x 11 = 440 CTAs
    assert msl.wave_splits(17408, [5120]) == [11]
    # the 4096x4096 gate projection: 32 blocks x 13 = 416
    assert msl.wave_splits(4096, [4096]) == [13]
    # two input blocks per split at least: a 256-wide input is never split
    assert msl.wave_splits(256, [128]) == [1]
    # wider than eight waves at factor 1: stays unsplit
    assert msl.wave_splits(5120, [17408 * 16]) == [1]
    # row jobs multiply the block count: 8 x 57 = 456 blocks, x 5 = 2280 CTAs fill six waves to 86%
    assert msl.wave_splits(2048, [1024], njobs=57) == [5]

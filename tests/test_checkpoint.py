"""Checkpoint leaf ingestion: structural checks on CPU (no kernels run), and on the
GPU a round trip -- synthetic export written as .safetensors, streamed back, modules
built, outputs equal to modules built directly.  Mirrors the structural half of the
reference's tests/test_dense_checkpoint.py:55-165 and the loaders' error behaviour."""
from __future__ import annotations

import numpy as np
import pytest

from escha_mlx_b200 import synth


def _dense_export(rng, prefix="model.language_model."):
    t = {}
    for base, (ic, oc, k) in {"layers.0.self_attn.q_proj": (256, 384, 2),
                              "layers.0.mlp.down_proj": (384, 256, 3)}.items():
        code, rin, rout = synth.coded_projection(rng, ic, oc, k)
        t[f"{prefix}{base}.escha_code"] = code
        t[f"{prefix}{base}.escha_rin"] = rin
        t[f"{prefix}{base}.escha_rout"] = rout
        t[f"{prefix}{base}.escha_s_in"] = (rng.random(ic) + 0.5).astype(np.float32)
        t[f"{prefix}{base}.escha_s_out"] = (rng.random(oc) + 0.5).astype(np.float32)
        t[f"{prefix}{base}.escha_config"] = np.array([16, k, 2, 1, ic, oc], np.int32)
    w8, sc = synth.int8_linear(rng, 512, 256)
    t["lm_head.weight_int8"], t["lm_head.weight_scale"] = w8, sc
    w8, sc = synth.int8_linear(rng, 512, 256)
    t[f"{prefix}embed_tokens.weight_int8"], t[f"{prefix}embed_tokens.weight_scale"] = w8, sc
    t[f"{prefix}layers.0.input_layernorm.weight"] = np.ones(256, np.float16)
    t["mtp.layers.0.whatever"] = np.zeros(4, np.float16)
    return t


def test_check_structure_accepts_and_rejects():
    from escha_mlx_b200 import checkpoint
    rng = np.random.default_rng(0)
    t = {checkpoint.strip_lm_prefix(k): v for k, v in _dense_export(rng).items()}
    shapes = {k: list(v.shape) for k, v in t.items()}
    meta = {"layers.0.self_attn.q_proj": {"K": 2, "in_features": 256, "out_features": 384},
            "layers.0.mlp.down_proj": {"K": 3, "in_features": 384, "out_features": 256}}
    checkpoint.check_structure(shapes, meta)
    bad = dict(shapes)
    del bad["layers.0.mlp.down_proj.escha_rout"]
    with pytest.raises(ValueError, match="missing leaves"):
        checkpoint.check_structure(bad)
    bad = dict(shapes)
    bad["layers.0.self_attn.q_proj.escha_rin"] = [128]
    with pytest.raises(ValueError, match="transform vectors"):
        checkpoint.check_structure(bad)
    wrong = {k: dict(v) for k, v in meta.items()}
    wrong["layers.0.self_attn.q_proj"]["K"] = 3
    with pytest.raises(ValueError, match="disagrees with the code stream"):
        checkpoint.check_structure(shapes, wrong)
    with pytest.raises(ValueError, match="no coded linears"):
        checkpoint.check_structure({"a.weight": [4]})


def test_consume_rejects_unknown_and_incomplete():
    from escha_mlx_b200 import checkpoint
    ld = checkpoint.CheckpointLoader()
    with pytest.raises(ValueError, match="unknown escha tensor 'escha_learned_rot'"):
        ld.consume("model.language_model.layers.0.mlp.up_proj.escha_learned_rot", np.zeros(4))
    ld.consume("model.language_model.layers.0.mlp.up_proj.escha_code", np.zeros((8, 8, 32), np.int16))
    with pytest.raises(ValueError, match="incomplete escha linear"):
        ld.finalize()
    ld = checkpoint.CheckpointLoader()
    ld.consume("lm_head.weight_int8", np.zeros((16, 16), np.int8))
    with pytest.raises(ValueError, match="incomplete int8 tensor pairs"):
        ld.finalize()
    ld = checkpoint.CheckpointLoader()
    ld.consume("visual.blocks.0.w", np.zeros(4))
    ld.consume("mtp.fc.weight", np.zeros(4))
    ld.consume("model.language_model.norm.weight", np.ones(4))
    assert ld.dropped == 2 and list(ld.remainder) == ["model.language_model.norm.weight"]


@pytest.mark.gpu
def test_safetensors_round_trip_builds_equal_modules(cuda, tmp_path):
    import torch
    from safetensors.numpy import save_file
    from escha_mlx_b200 import checkpoint, dense, moe, quant
    from escha_mlx_b200.models.qwen3_5_moe import EschaSparseMoeBlock
    rng = np.random.default_rng(1)
    t = _dense_export(rng)
    E, H, I, top_k = 8, 256, 128, 2
    w = synth.moe_weights(rng, E, H, I, 2, 3)
    pre = "model.language_model.layers.1.mlp."
    for proj, key in (("gate_up_proj", "gu"), ("down_proj", "dn")):
        for leaf in ("code", "rin", "rout"):
            t[f"{pre}experts.{proj}.escha_{leaf}"] = w[f"{key}_{leaf}"]
        t[f"{pre}experts.{proj}.escha_config"] = np.zeros(6, np.int32)      # dropped for experts
    for p in ("gate", "up", "down"):
        t[f"{pre}shared_expert.{p}_proj.weight_int8"] = w[f"sh_{p}_w8"]
        t[f"{pre}shared_expert.{p}_proj.weight_scale"] = w[f"sh_{p}_scale"]
    t[f"{pre}gate.weight"] = w["gate_w"]
    t[f"{pre}shared_expert_gate.weight"] = w["shg_w"]
    path = str(tmp_path / "model.safetensors")
    save_file({k: np.ascontiguousarray(v) for k, v in t.items()}, path)

    ld = checkpoint.CheckpointLoader(num_experts=E, top_k=top_k, hidden_size=H, device=cuda)
    for name, arr in checkpoint.stream_safetensors(path):
        ld.consume(name, arr)
    mods = ld.finalize()
    assert (ld.n_coded, ld.n_q8, ld.n_moe) == (2, 2, 1) and ld.dropped == 3
    assert set(mods) == {"layers.0.self_attn.q_proj", "layers.0.mlp.down_proj", "lm_head",
                         "embed_tokens", "layers.1.mlp"}
    assert isinstance(mods["lm_head"], quant.EschaQ8Head)
    assert isinstance(mods["embed_tokens"], quant.EschaQ8Embedding)
    assert isinstance(mods["layers.1.mlp"], EschaSparseMoeBlock)

    p = "model.language_model.layers.0.self_attn.q_proj."
    direct = dense.build({leaf: t[p + leaf] for leaf in ("escha_code", "escha_rin", "escha_rout",
                                                         "escha_s_in", "escha_s_out", "escha_config")},
                         device=cuda)
    x = torch.from_numpy(synth.activations(rng, 3, 256)).to(cuda)
    assert torch.equal(mods["layers.0.self_attn.q_proj"](x), direct(x))
    shared = {k[3:]: v for k, v in w.items() if k.startswith("sh_")}
    blk = EschaSparseMoeBlock(H, E, top_k,
                              moe.EschaExperts(w["gu_code"], w["gu_rin"], w["gu_rout"], device=cuda),
                              moe.EschaExperts(w["dn_code"], w["dn_rin"], w["dn_rout"], device=cuda),
                              w["gate_w"], w["shg_w"], shared)
    xm = torch.from_numpy(synth.activations(rng, 5, H)).to(cuda)
    assert torch.equal(mods["layers.1.mlp"](xm), blk(xm))

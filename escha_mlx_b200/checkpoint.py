"""Checkpoint leaf ingestion for the coded-projection path.

Counterpart of ``CheckpointLoader.consume`` / ``finalize`` in the reference's
``escha_mlx/models/qwen3_5.py:248-361`` (dense) and
``escha_mlx/models/qwen3_5_moe.py:322-406`` (MoE).  The reference installs what it
builds into an mlx-lm model skeleton; that skeleton (attention, norms, caches) is not
part of this path, so here the loader returns the built modules keyed by their
checkpoint path and leaves everything it does not own (fp16 norms, convolutions ...)
in ``remainder`` for the caller:

    loader = CheckpointLoader(num_experts=256, top_k=8, hidden_size=2048, device="cuda")
    for name, array in tensors:          # e.g. stream_safetensors(path)
        loader.consume(name, array)
    modules = loader.finalize()          # {"layers.0.self_attn.q_proj": EschaLinear, ...,
                                         #  "layers.0.mlp": EschaSparseMoeBlock, "lm_head": ...}

Tensor names, leaf names, dtypes and the structural checks are the export's
(``escha_code`` int16 [TK, TN, 16K] or [E, TK, TN, 16K], ``escha_rin`` / ``escha_rout``
f16, ``escha_s_in`` / ``escha_s_out`` f32, ``escha_config`` i32, ``bias`` f16,
``weight_int8`` / ``weight_scale``).  Mistakes raise ``ValueError`` with the offending
name -- never an assert, never a silently half-loaded model.
"""
from __future__ import annotations

from typing import Iterable, Iterator

import numpy as np

from . import dense, moe, quant
from .models.qwen3_5_moe import EschaSparseMoeBlock

_CODED_LEAVES = frozenset(leaf for leaf in dense.LEAVES if leaf.startswith("escha_"))
_EXPERT_DROP_LEAVES = frozenset({"escha_s_in", "escha_s_out", "escha_config"})
_LM_PREFIXES = ("model.language_model.", "language_model.model.", "language_model.", "model.")


def strip_lm_prefix(name: str) -> str:
    """Checkpoint names with the wrapper prefixes of the HF export removed
    (reference: escha_mlx/loader.py strip_lm_prefix)."""
    for prefix in _LM_PREFIXES:
        if name.startswith(prefix):
            return name[len(prefix):]
    return name


def stream_safetensors(path: str) -> Iterator[tuple[str, np.ndarray]]:
    """Yield (name, array) for every tensor of one .safetensors file, one at a time."""
    from safetensors import safe_open
    with safe_open(path, framework="np") as f:
        for name in f.keys():
            yield name, f.get_tensor(name)


class CheckpointLoader:
    """Builds the coded linears, int8 linears and MoE blocks of an escha export."""

    def __init__(self, num_experts: int | None = None, top_k: int | None = None,
                 hidden_size: int | None = None, group_size: int = quant.DEFAULT_GROUP,
                 device=None, expert_range: tuple[int, int] | None = None) -> None:
        self.num_experts, self.top_k, self.hidden_size = num_experts, top_k, hidden_size
        self.group_size, self.device, self.expert_range = group_size, device, expert_range
        self._coded: dict[str, dict] = {}
        self._bias: dict[str, tuple[str, np.ndarray]] = {}
        self._int8: dict[str, dict] = {}
        self._shared: dict[str, dict] = {}
        self._experts: dict[tuple[int, str], dict] = {}
        self._mlp_fp16: dict[tuple[int, str], np.ndarray] = {}
        self.modules: dict[str, object] = {}
        self.remainder: dict[str, np.ndarray] = {}
        self.n_coded = self.n_q8 = self.n_bias = self.n_moe = self.dropped = 0

    # ------------------------------------------------------------------ consume

    def consume(self, name: str, w: np.ndarray) -> None:
        if name.startswith("mtp.") or ".visual." in name or name.startswith("visual."):
            self.dropped += 1
            return
        s = strip_lm_prefix(name)
        parts = s.split(".")
        if ".mlp.experts." in s:
            if len(parts) < 6 or parts[0] != "layers":
                raise ValueError(f"{name}: unexpected expert tensor name")
            layer, proj, leaf = int(parts[1]), parts[4], parts[5]
            if leaf in _EXPERT_DROP_LEAVES:
                self.dropped += 1
                return
            if leaf not in ("escha_code", "escha_rin", "escha_rout"):
                raise ValueError(f"{name}: unknown expert tensor {leaf!r}")
            self._experts.setdefault((layer, proj), {})[leaf] = w
            return
        base, _, leaf = s.rpartition(".")
        if leaf in _CODED_LEAVES:
            self._coded.setdefault(base, {})[leaf] = w
            return
        if leaf.startswith("escha_"):
            raise ValueError(
                f"{name}: unknown escha tensor {leaf!r}. This export uses a format feature this "
                f"runtime does not implement (known leaves: {sorted(dense.LEAVES)}).")
        if leaf == "bias":
            self._bias[base] = (name, w)
            return
        if leaf in ("weight_int8", "weight_scale"):
            target = self._shared if ".shared_expert." in s else self._int8
            target.setdefault(base, {})[leaf] = w
            return
        if s.endswith(".mlp.gate.weight") or s.endswith(".mlp.shared_expert_gate.weight"):
            self._mlp_fp16[(int(parts[1]), parts[3])] = w
            return
        self.remainder[name] = w

    # ----------------------------------------------------------------- finalize

    def _build_q8(self, base: str, pair: dict):
        w8, scale = pair["weight_int8"], pair["weight_scale"]
        if base == "lm_head":
            return quant.make_head(w8, scale, self.group_size, self.device)
        if base == "embed_tokens":
            return quant.make_embedding(w8, scale, self.group_size, self.device)
        if base.startswith("layers."):
            return quant.make_linear(w8, scale, self.group_size, self.device)
        raise ValueError(f"unexpected int8 tensor: {base}")

    def finalize(self) -> dict[str, object]:
        # ---- int8 linears, head, embedding
        for store in (self._int8, self._shared):
            bad = {k: sorted(v) for k, v in store.items() if len(v) != 2}
            if bad:
                raise ValueError(f"incomplete int8 tensor pairs: {bad}")
        for base in sorted(self._int8):
            self.modules[base] = self._build_q8(base, self._int8[base])
            self.n_q8 += 1
        self._int8.clear()

        # ---- coded dense linears
        for base in sorted(self._coded):
            group = self._coded[base]
            missing = dense.REQUIRED - set(group)
            if missing:
                raise ValueError(f"{base}: incomplete escha linear, missing {sorted(missing)}")
            if not base.startswith("layers."):
                raise ValueError(f"coded linear outside the decoder stack: {base}")
            held = self._bias.pop(base, None)
            if held is not None:
                group["bias"] = held[1]
                self.n_bias += 1
            self.modules[base] = dense.build(group, device=self.device)
            self.n_coded += 1
        self._coded.clear()
        for orig, w in self._bias.values():     # a bias nobody claimed is an ordinary tensor
            self.remainder[orig] = w
        self._bias.clear()

        # ---- MoE blocks
        layers = sorted({layer for layer, _ in self._experts})
        for i in layers:
            groups = {}
            for proj in ("gate_up_proj", "down_proj"):
                g = self._experts.pop((i, proj), None)
                if g is None or set(g) != {"escha_code", "escha_rin", "escha_rout"}:
                    raise ValueError(f"layers.{i}.mlp.experts.{proj}: incomplete expert stack "
                                     f"({sorted(g) if g else 'absent'})")
                groups[proj] = g
            if self.num_experts is None or self.top_k is None or self.hidden_size is None:
                raise ValueError("an MoE checkpoint needs num_experts, top_k and hidden_size")
            lo, hi = self.expert_range or (0, self.num_experts)

            def stack(g):
                return moe.EschaExperts(g["escha_code"][lo:hi], g["escha_rin"][lo:hi],
                                        g["escha_rout"][lo:hi], device=self.device)
            gu, dn = stack(groups["gate_up_proj"]), stack(groups["down_proj"])
            shared = {}
            for p in ("gate", "up", "down"):
                pair = self._shared.pop(f"layers.{i}.mlp.shared_expert.{p}_proj", None)
                if pair is None:
                    raise ValueError(f"layers.{i}.mlp.shared_expert.{p}_proj: int8 pair missing")
                shared[f"{p}_w8"], shared[f"{p}_scale"] = pair["weight_int8"], pair["weight_scale"]
            try:
                gate_w = self._mlp_fp16.pop((i, "gate"))
                shg_w = self._mlp_fp16.pop((i, "shared_expert_gate"))
            except KeyError as e:
                raise ValueError(f"layers.{i}.mlp: router tensor {e.args[0][1]!r} missing") from None
            self.modules[f"layers.{i}.mlp"] = EschaSparseMoeBlock(
                self.hidden_size, self.num_experts, self.top_k, gu, dn, gate_w, shg_w, shared,
                self.group_size, expert_range=self.expert_range)
            self.n_moe += 1
        if self._experts:
            raise ValueError(f"unconsumed expert tensors: {sorted(self._experts)[:4]}")
        if self._shared:
            raise ValueError(f"shared-expert tensors without an MoE layer: {sorted(self._shared)[:4]}")
        return self.modules


def check_structure(tensor_shapes: dict[str, list[int]], layer_meta: dict | None = None) -> None:
    """The structural checks the reference runs against a real export
    (tests/test_dense_checkpoint.py:63-118), on a {name: shape} map such as a
    safetensors header: every coded linear has its full leaf set, both dimensions are
    multiples of 128 with matching transform vectors, and -- given the export's
    ``quantization_config.layer_meta`` -- the declared rate and shape of every linear
    agree with its code stream."""
    bases = {n.rsplit(".", 1)[0] for n in tensor_shapes if n.endswith(".escha_code")}
    if not bases:
        raise ValueError("no coded linears found")
    for b in sorted(bases):
        missing = [leaf for leaf in sorted(dense.REQUIRED) if f"{b}.{leaf}" not in tensor_shapes]
        if missing:
            raise ValueError(f"{b}: missing leaves {missing}")
        shape = list(tensor_shapes[f"{b}.escha_code"])
        lead, (tk, tn, wpt) = shape[:-3], shape[-3:]
        if wpt % 16:
            raise ValueError(f"{b}: code last dim {wpt} is not 16*K")
        ic, oc = tk * 16, tn * 16
        if ic % 128 or oc % 128:
            raise ValueError(f"{b}: {ic}x{oc} is not a multiple of 128 in both dimensions")
        if (list(tensor_shapes[f"{b}.escha_rin"]) != lead + [ic]
                or list(tensor_shapes[f"{b}.escha_rout"]) != lead + [oc]):
            raise ValueError(f"{b}: transform vectors do not match the code stream's {ic}x{oc}")
    if layer_meta is not None:
        for base, m in layer_meta.items():
            shape = tensor_shapes.get(f"{base}.escha_code")
            if shape is None:
                raise ValueError(f"layer_meta names {base} but it has no code")
            tk, tn, wpt = list(shape)[-3:]
            if wpt // 16 != m["K"] or (tk * 16, tn * 16) != (m["in_features"], m["out_features"]):
                raise ValueError(f"{base}: layer_meta {m} disagrees with the code stream "
                                 f"(K={wpt // 16}, {tk * 16}x{tn * 16})")
        if len(layer_meta) != len(bases):
            raise ValueError(f"layer_meta lists {len(layer_meta)} linears, the export holds {len(bases)}")

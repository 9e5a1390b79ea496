"""Synthetic, device-resident layer stacks with the shapes of the published
benchmark configurations (random code bits, |N(0, 0.02)| + 1e-3 scales with random
signs, random int8 weights): there are no checkpoints here, and a random code
stream decodes with exactly the same instruction and byte counts as a trained one.

* ``MoeLayer`` -- one 35B-A3B-class MoE decode layer: 256 routed 2-bit experts
  (gate_up 2048 -> 1024, down 512 -> 2048), top-8 softmax routing, one int8 shared
  expert, optionally preceded by the int8 attention projections of the full
  decode step (16 query heads, 2 key/value heads, head size 256).
* ``moe_stack`` -- several such layers with distinct weights, so that a pass over
  the stack never finds a layer's bytes in L2.
"""
from __future__ import annotations

import numpy as np
import torch

from . import moe, quant
from .models.qwen3_5_moe import EschaSparseMoeBlock

MOE_35B = dict(hidden=2048, inter=512, experts=256, top_k=8, K_gate_up=2, K_down=2,
               q_heads=16, kv_heads=2, head_dim=256)


def _signed_scale(shape, device, gen) -> torch.Tensor:
    scale = torch.randn(shape, device=device, generator=gen).abs() * 0.02 + 1e-3
    sign = torch.randint(0, 2, shape, device=device, generator=gen).float() * 2 - 1
    return (scale * sign).half().float()      # f16-representable, held as f32


def _experts(E, ic, oc, k, device, gen) -> moe.EschaExperts:
    code = torch.randint(-2**31, 2**31 - 1, (E, ic // 16, oc // 16, 8 * k), dtype=torch.int32,
                         device=device, generator=gen)
    return moe.EschaExperts(code, _signed_scale((E, ic), device, gen),
                            _signed_scale((E, oc), device, gen))


def _q8(n, kd, device, gen) -> quant.EschaQ8Linear:
    w8 = torch.randint(-127, 128, (n, kd), dtype=torch.int8, device=device, generator=gen)
    # uniform int8 has rms ~73: scales near 1 / (73 sqrt(kd)) keep the output at the
    # input's magnitude, so activations stay in range through a stack of layers
    scale = ((torch.rand((n,), device=device, generator=gen) + 0.5) / (73.0 * kd ** 0.5)).half()
    return quant.EschaQ8Linear(w8, scale)


class MoeLayer(torch.nn.Module):
    """One decode layer's projections on this path: [int8 q/k/v/o] + the MoE block.

    Attention itself (scores, cache) is not part of the coded-projection path; the
    o projection consumes the q projection's output so that the four int8 linears
    run with their real shapes and dependencies.
    """

    def __init__(self, device, gen, cfg=MOE_35B, attention: bool = False,
                 expert_range: tuple[int, int] | None = None, gen_experts=None,
                 peer_group=None) -> None:
        """``gen`` draws everything every rank replicates (router, shared expert, int8
        projections) and must be seeded alike on all ranks; ``gen_experts`` draws this
        rank's expert shard."""
        super().__init__()
        H, I, E = cfg["hidden"], cfg["inter"], cfg["experts"]
        lo, hi = expert_range or (0, E)
        self._e_lo, self._e_hi = lo, hi
        ge = gen_experts or gen
        gu = _experts(hi - lo, H, 2 * I, cfg["K_gate_up"], device, ge)
        dn = _experts(hi - lo, I, H, cfg["K_down"], device, ge)
        cpu = np.random.default_rng(int(torch.randint(0, 2**31 - 1, (1,), device=device,
                                                      generator=gen).item()))
        gate_w = (cpu.standard_normal((E, H)) * 0.5).astype(np.float16)
        shg_w = (cpu.standard_normal((H,)) * 0.05).astype(np.float16)
        shared = {}
        for name, (n, kd) in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I))):
            lin = _q8(n, kd, device, gen)
            shared[f"{name}_w8"], shared[f"{name}_scale"] = lin._w8, lin._scale
        self.block = EschaSparseMoeBlock(H, E, cfg["top_k"], gu, dn, gate_w, shg_w, shared,
                                         expert_range=expert_range, peer_group=peer_group)
        self.attention = attention
        if attention:
            qd, kvd = cfg["q_heads"] * cfg["head_dim"], cfg["kv_heads"] * cfg["head_dim"]
            self.q, self.k, self.v = _q8(qd, H, device, gen), _q8(kvd, H, device, gen), \
                _q8(kvd, H, device, gen)
            self.o = _q8(H, qd, device, gen)
        self.expert_bytes = (H * 2 * I * cfg["K_gate_up"] + I * H * cfg["K_down"]) // 8
        self.int8_bytes = 3 * H * I + (2 * H * (qd + kvd) if attention else 0)
        self.router_bytes = 2 * E * H

    def _attention_projections(self, x: torch.Tensor) -> torch.Tensor:
        if not self.attention:
            return x
        q, _, _ = quant.project_many_q8([self.q, self.k, self.v], x)   # one launch, as one input
        return torch.add(x, self.o(q), alpha=0.01)   # residual keeps the scale bounded

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.block(self._attention_projections(x))

    def routed_experts(self, x: torch.Tensor) -> int:
        """Distinct experts of this rank's shard that the rows of ``x`` are routed to
        (host count, for byte accounting)."""
        xb = self._attention_projections(x)
        ids, _ = self.block.route(xb.reshape(-1, xb.shape[-1]).half())
        u = torch.unique(ids)
        return int(((u >= self._e_lo) & (u < self._e_hi)).sum().item())


def moe_stack(n_layers: int, device, seed: int = 1234, attention: bool = False,
              expert_range: tuple[int, int] | None = None, rank: int = 0,
              cfg=MOE_35B, peer_group=None) -> list[MoeLayer]:
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    gen_experts = torch.Generator(device=device)
    gen_experts.manual_seed(seed + 1 + rank)
    return [MoeLayer(device, gen, cfg, attention, expert_range, gen_experts, peer_group)
            for _ in range(n_layers)]

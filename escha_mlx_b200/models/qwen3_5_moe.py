"""The SwitchGLU-style MoE block of the qwen3_5_moe architecture, executing the
escha trellis-coded routed experts on B200.

Mirror of ``EschaSparseMoeBlock`` in the reference's
``escha_mlx/models/qwen3_5_moe.py:62-273`` (the checkpoint loader half of that
file belongs to the mlx-lm model skeleton and is not part of this path).

Routing convention: fp32 logits from the fp16 gate Linear (one f16 round), top-k,
softmax over the top-k values.  Each (token, slot) pair becomes one GEMV row;
rows are laid out token-major.  Expert forward per row:

    xh   = f16( H128(x * rin[e]) * RS )
    mid  = xh @ decode(code[e])                       (f32 accumulate)
    gu16 = f16( H128(mid) * RS * rout[e] )            -> f16(silu(g)) * u -> h
    xh2  = f16( H128(h * rin_dn[e]) * RS )
    d16  = f16( H128(xh2 @ decode_dn) * RS * rout_dn[e] )
    y[token] = sum over slots, in slot order, of f32(d16) * f32(f16(score))

plus the shared expert (int8 SwiGLU, sigmoid-gated).  The slot sum is a fixed
order reduction -- never a scatter-add -- so the block is bit-reproducible.

With ``torch.distributed`` initialised and ``expert_parallel=True`` the routed
experts are sharded over ranks (this rank holds ``gu``/``dn`` for experts
[e_lo, e_hi)); each rank computes the rows whose expert it owns, the f16 expert
outputs are all-gathered, and every rank runs the same combine, so the result is
bit-identical to one GPU.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F

from .. import envs, moe, msl, quant, sharding

MODEL_TYPE = "qwen3_5_moe"
RS = msl.RS


class EschaSparseMoeBlock(torch.nn.Module):
    """Drop-in MoE block: router, routed coded experts, shared int8 expert."""

    def __init__(self, hidden_size: int, num_experts: int, top_k: int,
                 gu: moe.EschaExperts, dn: moe.EschaExperts,
                 gate_w: np.ndarray, shg_w: np.ndarray, shared: dict,
                 group_size: int = quant.DEFAULT_GROUP,
                 expert_range: tuple[int, int] | None = None, peer_group=None) -> None:
        super().__init__()
        self.top_k = top_k
        self.num_experts = num_experts
        self._gu = gu
        self._dn = dn
        self._inter = gu.OC // 2
        dev = gu.code.device
        self._e_lo, self._e_hi = expert_range or (0, num_experts)
        if self._e_hi - self._e_lo != gu.E or gu.E != dn.E:
            raise ValueError(
                f"expert stacks hold {gu.E}/{dn.E} experts, the block expects "
                f"{self._e_hi - self._e_lo}")
        if gu.IC != hidden_size or dn.OC != hidden_size or dn.IC != self._inter:
            raise ValueError(
                f"expert shapes {gu.IC}x{gu.OC} / {dn.IC}x{dn.OC} do not form a "
                f"hidden={hidden_size} SwiGLU expert")
        self.gate_weight = torch.from_numpy(np.asarray(gate_w).astype(np.float16)).to(dev)
        self.shared_expert_gate_weight = torch.from_numpy(
            np.asarray(shg_w).astype(np.float16).reshape(1, hidden_size)).to(dev)
        self.sh_gate = quant.make_linear(shared["gate_w8"], shared["gate_scale"], group_size, dev)
        self.sh_up = quant.make_linear(shared["up_w8"], shared["up_scale"], group_size, dev)
        self.sh_down = quant.make_linear(shared["down_w8"], shared["down_scale"], group_size, dev)
        # gate and up of the shared expert as one [2I, H] matrix: one launch, merged output
        self._sh_gu_w8 = torch.cat([self.sh_gate._w8, self.sh_up._w8]).contiguous()
        self._sh_gu_scale = torch.cat([self.sh_gate._scale, self.sh_up._scale]).contiguous()
        # expert parallel over peer-mapped memory (peer.PeerGroup): the second expert leg
        # stores its rows into every GPU's buffer and one barrier kernel replaces the
        # all-gather.  Two buffers per row count, alternated call by call.
        self._side: torch.cuda.Stream | None = None
        self._peers = peer_group
        self._peer_bufs: dict[int, list] = {}
        self._peer_calls = 0
        self._mode = "fused"
        self._fused_had = msl.use_fused_had()
        self._block_env = envs.ESCHA_MLX_BLOCK_R.get()

    # -- expert path ------------------------------------------------------

    def _rows(self, xf: torch.Tensor, ids: torch.Tensor):
        """Token-major rows: row t*top_k+s is (token t, slot s)."""
        t = xf.shape[0]
        row_expert = ids.reshape(t * self.top_k).to(torch.int32)
        row_token = torch.arange(t, dtype=torch.int32, device=xf.device).repeat_interleave(self.top_k)
        return row_expert, row_token

    def _blocked_R(self, m: int) -> int:
        """Rows-per-group policy of the reference (:124-170), kept for callers
        that query it.  The tensor-core kernel needs no such policy: every
        expert's stream is read once and shared by all of its rows."""
        if self._block_env is not None:
            return self._block_env
        if m >= 2048:
            return 12
        if m >= 1024:
            return 4
        if m >= 320:
            return 3
        if m >= 128:
            return 2
        return 1

    def _gemv(self, xh: torch.Tensor, row_expert: torch.Tensor, ex: moe.EschaExperts,
              jobs: torch.Tensor | None = None) -> torch.Tensor:
        return msl.moe_gemv(xh, ex.code, row_expert, ex.K, ex.IC, ex.OC, jobs=jobs)

    def _leg(self, rows: torch.Tensor, row_expert: torch.Tensor, ex: moe.EschaExperts,
             jobs: torch.Tensor | None) -> torch.Tensor:
        """One coded projection over expert-indexed rows -> f16 [m, OC]."""
        xh = msl.scaled_had(rows, ex.rin, row_expert, RS)
        if msl.gemv_family() == "mma" and self._fused_had:
            out = torch.zeros((rows.shape[0], ex.OC), dtype=torch.float16, device=rows.device) \
                if self._sharded() else None
            return msl.coded_gemv_jobs(xh, ex.code, jobs, ex.rout, ex.K, ex.IC, ex.OC, ex.E,
                                       out=out)
        mid = self._gemv(xh, row_expert, ex, jobs)
        return msl.scaled_had_out(mid, ex.rout, row_expert, RS)

    def _sharded(self) -> bool:
        return (self._e_hi - self._e_lo) != self.num_experts

    def _expert_rows(self, xf: torch.Tensor, ids: torch.Tensor,
                     jobs: torch.Tensor | None = None, local_only: bool = False) -> torch.Tensor:
        """Expert outputs d16 [T*top_k, H] f16 for the (token, slot) rows, complete on
        every rank (under expert parallelism the owners' rows are all-gathered).
        ``jobs`` are the row jobs of this rank's experts when the router launch has
        already built them.  ``local_only`` (needs ``jobs``): return this rank's buffer
        as it is -- rows of other ranks' experts are left unwritten."""
        row_expert = ids.reshape(xf.shape[0] * self.top_k).to(torch.int32)
        m = row_expert.shape[0]
        owned = None
        job_expert = row_expert
        if self._sharded() and not local_only:
            # rows of experts another rank owns get no job here (expert -1 matches no
            # local expert); their output rows stay zero and are replaced by the
            # owner's rows in the ownership-selecting all-gather below
            owned = (row_expert >= self._e_lo) & (row_expert < self._e_hi)
            local = row_expert - self._e_lo
            job_expert = torch.where(owned, local, torch.full_like(local, -1))
            row_expert = torch.where(owned, local, torch.zeros_like(local))
        gu, dn = self._gu, self._dn
        if msl.gemv_family() == "mma" and self._fused_had:
            # two launches: each leg's input transform (with the token gather, resp.
            # the SwiGLU), product and output transform in one kernel
            if jobs is None:
                jobs = msl.group_rows(job_expert, gu.E)
            zeros = (lambda oc: [torch.zeros((m, oc), dtype=torch.float16, device=xf.device)]) \
                if owned is not None else (lambda oc: None)
            gu16 = msl.coded_projections(xf, [gu.code], [gu.rin], [gu.rout], gu.K, gu.IC, [gu.OC],
                                         input_mode=msl.INPUT_RAW, jobs=jobs, E=gu.E, rows=m,
                                         x_stride=gu.IC, x_row_div=self.top_k,
                                         outs=zeros(gu.OC))[0]
            inter = self._inter
            d16 = msl.coded_projections(gu16[:, :inter], [dn.code], [dn.rin], [dn.rout], dn.K,
                                        dn.IC, [dn.OC], input_mode=msl.INPUT_SWIGLU,
                                        x_up=gu16[:, inter:], jobs=jobs, E=dn.E, rows=m,
                                        x_stride=2 * inter, outs=zeros(dn.OC))[0]
        else:
            jobs = msl.group_rows(job_expert, gu.E) if msl.gemv_family() == "mma" else None
            _, row_token = self._rows(xf, ids)
            rows = xf[row_token.long()]
            gu16 = self._leg(rows, row_expert, gu, jobs)
            h = msl.swiglu(gu16)
            d16 = self._leg(h, row_expert, dn, jobs)
        if owned is not None:
            d16 = sharding.all_gather_rows_by_owner(d16, owned)
        return d16

    def _expert_rows_to_peers(self, xf: torch.Tensor, jobs: torch.Tensor) -> torch.Tensor:
        """Both expert legs for this rank's jobs; the second leg's epilogue stores each
        output row into every GPU's [T*top_k, H] buffer, then the ranks meet in the peer
        barrier.  Returns the local buffer, complete.

        A buffer is rewritten two calls later; between the two, every rank must have
        passed a later barrier (the next call's, or another layer's in the same graph).
        A CUDA graph that holds a single call of a single block and is replayed back to
        back does not satisfy this: capture at least two calls or two layers."""
        gu, dn, inter = self._gu, self._dn, self._inter
        m = xf.shape[0] * self.top_k
        bufs = self._peer_bufs.get(m)
        if bufs is None:
            bufs = [self._peers.empty((m, dn.OC), torch.float16) for _ in range(2)]
            self._peer_bufs[m] = bufs
        buf = bufs[self._peer_calls % 2]
        self._peer_calls += 1
        gu16 = msl.coded_projections(xf, [gu.code], [gu.rin], [gu.rout], gu.K, gu.IC, [gu.OC],
                                     input_mode=msl.INPUT_RAW, jobs=jobs, E=gu.E, rows=m,
                                     x_stride=gu.IC, x_row_div=self.top_k)[0]
        d16 = msl.coded_projections(gu16[:, :inter], [dn.code], [dn.rin], [dn.rout], dn.K, dn.IC,
                                    [dn.OC], input_mode=msl.INPUT_SWIGLU, x_up=gu16[:, inter:],
                                    jobs=jobs, E=dn.E, rows=m, x_stride=2 * inter,
                                    gather=[(buf, 0)])[0]
        self._peers.barrier()
        return d16

    def _expert_path(self, xf: torch.Tensor, ids: torch.Tensor, scores: torch.Tensor) -> torch.Tensor:
        t = xf.shape[0]
        d16 = self._expert_rows(xf, ids)
        y16 = msl.moe_combine(d16, scores.reshape(t * self.top_k).to(torch.float32).contiguous(),
                              t, self.top_k)
        # the routed-expert sum is rounded to f16 before the shared expert is added
        return y16.float()

    # -- block forward ----------------------------------------------------

    def route(self, xf: torch.Tensor):
        logits = F.linear(xf, self.gate_weight).float()
        top, ids = torch.topk(logits, self.top_k, dim=-1)
        scores = torch.softmax(top, dim=-1)
        return ids, scores

    def _single_pass(self) -> bool:
        """Whether the block runs as router -> two expert legs -> shared gate/up ->
        tail (six launches) instead of the op-by-op composition."""
        return (msl.gemv_family() == "mma" and self._fused_had
                and self.num_experts <= msl.ROUTE_MAX_EXPERTS and self.top_k <= msl.ROUTE_MAX_TOP_K
                and self._sh_gu_w8.shape[1] % 64 == 0 and self.sh_down.in_features % 64 == 0
                and self.sh_down.out_features % 16 == 0 and self._sh_gu_w8.shape[0] % 16 == 0)

    def forward(self, x: torch.Tensor, ids: torch.Tensor | None = None,
                scores: torch.Tensor | None = None) -> torch.Tensor:
        shape = x.shape
        hdim = shape[-1]
        xf = x.reshape(-1, hdim).to(torch.float16).contiguous()
        if self._single_pass():
            t = xf.shape[0]
            # the shared expert's gate/up linear depends on nothing but x: it runs on a
            # second stream beside the router and the expert legs (a fork/join that a
            # CUDA-graph capture records as parallel branches)
            main = torch.cuda.current_stream()
            if self._side is None:
                self._side = torch.cuda.Stream()
            self._side.wait_stream(main)
            with torch.cuda.stream(self._side):
                gu_sh = quant.w8a16(xf, self._sh_gu_w8, self._sh_gu_scale)
            gu_sh.record_stream(main)
            ids_r, scores_r, slog, jobs = msl.moe_route(
                xf, self.gate_weight, self.shared_expert_gate_weight.reshape(-1), self.top_k,
                self.num_experts, ids=ids, expert_range=(self._e_lo, self._e_hi))
            if ids is None:
                scores = scores_r
            sc = scores.reshape(t * self.top_k).to(torch.float32).contiguous()
            if self._sharded() and self._peers is not None:
                # expert rows land in every GPU's buffer straight from the kernel epilogue
                d16 = self._expert_rows_to_peers(xf, jobs)
                main.wait_stream(self._side)
                out = msl.moe_shared_finish(gu_sh, self.sh_down._w8, self.sh_down._scale, d16, sc,
                                            slog, self.top_k)
            elif self._sharded():
                # one collective per block: every rank's buffer side by side; the tail
                # picks each row from the rank that owns its expert
                d16 = sharding.all_gather_rows(self._expert_rows(xf, ids_r, jobs, local_only=True))
                main.wait_stream(self._side)
                out = msl.moe_shared_finish(
                    gu_sh, self.sh_down._w8, self.sh_down._scale, d16, sc, slog, self.top_k,
                    ids=ids_r.reshape(-1).to(torch.int32).contiguous(),
                    experts_per_rank=self._e_hi - self._e_lo)
            else:
                d16 = self._expert_rows(xf, ids_r, jobs)
                main.wait_stream(self._side)
                out = msl.moe_shared_finish(gu_sh, self.sh_down._w8, self.sh_down._scale, d16, sc,
                                            slog, self.top_k)
            return out.to(x.dtype).reshape(shape)
        if ids is None:
            ids, scores = self.route(xf)
        y = self._expert_path(xf, ids, scores)

        g = self.sh_gate(xf).float()
        u = self.sh_up(xf).float()
        hh = ((g * torch.sigmoid(g)) * u).to(torch.float16)
        sh = self.sh_down(hh).float()
        sgate = torch.sigmoid(F.linear(xf, self.shared_expert_gate_weight).float())
        out = (y + sh * sgate).to(x.dtype)
        return out.reshape(shape)

"""Dense coded linears: one trellis-coded weight stream per projection.

Mirror of the reference's ``escha_mlx/dense.py`` (``EschaWeight`` :158-265,
``EschaLinear`` :268-362, ``project_pair`` :365-437, ``build`` :440-452,
``pack_code`` :145-155, ``coded_bytes`` :455-483) over CUDA ``torch.Tensor``s.
The forward contract is the reference's, rounding points included:

    xh  = f16( H128(x_f32 * rin_f32) * RS )
    mid = xh_f32 @ W_f32                      (W = decoded fp16 tiles, f32 accumulate)
    y   = f16( H128(mid) * RS * rout_f32 )    [+ f16(f32(y) + f32(bias)) if enabled]

There is no NumPy "ops" path here: every forward runs the CUDA kernels, and a
missing GPU or library is an error, not a fallback.
"""
from __future__ import annotations

import logging

import numpy as np
import torch

from . import envs, msl

logger = logging.getLogger(__name__)

RS = msl.RS

#: Rates the codec implements; anything else is refused at load (reference :66-68).
SUPPORTED_K = frozenset({2, 3})

#: escha_config layout: [L, K, V, codebook_id, in_features, out_features].
_CONFIG_LEN = 6
_PRODUCTION_CODEBOOK = 1


def _check_scale(name: str, vec, expect: int) -> None:
    """A scale vector must be 1-D of exactly ``expect`` entries, or absent."""
    if vec is None:
        return
    shape = tuple(np.shape(vec))
    if shape != (expect,):
        raise ValueError(f"{name} must have shape ({expect},), got {shape}")


def fold_scales(rin, rout, s_in=None, s_out=None):
    """rin_eff = f32(rin) * f32(s_in), rout_eff = f32(rout) * f32(s_out)
    (reference: escha_mlx/ref.py:242-277).  None leaves that vector unchanged."""
    ri = np.asarray(rin).astype(np.float32)
    ro = np.asarray(rout).astype(np.float32)
    if s_in is not None:
        ri = ri * np.asarray(s_in).astype(np.float32)
    if s_out is not None:
        ro = ro * np.asarray(s_out).astype(np.float32)
    return ri, ro


def apply_bias() -> bool:
    """Whether to apply the per-linear correction a dense export ships.  Default
    NO, as in the reference (:107-132): the published numbers for those
    checkpoints were produced without it; ESCHA_MLX_BIAS=1 applies it."""
    return bool(envs.ESCHA_MLX_BIAS.get())


def linear_mode() -> str:
    """Always ``fused``: the CUDA kernels are the only execution path."""
    return "fused"


def pack_code(code_i16: np.ndarray, device=None) -> torch.Tensor:
    """int16 [TK, TN, 16K] -> 32-bit words [TK, TN, 8K] on the device (:145-155)."""
    return msl.code_tensor(code_i16, device)


class _StreamGeometry:
    """What a code array's shape says about the linear: rate, input and output width."""

    def __init__(self, K: int, IC: int, OC: int) -> None:
        self.K, self.IC, self.OC = K, IC, OC

    @classmethod
    def of(cls, shape: tuple, packed: bool) -> "_StreamGeometry":
        if len(shape) != 3:
            raise ValueError(f"escha code must be [TK, TN, words per tile], got shape {shape}")
        words = 8 if packed else 16          # 32-bit or 16-bit words per tile and bit of rate
        if shape[2] % words:
            raise ValueError(f"{'packed ' if packed else ''}escha code last dim must be "
                             f"{words}*K, got {shape[2]}")
        return cls(shape[2] // words, shape[0] * 16, shape[1] * 16)

    def require(self, rin, rout, s_in, s_out, config) -> None:
        """Raise ValueError for the first contract violation, in the order the reference
        checks them: rate, vector shapes, alignment, the export's config record, scales."""
        shapes = (tuple(np.shape(rin)), tuple(np.shape(rout)))
        problems = (
            (self.K not in SUPPORTED_K,
             f"escha code implies K={self.K}; this runtime implements K in {sorted(SUPPORTED_K)}"),
            (shapes != ((self.IC,), (self.OC,)),
             f"transform vectors {shapes[0]}/{shapes[1]} do not match the code stream's "
             f"{self.IC}x{self.OC}; both must be 1-D ({self.IC},)/({self.OC},)"),
            (self.IC % 128 != 0 or self.OC % 128 != 0,
             f"escha linear dimensions must be multiples of 128, got {self.IC}x{self.OC}"),
        )
        for bad, message in problems:
            if bad:
                raise ValueError(message)
        if config is not None:
            self._require_config([int(v) for v in np.asarray(config).ravel()])
        _check_scale("escha_s_in", s_in, self.IC)
        _check_scale("escha_s_out", s_out, self.OC)

    def _require_config(self, record: list) -> None:
        if len(record) != _CONFIG_LEN:
            raise ValueError(
                f"escha_config has {len(record)} fields, expected {_CONFIG_LEN} ([L, K, V, "
                f"codebook_id, in_features, out_features]); this export was written by an "
                f"incompatible version")
        claimed = (record[1], record[4], record[5])
        if claimed != (self.K, self.IC, self.OC):
            raise ValueError(f"escha_config {claimed} disagrees with the code stream "
                             f"{(self.K, self.IC, self.OC)}")
        if record[3] != _PRODUCTION_CODEBOOK:
            raise ValueError(
                f"escha_config selects codebook id {record[3]}; this runtime implements the "
                f"production codebook (id {_PRODUCTION_CODEBOOK}) only")


class EschaWeight:
    """One dense linear's coded stream plus its folded transform vectors.

    Kept off the module parameter tree (the owner holds it under a
    leading-underscore attribute); ``arrays()`` enumerates its device tensors.
    """

    def __init__(self, code, rin, rout, s_in=None, s_out=None, config=None, device=None) -> None:
        """``code`` is the export's int16 [TK, TN, 16K] array or an already packed device
        tensor [TK, TN, 8K] of 32-bit words; ``rin``/``rout`` are the folded sign*scale
        vectors, ``s_in``/``s_out`` optional extra scales, ``config`` the export's
        [L, K, V, codebook, IC, OC] record.  Refuses what the reference's constructor
        refuses (escha_mlx/dense.py:168-242), before anything reaches a kernel."""
        packed = isinstance(code, torch.Tensor)
        geo = _StreamGeometry.of(tuple(code.shape) if packed else tuple(np.shape(code)), packed)
        geo.require(rin, rout, s_in, s_out, config)
        self.K, self.IC, self.OC = geo.K, geo.IC, geo.OC
        self.code = code if packed else pack_code(code, device)   # [TK, TN, 8K] 32-bit words
        ri, ro = fold_scales(_to_numpy(rin), _to_numpy(rout), _to_numpy(s_in), _to_numpy(s_out))
        self.rin = torch.from_numpy(ri).to(self.code.device)      # [IC] f32
        self.rout = torch.from_numpy(ro).to(self.code.device)     # [OC] f32

    @classmethod
    def from_device(cls, code: torch.Tensor, rin: torch.Tensor, rout: torch.Tensor) -> "EschaWeight":
        """A weight whose packed stream and already folded f32 vectors live on the device
        (synthetic workloads, weights produced by another stage).  Same refusals as the
        constructor; nothing is copied."""
        geo = _StreamGeometry.of(tuple(code.shape), True)
        geo.require(rin, rout, None, None, None)
        for name, v in (("rin", rin), ("rout", rout)):
            if v.dtype != torch.float32 or v.device != code.device or not v.is_contiguous():
                raise ValueError(f"{name} must be a contiguous float32 tensor on the code's device")
        w = cls.__new__(cls)
        w.K, w.IC, w.OC = geo.K, geo.IC, geo.OC
        w.code, w.rin, w.rout = code.contiguous(), rin, rout
        return w

    def weight_numpy(self) -> np.ndarray:
        """Decoded bare weight [IC, OC] as f32 (debug/inspection; decoded on the GPU)."""
        return msl.decode_tiles(self.code, self.K, self.IC, self.OC).float().cpu().numpy()

    def arrays(self) -> list[torch.Tensor]:
        return [self.code, self.rin, self.rout]

    def shard_out(self, index: int, count: int) -> "EschaWeight":
        """Split-N shard: output channels [index*OC/count, (index+1)*OC/count), whole
        128-channel blocks.  Decode tiles, GEMV columns and the output transform
        are block-local, so a shard's output equals the matching slice of the
        full linear bit for bit."""
        blocks = self.OC // 128
        if blocks % count:
            raise ValueError(f"{blocks} output blocks do not split {count} ways")
        per = self.OC // count
        tn0, tn1 = index * per // 16, (index + 1) * per // 16
        w = object.__new__(EschaWeight)
        w.K, w.IC, w.OC = self.K, self.IC, per
        w.code = self.code[:, tn0:tn1, :].contiguous()
        w.rin = self.rin
        w.rout = self.rout[index * per:(index + 1) * per].contiguous()
        return w


def _to_numpy(v):
    if v is None:
        return None
    if isinstance(v, torch.Tensor):
        return v.detach().cpu().numpy()
    return np.asarray(v)


class EschaLinear(torch.nn.Module):
    """A trellis-coded dense linear.  Drop-in for ``nn.Linear`` (bias folded in)."""

    def __init__(self, w: EschaWeight, bias: np.ndarray | None = None) -> None:
        super().__init__()
        self._w = w
        self.bias = None if bias is None else torch.from_numpy(
            np.asarray(bias).astype(np.float16)).to(w.code.device)
        self._mode = linear_mode()
        # latched at construction so a forward is self-consistent (reference :278-281)
        self._fused_had = msl.use_fused_had()
        self._block_r_pin = msl.dense_block_r_pin()

    @property
    def K(self) -> int:
        return self._w.K

    def _input_rows(self, rows: torch.Tensor) -> torch.Tensor:
        """f16( H128(rows * rin) * RS )."""
        return msl.dense_scaled_had(rows, self._w.rin, RS)

    def _output_rows(self, mid: torch.Tensor) -> torch.Tensor:
        """f16( H128(mid) * RS * rout )."""
        return msl.dense_scaled_had_out(mid, self._w.rout, RS)

    def _gemv(self, xh: torch.Tensor) -> torch.Tensor:
        w = self._w
        return msl.dense_gemv(xh, w.code, w.K, w.IC, w.OC)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        if shape[-1] != self._w.IC:
            raise ValueError(f"input has {shape[-1]} channels, the linear takes {self._w.IC}")
        rows = x.reshape(-1, shape[-1])
        if rows.dtype != torch.float16:
            rows = rows.to(torch.float16)
        rows = rows.contiguous()
        if self._single_launch(rows.shape[0]):
            # input transform, product and output transform in one kernel
            w = self._w
            y = msl.coded_projections(rows, [w.code], [w.rin], [w.rout], w.K, w.IC, [w.OC],
                                      input_mode=msl.INPUT_RAW, rs=RS)[0]
            return self._finish(y, shape, x.dtype)
        return self._finish(self._product_rows(self._input_rows(rows)), shape, x.dtype)

    def _product_rows(self, xh: torch.Tensor) -> torch.Tensor:
        """Transformed rows -> f16 output rows: product and output transform."""
        w = self._w
        if msl.use_prefill_kernel(xh.shape[0]):
            # prefill: decode once per 256 rows into tensor memory, contract on tcgen05
            return msl.dense_gemm_tc(xh, w.code, w.K, w.IC, w.OC, rout=w.rout, rs=RS)
        if self._fused_had:
            return msl.dense_gemm_rows_direct_out(
                xh, w.code, w.rout, self.K, w.IC, w.OC,
                msl.dense_block_r(xh.shape[0], self._block_r_pin), RS)
        return self._output_rows(self._gemv(xh))

    def _single_launch(self, m: int) -> bool:
        """Whether a forward over m rows runs as one fused kernel (small decode
        batches on the tensor-core family with fused transforms)."""
        return (self._fused_had and msl.gemv_family() == "mma"
                and m <= msl.FUSE_INPUT_MAX_ROWS)

    def _finish(self, y: torch.Tensor, shape, dtype) -> torch.Tensor:
        if self.bias is not None:
            # the transform output is rounded to f16 before the correction is added
            y = (y.float() + self.bias.float()).to(torch.float16)
        return y.reshape(*shape[:-1], self._w.OC).to(dtype)


def _joint_prefill(linears) -> bool:
    """Whether a group of prefill projections runs as one tcgen05 launch: only when their
    column blocks together still fit one wave (one CTA per SM holds a whole SM), i.e. when each
    alone would be split along K and pay a launch's fixed cost for little work."""
    return sum(lin._w.OC // 128 for lin in linears) <= msl.sm_count()


def project_many(linears, x: torch.Tensor, one_wave: bool = False):
    """Evaluate up to eight coded projections of the same input (Q/K/V, gate/up, or
    everything that reads one hidden state) in one launch at decode batch sizes,
    whatever their rates.  Outputs equal ``[lin(x) for lin in linears]`` bit for
    bit: every projection keeps the split factor and the summation order it has
    when called alone.  ``one_wave=True`` gives that identity up for speed: split factors
    are chosen for each launch as a whole (``msl.wave_splits``), so sums are formed in an
    order of their own (deterministic, within the path's tolerance of the separate calls)."""
    linears = list(linears)
    shape = x.shape
    rows = x.reshape(-1, shape[-1])
    first = linears[0]
    mixed = any(lin.K != first.K for lin in linears)
    if (mixed and not msl.mixed_rates_supported() and first._single_launch(rows.shape[0])
            and msl.gemv_family() == "mma"):
        # one launch per rate: the projections of each rate together
        outs: dict[int, torch.Tensor] = {}
        for k in sorted({lin.K for lin in linears}):
            idx = [i for i, lin in enumerate(linears) if lin.K == k]
            for i, y in zip(idx, project_many([linears[i] for i in idx], x, one_wave)):
                outs[i] = y
        return [outs[i] for i in range(len(linears))]
    joint = (
        1 < len(linears) <= (msl.MAX_PROJECTIONS if first._single_launch(rows.shape[0]) else 4)
        and msl.gemv_family() == "mma"
        and all(lin._fused_had for lin in linears)
        and all(lin._w.IC == rows.shape[-1] for lin in linears)
        and (not mixed or msl.mixed_rates_supported())
        and rows.dtype == torch.float16
    )
    same_input = (1 < len(linears) <= 4 and rows.dtype == torch.float16
                  and all(lin._w.IC == rows.shape[-1] for lin in linears))
    if same_input and msl.use_prefill_kernel(rows.shape[0]):
        # prefill: one launch for all input transforms, then one tcgen05 GEMM per projection
        xhs = msl.dense_scaled_had_many(rows.contiguous(), [lin._w.rin for lin in linears], RS)
        if len(linears) <= 3 and all(lin.K == first.K for lin in linears) and _joint_prefill(linears):
            # projections too narrow to fill the GPU on their own share one launch
            ys = msl.dense_gemm_tc_many(xhs, [lin._w.code for lin in linears], first.K, first._w.IC,
                                        [lin._w.OC for lin in linears],
                                        [lin._w.rout for lin in linears], RS)
            return [lin._finish(y, shape, x.dtype) for lin, y in zip(linears, ys)]
        return [lin._finish(lin._product_rows(xh), shape, x.dtype) for lin, xh in zip(linears, xhs)]
    if not joint or msl.use_prefill_kernel(rows.shape[0]):
        return [lin(x) for lin in linears]
    rows = rows.contiguous()
    ws = [lin._w for lin in linears]
    codes, routs, ocs = [w.code for w in ws], [w.rout for w in ws], [w.OC for w in ws]
    splits = msl.wave_splits(first._w.IC, ocs) if one_wave else None
    if first._single_launch(rows.shape[0]):
        outs = msl.coded_projections(rows, codes, [w.rin for w in ws], routs, [w.K for w in ws],
                                     first._w.IC, ocs, input_mode=msl.INPUT_RAW, rs=RS,
                                     splits=splits)
    else:
        xhs = msl.dense_scaled_had_many(rows, [w.rin for w in ws], RS)
        outs = msl.coded_projections(xhs[0], codes, None, routs, [w.K for w in ws], first._w.IC,
                                     ocs, rs=RS, xs=xhs, splits=splits)
    return [lin._finish(y, shape, x.dtype) for lin, y in zip(linears, outs)]


def project_pair(first: EschaLinear, second: EschaLinear, x: torch.Tensor):
    """Evaluate two coded projections of the same input (gate/up, K/V) with one
    GEMM dispatch (:365-437).  Outputs equal ``first(x), second(x)`` bit for bit;
    a mixed-rate pair falls back to two calls."""
    a, b = project_many([first, second], x)
    return a, b


def swiglu_project(down: EschaLinear, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``down(f16(f16(silu(gate)) * up))`` -- the tail of a SwiGLU MLP.  For small
    decode batches the activation, the input transform, the product and the
    output transform run as one kernel; the result equals the unfused chain bit
    for bit."""
    shape = gate.shape
    g = gate.reshape(-1, shape[-1]).contiguous()
    u = up.reshape(-1, shape[-1]).contiguous()
    if g.shape != u.shape or g.shape[-1] != down._w.IC:
        raise ValueError(f"gate/up of shape {tuple(gate.shape)}/{tuple(up.shape)} do not feed a "
                         f"{down._w.IC}-channel projection")
    if down._single_launch(g.shape[0]) and g.dtype == torch.float16 and u.dtype == torch.float16:
        w = down._w
        y = msl.coded_projections(g, [w.code], [w.rin], [w.rout], w.K, w.IC, [w.OC],
                                  input_mode=msl.INPUT_SWIGLU, x_up=u, rs=RS)[0]
        return down._finish(y, shape, gate.dtype)
    # SwiGLU inside the input transform: one launch, no activation round trip
    xh = msl.dense_scaled_had_many(g.to(torch.float16), [down._w.rin], RS, up=u.to(torch.float16))[0]
    return down._finish(down._product_rows(xh), shape, gate.dtype)


def build(group: dict, device=None) -> EschaLinear:
    """Assemble one linear from its streamed tensors, keyed by HF leaf name (:440-452).

    Required: ``escha_code``, ``escha_rin``, ``escha_rout``.  Optional:
    ``escha_s_in``/``escha_s_out`` (implicitly ones when absent), ``escha_config``
    (cross-checked), ``bias`` (applied only with ESCHA_MLX_BIAS=1).
    """
    missing = REQUIRED - set(group)
    if missing:
        raise ValueError(f"coded linear is missing leaves {sorted(missing)}")
    w = EschaWeight(group["escha_code"], group["escha_rin"], group["escha_rout"],
                    group.get("escha_s_in"), group.get("escha_s_out"),
                    group.get("escha_config"), device=device)
    bias = group.get("bias") if apply_bias() else None
    return EschaLinear(w, bias)


def coded_bytes(obj) -> int:
    """Bytes of every coded stream under ``obj`` -- the ones NOT on the parameter
    tree (:455-483).  Accepts a Module or any list/tuple/dict of them."""
    total = 0
    stack = [obj]
    seen: set[int] = set()
    while stack:
        node = stack.pop()
        if id(node) in seen:
            continue
        seen.add(id(node))
        if isinstance(node, EschaLinear):
            total += sum(a.numel() * a.element_size() for a in node._w.arrays())
            continue
        if isinstance(node, torch.nn.Module):
            stack.extend(node.children())
            stack.extend(v for k, v in vars(node).items() if k.startswith("_") and
                         isinstance(v, (list, tuple, dict, torch.nn.Module)))
        elif isinstance(node, dict):
            stack.extend(node.values())
        elif isinstance(node, (list, tuple)):
            stack.extend(node)
    return total


#: Leaf names that together define one coded linear.
LEAVES = frozenset({"escha_code", "escha_rin", "escha_rout",
                    "escha_s_in", "escha_s_out", "escha_config", "bias"})

#: The subset that must be present before a linear can be built.
REQUIRED = frozenset({"escha_code", "escha_rin", "escha_rout"})

"""int8 dense linears (per-output-row fp16 scale) of the escha exports.

Counterpart of the reference's ``escha_mlx/quant.py``.  The reference repacks the
export's ``weight_int8 [N, K]`` + ``weight_scale [N]`` into MLX's affine-Q8 group
layout (``pack_q8`` :82-97, ``validate_pack`` :100-122) because that is the
format ``mx.quantized_matmul`` consumes; that repack is exact, so the arithmetic
contract is the un-repacked one, ``ref.w8a16`` (escha_mlx/ref.py:308-311):

    y = f16( f32(x) @ f32( f16( f32(w8) * f32(scale) ) )^T )

On B200 the kernel reads the export's own layout, so there is nothing to repack:
``pack_q8`` validates and returns ``(w8, f16 scale)`` instead of the reference's MLX
triple ``(u32 weight, scales, biases)``; ``validate_pack(group_size)`` is, as in the
reference, a one-time on-device check that the dequantised weight equals
``f16(w8 * scale)`` bit for bit; ``group_size`` arguments are accepted everywhere and do
not change the arithmetic (the reference documents group size as numerically free,
tests/test_mlx_cpu.py:19-41).
"""
from __future__ import annotations

import numpy as np
import torch

from ._lib import check, lib, ptr, stream

DEFAULT_GROUP = 64


def fit_group(k: int, group_size: int = DEFAULT_GROUP) -> int:
    """Largest supported group size dividing ``k`` (reference :68-79); informational."""
    for g in (group_size, 128, 64, 32):
        if g <= group_size and k % g == 0:
            return g
    raise ValueError(f"no supported group size divides K={k}")


def pack_q8(w8: np.ndarray, scale: np.ndarray, group_size: int = DEFAULT_GROUP):
    """Validate and return the int8 matrix and its f16 row scales in kernel layout."""
    w8 = np.ascontiguousarray(w8)
    scale = np.asarray(scale)
    if w8.dtype != np.int8 or w8.ndim != 2:
        raise ValueError(f"weight_int8 must be a 2-D int8 array, got {w8.dtype} {w8.shape}")
    if scale.shape != (w8.shape[0],):
        raise ValueError(f"weight_scale must have shape ({w8.shape[0]},), got {scale.shape}")
    if w8.shape[1] % 16:
        raise ValueError(f"int8 linear input width must be a multiple of 16, got {w8.shape[1]}")
    return w8, scale.astype(np.float16)


_VALIDATED: set[int] = set()


def validate_pack(group_size: int = DEFAULT_GROUP, device=None) -> None:
    """One-time on-device check, per group size like the reference's (:100-122): the int8
    linear fed one-hot rows must reproduce ``f16(w8 * scale)`` exactly, i.e. what the
    kernel dequantises is the export's weight bit for bit.  ``group_size`` only keys the
    cache: the kernel's layout has one scale per output row whatever the export's groups."""
    if group_size in _VALIDATED:
        return
    rng = np.random.default_rng(0)
    w8 = rng.integers(-128, 128, size=(16, 512), dtype=np.int8)
    scale = (rng.random(16, dtype=np.float32) * 0.05 + 1e-3).astype(np.float16)
    pw, ps = pack_q8(w8, scale, fit_group(512, group_size))
    dev = torch.device(device or "cuda")
    eye = torch.eye(512, dtype=torch.float16, device=dev)
    got = w8a16(eye, torch.from_numpy(pw).to(dev), torch.from_numpy(ps).to(dev)).T.cpu().numpy()
    want = (w8.astype(np.float32) * scale.astype(np.float32)[:, None]).astype(np.float16)
    if not np.array_equal(got.view(np.uint16), want.view(np.uint16)):
        raise ValueError(f"int8 repack is not bit-exact for group size {group_size}")
    _VALIDATED.add(group_size)


def w8a16(x: torch.Tensor, w8: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """x [M, K] f16, w8 [N, K] int8, scale [N] f16 -> y [M, N] f16."""
    m, kd = x.shape
    n = w8.shape[0]
    if w8.shape[1] != kd:
        raise ValueError(f"input has {kd} channels, the int8 linear takes {w8.shape[1]}")
    y = torch.empty((m, n), dtype=torch.float16, device=x.device)
    check(lib.escha_w8a16(ptr(x, torch.float16), ptr(w8, torch.int8), ptr(scale, torch.float16),
                          m, n, kd, ptr(y), stream()))
    return y


Q8_MANY_MAX = 4


def w8a16_many(x: torch.Tensor, weights: list[tuple[torch.Tensor, torch.Tensor]]) -> list[torch.Tensor]:
    """Several int8 linears of the same rows in one launch (1..4; output widths multiples of
    16, input width a multiple of 64), each output bit-identical to its own `w8a16` call.
    No reference counterpart: it issues one quantized matmul per linear (:129-143)."""
    import ctypes
    n = len(weights)
    if not 1 <= n <= Q8_MANY_MAX:
        raise ValueError(f"w8a16_many takes 1..{Q8_MANY_MAX} linears, got {n}")
    m, kd = x.shape
    for w8, _ in weights:
        if w8.shape[1] != kd:
            raise ValueError(f"input has {kd} channels, an int8 linear takes {w8.shape[1]}")
    ys = [torch.empty((m, w8.shape[0]), dtype=torch.float16, device=x.device) for w8, _ in weights]
    table = ctypes.c_void_p * n
    check(lib.escha_w8a16_many(
        ptr(x, torch.float16), n,
        table(*[ptr(w8, torch.int8).value for w8, _ in weights]),
        table(*[ptr(sc, torch.float16).value for _, sc in weights]),
        (ctypes.c_int * n)(*[w8.shape[0] for w8, _ in weights]), kd, m,
        table(*[ptr(y).value for y in ys]), stream()))
    return ys


def project_many_q8(linears: list["EschaQ8Linear"], x: torch.Tensor) -> list[torch.Tensor]:
    """`[lin(x) for lin in linears]` in one launch when the shapes allow it (as `w8a16_many`),
    otherwise one launch each."""
    shape = x.shape
    rows = x.reshape(-1, shape[-1]).to(torch.float16).contiguous()
    ok = (1 <= len(linears) <= Q8_MANY_MAX and rows.shape[1] % 64 == 0
          and all(l.out_features % 16 == 0 and l.in_features == rows.shape[1] for l in linears))
    if not ok:
        return [lin(x) for lin in linears]
    ys = w8a16_many(rows, [(l._w8, l._scale) for l in linears])
    return [y.reshape(*shape[:-1], l.out_features) for y, l in zip(ys, linears)]


class EschaQ8Linear(torch.nn.Module):
    """An int8-weight linear with per-output-row scale (reference :129-143)."""

    def __init__(self, w8, scale, group_size: int = DEFAULT_GROUP, device=None) -> None:
        super().__init__()
        if isinstance(w8, torch.Tensor):
            # leaves already resident: int8 [N, K] and one scale per output row
            if w8.dtype != torch.int8 or w8.dim() != 2 or w8.shape[1] % 16:
                raise ValueError("weight_int8 must be a 2-D int8 tensor with a multiple of 16 "
                                 f"input channels, got {w8.dtype} {tuple(w8.shape)}")
            if tuple(scale.shape) != (w8.shape[0],):
                raise ValueError(f"weight_scale must have shape ({w8.shape[0]},), got {tuple(scale.shape)}")
            self._w8 = w8.contiguous()
            self._scale = scale.to(device=w8.device, dtype=torch.float16).contiguous()
            self.out_features, self.in_features = w8.shape
            return
        pw, ps = pack_q8(w8, scale, group_size)
        dev = device or "cuda"
        validate_pack(group_size, dev)
        self._w8 = torch.from_numpy(pw).to(dev)
        self._scale = torch.from_numpy(ps).to(dev)
        self.out_features, self.in_features = pw.shape

    def arrays(self) -> list[torch.Tensor]:
        return [self._w8, self._scale]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        rows = x.reshape(-1, shape[-1]).to(torch.float16).contiguous()
        return w8a16(rows, self._w8, self._scale).reshape(*shape[:-1], self.out_features)


Q8_HEAD_MAX_ROWS = 8


def q8_head(x: torch.Tensor, w8: torch.Tensor, scale: torch.Tensor,
            group_size: int = DEFAULT_GROUP) -> torch.Tensor:
    """Project 1..8 flattened rows through an int8 vocabulary matrix (reference
    :203-240; ``group_size`` is accepted for the reference's signature and unused, the
    scales here are per output row).  The reference needs a separate small-row kernel for this; here it is
    the same tensor-core int8 linear, which streams a 311 MB head at 85% of the HBM
    peak at one row."""
    rows = x.reshape(-1, x.shape[-1])
    if not 1 <= rows.shape[0] <= Q8_HEAD_MAX_ROWS:
        raise ValueError(f"q8_head supports 1..{Q8_HEAD_MAX_ROWS} rows, got {rows.shape[0]}")
    return w8a16(rows.to(torch.float16).contiguous(), w8, scale).reshape(*x.shape[:-1], w8.shape[0])


class EschaQ8Head(EschaQ8Linear):
    """int8 vocabulary head (reference :243-257); every row count takes the same kernel."""


class EschaQ8Embedding(torch.nn.Module):
    """Embedding over an int8 table with per-row scale (reference :260-273):
    ``f16(f32(w8[ids]) * f32(scale[ids]))``."""

    def __init__(self, w8, scale, group_size: int = DEFAULT_GROUP, device=None,
                 dtype=torch.float16) -> None:
        super().__init__()
        lin = EschaQ8Linear(w8, scale, group_size, device)
        self._w8, self._scale = lin._w8, lin._scale
        self.num_embeddings, self.embedding_dim = self._w8.shape
        self._dtype = dtype

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        flat = ids.reshape(-1).to(device=self._w8.device, dtype=torch.int64).contiguous()
        if flat.numel() == 0:
            raise ValueError("embedding lookup needs at least one id")
        out = torch.empty((flat.numel(), self.embedding_dim), dtype=torch.float16,
                          device=self._w8.device)
        check(lib.escha_q8_embed(ptr(flat, torch.int64), ptr(self._w8, torch.int8),
                                 ptr(self._scale, torch.float16), flat.numel(),
                                 self.num_embeddings, self.embedding_dim, ptr(out), stream()))
        return out.reshape(*ids.shape, self.embedding_dim).to(self._dtype)


def make_head(w8, scale, group_size: int = DEFAULT_GROUP, device=None) -> EschaQ8Head:
    """Build the vocabulary projection (reference :289-306)."""
    return EschaQ8Head(w8, scale, group_size, device)


def make_embedding(w8, scale, group_size: int = DEFAULT_GROUP, device=None) -> EschaQ8Embedding:
    """Build the int8 embedding (reference :309-322)."""
    return EschaQ8Embedding(w8, scale, group_size, device)


def make_linear(w8: np.ndarray, scale: np.ndarray, group_size: int = DEFAULT_GROUP,
                device=None) -> EschaQ8Linear:
    """Build the int8 linear module from export leaves (reference :269-308)."""
    return EschaQ8Linear(w8, scale, group_size, device)

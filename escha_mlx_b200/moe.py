"""Architecture-agnostic expert toolkit: the E-stacked expert container, the
128-block Hadamard transform and row grouping.

Mirror of the reference's ``escha_mlx/moe.py`` (``had_blocks`` :19-27,
``build_groups`` :30-78, ``n_groups_bound`` :81-83, ``EschaExperts`` :86-105)
over CUDA ``torch.Tensor``s.  ``build_groups`` keeps the reference's output format
for callers written against it; the tensor-core kernel itself consumes the more
compact row jobs of ``msl.group_rows`` (no padding rows).
"""
from __future__ import annotations

import numpy as np
import torch

from . import msl
from ._lib import check, lib, ptr, stream

RS = msl.RS


def had_blocks(x: torch.Tensor) -> torch.Tensor:
    """Unnormalised 128-point WHT on last-dimension blocks of an f32 tensor (:19-27)."""
    shape = x.shape
    if shape[-1] % 128:
        raise ValueError(f"Hadamard dimension must be divisible by 128, got {shape[-1]}")
    xf = x.to(torch.float32).contiguous()
    out = torch.empty_like(xf)
    check(lib.escha_had128(ptr(xf), xf.numel() // 128, ptr(out), stream()))
    return out.reshape(shape)


def build_groups(row_expert: torch.Tensor, E: int, R: int, n_groups: int,
                 with_sorted: bool = False):
    """Sort rows by expert and pack them into fixed R-row groups (:30-78).

    Returns (rows_idx [n_groups*R] i32, group_expert [n_groups] i32).  Padding
    slots hold M (the caller appends a zero row at index M); groups past the end
    hold expert -1.  Device-resident, static shapes, no host synchronisation.
    """
    m = row_expert.shape[0]
    dev = row_expert.device
    re64 = row_expert.long()
    order = torch.argsort(re64, stable=True)
    se = re64[order]
    counts = torch.zeros(E, dtype=torch.int64, device=dev).scatter_add_(
        0, re64, torch.ones(m, dtype=torch.int64, device=dev))
    padded = (counts + (R - 1)) // R * R
    cum_padded = torch.cumsum(padded, 0)
    dst_start = cum_padded - padded
    src_start = torch.cumsum(counts, 0) - counts
    dst = dst_start[se] + (torch.arange(m, device=dev) - src_start[se])
    rows_idx = torch.full((n_groups * R,), m, dtype=torch.int32, device=dev)
    rows_idx[dst] = order.to(torch.int32)
    gidx = torch.arange(n_groups, device=dev)
    total_groups = cum_padded[-1] // R
    # group g belongs to the first expert whose padded range ends after slot g*R
    owner = torch.searchsorted(cum_padded, gidx * R, right=True).clamp(max=E - 1)
    group_expert = torch.where(gidx < total_groups, owner,
                               torch.full_like(owner, -1)).to(torch.int32)
    if not with_sorted:
        return rows_idx, group_expert
    ge = group_expert.clamp(min=0).long()
    j = gidx - (dst_start // R)[ge]
    src_row0 = (src_start[ge] + j * R).to(torch.int32)
    n_valid = (counts[ge] - j * R).clamp(0, R).to(torch.int32)
    n_valid = torch.where(group_expert < 0, torch.zeros_like(n_valid), n_valid)
    return rows_idx, group_expert, order.to(torch.int32), src_row0, n_valid


def n_groups_bound(m: int, E: int, R: int) -> int:
    """Static upper bound on groups: every expert may waste up to R-1 slots (:81-83)."""
    return (m + E * (R - 1) + R - 1) // R


class EschaExperts:
    """Container for one projection's E-stacked arrays (kept off the module
    parameter tree via leading-underscore attributes on the owner)."""

    def __init__(self, code_i16, rin, rout, device=None) -> None:
        if isinstance(code_i16, torch.Tensor):
            # already packed and resident: [E, TK, TN, 8K] 32-bit words with f32
            # [E, IC] / [E, OC] vectors on the same device
            if code_i16.dim() != 4 or code_i16.dtype != torch.int32 or code_i16.shape[-1] % 8:
                raise ValueError("packed E-stacked code must be an int32 [E, TK, TN, 8K] tensor, "
                                 f"got {code_i16.dtype} {tuple(code_i16.shape)}")
            e, tk, tn, wpt = code_i16.shape
            self.K = wpt // 8
            packed = code_i16
        else:
            if np.ndim(code_i16) != 4:
                raise ValueError(f"E-stacked code must be [E, TK, TN, 16K], got shape {np.shape(code_i16)}")
            e, tk, tn, wpt2 = code_i16.shape
            if wpt2 % 16:
                raise ValueError(f"escha code last dim must be 16*K, got {wpt2}")
            self.K = wpt2 // 16
            packed = None
        if self.K not in (2, 3):
            raise ValueError(f"escha code implies K={self.K}; this runtime implements K in [2, 3]")
        self.E, self.IC, self.OC = e, tk * 16, tn * 16
        if self.IC % 128 or self.OC % 128:
            raise ValueError(
                f"escha expert dimensions must be multiples of 128, got {self.IC}x{self.OC}")
        if tuple(np.shape(rin)) != (e, self.IC) or tuple(np.shape(rout)) != (e, self.OC):
            raise ValueError(
                f"transform vectors {tuple(np.shape(rin))}/{tuple(np.shape(rout))} do not match the "
                f"E-stacked stream's ({e}, {self.IC})/({e}, {self.OC})")
        if packed is not None:
            self.code = packed.contiguous()
            self.rin = rin.to(device=packed.device, dtype=torch.float32).contiguous()
            self.rout = rout.to(device=packed.device, dtype=torch.float32).contiguous()
            return
        self.code = msl.code_tensor(code_i16, device)                     # [E, TK, TN, 8K] words
        dev = self.code.device
        self.rin = torch.from_numpy(np.asarray(rin).astype(np.float32)).to(dev)    # [E, IC] f32
        self.rout = torch.from_numpy(np.asarray(rout).astype(np.float32)).to(dev)  # [E, OC] f32

    def code_numpy(self) -> np.ndarray:
        return self.code.cpu().numpy().view(np.uint32)

    def arrays(self) -> list[torch.Tensor]:
        return [self.code, self.rin, self.rout]

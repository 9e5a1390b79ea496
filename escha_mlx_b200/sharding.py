"""Multi-GPU sharding of the coded path: one process per GPU, torch.distributed
(NCCL over NVLink on the GPUs, gloo in CPU tests) for the exchange steps.

The reference is single-device; these partitions are chosen so that no
arithmetic crosses a shard boundary and results stay bit-identical to one GPU:

* dense projections -- split-N tensor parallel: output channels are cut in whole
  128-channel blocks (one Hadamard block = one CTA's output tile), so decode,
  GEMV columns and the output transform are all shard-local; shards are joined by
  an all-gather of f16 outputs.  There is no all-reduce, hence no cross-GPU float
  sum and nothing that could reorder a reduction.
* routed experts -- expert parallel: the E-stacked streams are cut on the expert
  axis; each (token, slot) row is computed by the rank that owns its expert and
  the f16 expert outputs are all-gathered, after which every rank runs the same
  fixed slot-order combine.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist


def world() -> tuple[int, int]:
    """(rank, world_size); (0, 1) when torch.distributed is not initialised."""
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def block_range(n_blocks: int, rank: int, count: int) -> tuple[int, int]:
    """Contiguous, equal split of ``n_blocks`` 128-channel blocks; raises if uneven."""
    if count < 1 or not 0 <= rank < count:
        raise ValueError(f"rank {rank} outside a group of {count}")
    if n_blocks % count:
        raise ValueError(f"{n_blocks} blocks do not split evenly over {count} ranks")
    per = n_blocks // count
    return rank * per, (rank + 1) * per


def shard_code_out(code: np.ndarray, rout: np.ndarray, rank: int, count: int):
    """Split-N shard of one dense projection's host leaves: code [TK, TN, 16K] is cut
    on TN, rout on OC; rin and the input transform stay replicated."""
    tn = code.shape[1]
    b0, b1 = block_range(tn // 8, rank, count)
    return (np.ascontiguousarray(code[:, b0 * 8:b1 * 8, :]),
            np.ascontiguousarray(rout[b0 * 128:b1 * 128]))


def expert_range(E: int, rank: int, count: int) -> tuple[int, int]:
    """Experts [lo, hi) owned by ``rank`` (contiguous, equal split)."""
    if E % count:
        raise ValueError(f"{E} experts do not split evenly over {count} ranks")
    per = E // count
    return rank * per, (rank + 1) * per


def shard_experts(code: np.ndarray, rin: np.ndarray, rout: np.ndarray, rank: int, count: int):
    """Expert-parallel shard of one E-stacked projection's host leaves."""
    lo, hi = expert_range(code.shape[0], rank, count)
    return (np.ascontiguousarray(code[lo:hi]), np.ascontiguousarray(rin[lo:hi]),
            np.ascontiguousarray(rout[lo:hi]))


def all_gather_columns(y_local: torch.Tensor, group=None) -> torch.Tensor:
    """Join split-N output shards [M, OC/G] -> [M, OC] on every rank (exact)."""
    rank, size = world()
    if size == 1:
        return y_local
    m, oc_local = y_local.shape
    flat = torch.empty((size * m, oc_local), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(flat, y_local.contiguous(), group=group)
    if m == 1:
        return flat.view(1, size * oc_local)
    return flat.view(size, m, oc_local).permute(1, 0, 2).reshape(m, size * oc_local)


def all_gather_rows(rows_local: torch.Tensor, group=None) -> torch.Tensor:
    """Every rank's [m, H] buffer side by side -> [size * m, H] (rank-major)."""
    rank, size = world()
    if size == 1:
        return rows_local
    m, h = rows_local.shape
    flat = torch.empty((size * m, h), dtype=rows_local.dtype, device=rows_local.device)
    dist.all_gather_into_tensor(flat, rows_local.contiguous(), group=group)
    return flat


def all_gather_rows_by_owner(rows_local: torch.Tensor, owned: torch.Tensor, group=None) -> torch.Tensor:
    """Expert-parallel join: every rank computed the rows whose expert it owns
    (``owned`` [m] bool marks them; other rows of ``rows_local`` are ignored).
    Returns the full [m, H] tensor on every rank.  Rows are disjoint across
    ranks, so the join selects -- it never adds."""
    rank, size = world()
    if size == 1:
        return rows_local
    m, h = rows_local.shape
    flat = torch.empty((size * m, h), dtype=rows_local.dtype, device=rows_local.device)
    dist.all_gather_into_tensor(flat, rows_local.contiguous(), group=group)
    masks = torch.empty((size * m,), dtype=torch.int32, device=rows_local.device)
    dist.all_gather_into_tensor(masks, owned.to(torch.int32).contiguous(), group=group)
    owner = masks.view(size, m).argmax(dim=0)                         # [m]
    return flat.view(size, m, h)[owner, torch.arange(m, device=rows_local.device)]

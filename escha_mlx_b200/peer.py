"""Peer-mapped buffers for the fused GEMV + all-gather (one process per GPU of a node).

The reference is single-device; this module has no counterpart there.  Split-N
tensor parallelism needs every rank's output columns on every rank.  Instead of a
library all-gather after the kernel, the GEMV epilogue stores its 128-channel blocks
straight into the gathered row of every GPU (``msl.coded_projections(gather=...)``),
and the ranks meet in ``PeerGroup.barrier()`` -- a one-warp kernel over peer-mapped
flag words -- before anyone reads.

Buffers are ordinary CUDA allocations shared between the processes with CUDA IPC
(the same mechanism ``torch.multiprocessing`` uses for CUDA tensors); handles travel
through ``torch.distributed`` once, at set-up.  Nothing here is on the per-step path
except the barrier launch.

Rules for users:

* a gathered buffer may be overwritten only after a later barrier has passed on every
  rank (keep two buffers per tensor and alternate, or use one set per CUDA graph and
  at least two graphs);
* every rank must launch the same sequence of gathers and barriers;
* ranks must sit on different GPUs (the barrier kernels wait for one another).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ._lib import check, lib, stream


class PeerUnavailable(RuntimeError):
    """Raised on EVERY rank when any rank could not map its peers' memory (no CUDA IPC in
    this environment, no peer access between two GPUs ...): callers fall back to NCCL."""


class PeerTensor:
    """A tensor of identical shape on every rank, each mapped into every process."""

    def __init__(self, local: torch.Tensor, views: list[torch.Tensor | None], rank: int) -> None:
        self.local = local
        self._views = views                 # keeps the IPC mappings alive
        self.rank = rank
        self.ptrs = [local.data_ptr() if r == rank else v.data_ptr() for r, v in enumerate(views)]

    def peer_ptrs(self) -> list[int]:
        """Device addresses of the other ranks' copies, in rank order."""
        return [p for r, p in enumerate(self.ptrs) if r != self.rank]

    def carve(self, offset: int, shape) -> "PeerTensor":
        """A sub-tensor of ``shape`` starting ``offset`` elements into this (flat) tensor,
        at the same place in every rank's copy.  Offsets must keep 16-byte alignment."""
        numel = 1
        for d in shape:
            numel *= int(d)
        flat = self.local.reshape(-1)
        if offset < 0 or offset + numel > flat.numel() or (offset * flat.element_size()) % 16:
            raise ValueError(f"cannot carve {numel} elements at offset {offset} of {flat.numel()}")
        sub = object.__new__(PeerTensor)
        sub.local = flat[offset:offset + numel].view(*shape)
        sub._views = self._views
        sub.rank = self.rank
        sub.ptrs = [p + offset * flat.element_size() for p in self.ptrs]
        return sub


class PeerGroup:
    """The GPUs of one node, as seen from this rank."""

    def __init__(self, group=None) -> None:
        if not dist.is_initialized():
            raise RuntimeError("PeerGroup needs an initialised torch.distributed process group")
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)
        if not 2 <= self.size <= 8:
            raise ValueError(f"peer groups span 2 to 8 GPUs of one node, got {self.size}")
        self.device = torch.device("cuda", torch.cuda.current_device())
        self._made: list[PeerTensor] = []
        self._flags = self.empty((self.size + 2,), torch.int32, zero=True)
        self._flag_table = (ctypes.c_void_p * self.size)(*self._flags.ptrs)
        dist.barrier(group)     # every rank's flag words are zero before any kernel signals

    def empty(self, shape, dtype, zero: bool = False) -> PeerTensor:
        """Allocate ``shape`` on every rank and map all copies into this process."""
        numel = 1
        for d in shape:
            numel *= int(d)
        make = torch.zeros if zero else torch.empty
        # a dedicated allocation: an IPC handle exports the whole underlying block
        local = make((max(numel, 1),), dtype=dtype, device=self.device)
        torch.cuda.synchronize()
        error, handle = None, None
        try:
            handle = local.untyped_storage()._share_cuda_()
        except Exception as e:                      # noqa: BLE001 -- reported collectively below
            error = e
        gathered: list = [None] * self.size
        dist.all_gather_object(gathered, handle, group=self.group)
        views: list[torch.Tensor | None] = []
        for r, h in enumerate(gathered):
            if r == self.rank or error is not None or h is None:
                views.append(None)
                continue
            try:
                # the exporter's device index is not ours: open the handle on this device
                storage = torch.UntypedStorage._new_shared_cuda(self.device.index, *h[1:])
                views.append(torch.empty(0, dtype=dtype, device=self.device).set_(
                    storage, 0, (max(numel, 1),)))
            except Exception as e:                  # noqa: BLE001
                error = e
                views.append(None)
        # every rank learns whether every rank succeeded, so that all fall back together
        ok = torch.tensor([0 if (error is not None or any(h is None for h in gathered)) else 1],
                          device=self.device, dtype=torch.int32)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        if int(ok.item()) == 0:
            raise PeerUnavailable(f"peer-mapped memory is not available on every rank "
                                  f"(this rank: {error!r})")
        t = PeerTensor(local.view(*shape) if numel else local, views, self.rank)
        self._made.append(t)
        return t

    def close(self) -> None:
        """Drop every mapping of other ranks' memory made through this group.  Call on all
        ranks, with no kernel of this group in flight, before the process group is
        destroyed: the exporting rank must outlive its importers' mappings."""
        import gc
        torch.cuda.synchronize()
        dist.barrier(self.group)
        # 1. every rank lets go of what it imported (in place: tensors carved out of t share
        #    the list, and must let go as well) ...
        for t in self._made:
            t._views.clear()
        gc.collect()
        torch.cuda.synchronize()
        dist.barrier(self.group)
        # 2. ... and only then do the exporters free their blocks.  When both happened in one
        #    pass, a rank could free an export while another rank still had it mapped; with the
        #    80 buffers of a 40-layer MoE stack one rank then died with SIGSEGV in interpreter
        #    teardown, after its last line of Python, in two runs of two.  With the barrier in
        #    between, five runs of five (MoE layer, 40-layer step, dense layer) ended cleanly.
        for t in self._made:
            t.local = None
        self._made = []
        self._flags = None
        gc.collect()
        torch.cuda.ipc_collect()
        torch.cuda.synchronize()
        dist.barrier(self.group)

    def barrier(self) -> None:
        """Enqueue the cross-GPU barrier on the current stream (graph-capturable)."""
        check(lib.escha_peer_barrier(ctypes.c_void_p(self._flags.local.data_ptr()), self._flag_table,
                                     self.rank, self.size, stream()))

    def status(self) -> int:
        """1 if a barrier on this rank ever gave up waiting (synchronises the stream)."""
        torch.cuda.synchronize()
        return int(self._flags.local[self.size + 1].item())

"""One rank of the multi-GPU parity check (launched by test_gpu_multi.py through
``python -m torch.distributed.run``; one process per GPU, NCCL).

Every rank holds the full seeded weights as well as its shard, computes the
unsharded result on its own GPU, and checks that shard + collective reproduces it
bit for bit:

* split-N tensor parallel: ``EschaWeight.shard_out`` + ``all_gather_columns``;
* expert parallel: ``EschaSparseMoeBlock(expert_range=...)`` whose join is
  ``all_gather_rows_by_owner``;
* the same two with kernels and NCCL collectives captured in one CUDA graph.

Prints ``MULTI_GPU_OK <rank>`` on success; any mismatch raises.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from escha_mlx_b200 import dense, graphs, moe, msl, peer, sharding, synth  # noqa: E402
from escha_mlx_b200.models.qwen3_5_moe import EschaSparseMoeBlock  # noqa: E402


def same(a: torch.Tensor, b: torch.Tensor, what: str) -> None:
    if a.shape != b.shape or not torch.equal(a.view(torch.int16), b.view(torch.int16)):
        raise AssertionError(f"rank {dist.get_rank()}: {what} differs from the unsharded result")


def split_n(device, rank, size) -> None:
    for K, IC, OC in [(2, 1024, 128 * 2 * size), (3, 512, 128 * 3 * size)]:
        rng = np.random.default_rng(K * 7 + size)           # same on every rank
        code, rin, rout = synth.coded_projection(rng, IC, OC, K)
        w = dense.EschaWeight(code, rin, rout, device=device)
        full, part = dense.EschaLinear(w), dense.EschaLinear(w.shard_out(rank, size))
        for M in (1, 4, 16, 40):
            x = torch.from_numpy(synth.activations(rng, M, IC)).to(device)
            want = full(x)
            same(sharding.all_gather_columns(part(x)), want, f"split-N K={K} M={M}")
            g = graphs.GraphedCall(lambda t: sharding.all_gather_columns(part(t)), [x])
            for _ in range(2):
                same(g(x), want, f"graphed split-N K={K} M={M}")
            g.close()   # NCCL's teardown waits for graphs that captured its collectives


def fused_gather(device, rank, size) -> None:
    """Split-N shards whose GEMV epilogue stores straight into every GPU's gathered row,
    followed by the peer barrier: equal to the unsharded linear bit for bit."""
    pg = peer.PeerGroup()
    K, IC, OCs = 2, 1024, [128 * 2 * size, 128 * size]
    rng = np.random.default_rng(5 + size)
    ws = [dense.EschaWeight(*synth.coded_projection(rng, IC, oc, K), device=device) for oc in OCs]
    fulls = [dense.EschaLinear(w) for w in ws]
    shards = [w.shard_out(rank, size) for w in ws]
    for M in (1, 3, 12):
        x = torch.from_numpy(synth.activations(rng, M, IC)).to(device)
        want = [f(x) for f in fulls]
        # two buffer sets, alternated: a buffer is rewritten only after a later barrier
        bufs = [[pg.empty((M, oc), torch.float16) for oc in OCs] for _ in range(2)]

        def step(t, which):
            gather = [(b, rank * s.OC) for b, s in zip(bufs[which], shards)]
            outs = msl.coded_projections(t, [s.code for s in shards], [s.rin for s in shards],
                                         [s.rout for s in shards], K, IC, [s.OC for s in shards],
                                         input_mode=msl.INPUT_RAW, gather=gather)
            pg.barrier()
            return [o.clone() for o in outs]

        for it in range(4):
            got = step(x, it % 2)
            for g, w in zip(got, want):
                same(g, w, f"fused gather M={M} it={it}")
        graphed = [graphs.GraphedCall(lambda t, wch=wch: step(t, wch), [x]) for wch in range(2)]
        for it in range(4):
            got = graphed[it % 2](x)
            for g, w in zip(got, want):
                same(g, w, f"graphed fused gather M={M} it={it}")
        for g in graphed:
            g.close()
    if pg.status() != 0:
        raise AssertionError(f"rank {rank}: a peer barrier gave up waiting")
    del bufs, graphed
    pg.close()


def expert_parallel(device, rank, size) -> None:
    E, H, I, top_k = 8 * size, 256, 128, 4
    rng = np.random.default_rng(100 + size)
    w = synth.moe_weights(rng, E, H, I, 2, 3)
    shared = {k[3:]: v for k, v in w.items() if k.startswith("sh_")}

    def block(lo, hi):
        gu = moe.EschaExperts(w["gu_code"][lo:hi], w["gu_rin"][lo:hi], w["gu_rout"][lo:hi], device=device)
        dn = moe.EschaExperts(w["dn_code"][lo:hi], w["dn_rin"][lo:hi], w["dn_rout"][lo:hi], device=device)
        return EschaSparseMoeBlock(H, E, top_k, gu, dn, w["gate_w"], w["shg_w"], shared,
                                   expert_range=(lo, hi))

    full = block(0, E)
    part = block(*sharding.expert_range(E, rank, size))
    for T in (1, 8, 37):
        x = torch.from_numpy(synth.activations(rng, T, H)).to(device)
        want = full(x)
        same(part(x), want, f"expert-parallel T={T}")
        g = graphs.GraphedCall(lambda t: part(t), [x])
        for _ in range(2):
            same(g(x), want, f"graphed expert-parallel T={T}")
        g.close()


def expert_parallel_over_peers(device, rank, size) -> None:
    """Expert shards whose second leg stores its rows into every GPU's buffer, one peer
    barrier per block: equal to the unsharded block bit for bit."""
    pg = peer.PeerGroup()
    E, H, I, top_k = 8 * size, 256, 128, 4
    rng = np.random.default_rng(300 + size)
    w = synth.moe_weights(rng, E, H, I, 2, 2)
    shared = {k[3:]: v for k, v in w.items() if k.startswith("sh_")}

    def block(lo, hi, pgroup):
        gu = moe.EschaExperts(w["gu_code"][lo:hi], w["gu_rin"][lo:hi], w["gu_rout"][lo:hi], device=device)
        dn = moe.EschaExperts(w["dn_code"][lo:hi], w["dn_rin"][lo:hi], w["dn_rout"][lo:hi], device=device)
        return EschaSparseMoeBlock(H, E, top_k, gu, dn, w["gate_w"], w["shg_w"], shared,
                                   expert_range=(lo, hi), peer_group=pgroup)

    full = block(0, E, None)
    part = block(*sharding.expert_range(E, rank, size), pg)
    for T in (1, 8, 37):
        x = torch.from_numpy(synth.activations(rng, T, H)).to(device)
        want = full(x)
        for it in range(3):
            same(part(x), want, f"peer expert-parallel T={T} it={it}")
        # two calls per graph: a buffer is reused only after the other call's barrier
        g = graphs.GraphedCall(lambda t: torch.stack([part(t), part(t)]), [x])
        for it in range(3):
            both = g(x)
            same(both[0], want, f"graphed peer expert-parallel T={T} it={it} call 0")
            same(both[1], want, f"graphed peer expert-parallel T={T} it={it} call 1")
        g.close()
    if pg.status() != 0:
        raise AssertionError(f"rank {rank}: a peer barrier gave up waiting")
    part._peer_bufs = {}
    del part
    pg.close()


def main() -> None:
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    rank, size = dist.get_rank(), dist.get_world_size()
    split_n(device, rank, size)
    fused_gather(device, rank, size)
    expert_parallel(device, rank, size)
    expert_parallel_over_peers(device, rank, size)
    torch.cuda.synchronize()
    dist.barrier()
    print(f"MULTI_GPU_OK {rank}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

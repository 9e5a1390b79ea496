"""CPU, world_size 2 over gloo: the multi-GPU partitions are exact.  Each rank
computes its shard with the CPU oracle (standing in for the kernels, which the
GPU tests pin to it), the shards are joined with the package's collectives, and
the result must equal the unsharded computation bit for bit."""
from __future__ import annotations

import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _init(rank: int, size: int, port: int) -> None:
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=size)


def _split_n_worker(rank: int, size: int, port: int, q) -> None:
    _init(rank, size, port)
    from escha_mlx_b200 import sharding, synth
    from oracle import escha_oracle as oracle
    oracle.set_num_threads(2)
    rng = np.random.default_rng(3)
    K, IC, OC, M = 3, 256, 512, 3
    code, rin, rout = synth.coded_projection(rng, IC, OC, K)
    x = synth.activations(rng, M, IC)
    ri, ro = oracle.fold_scales(rin, rout)
    full = oracle.dense_linear(x, code, ri, ro, K)
    c_loc, ro_loc = sharding.shard_code_out(code, ro, rank, size)
    y_loc = oracle.dense_linear(x, c_loc, ri, ro_loc, K)
    joined = sharding.all_gather_columns(torch.from_numpy(y_loc)).numpy()
    ok = np.array_equal(joined.view(np.uint16), full.view(np.uint16))
    one = sharding.all_gather_columns(torch.from_numpy(y_loc[:1].copy())).numpy()
    ok = ok and np.array_equal(one.view(np.uint16), full[:1].view(np.uint16))
    q.put((rank, bool(ok)))
    dist.barrier()
    dist.destroy_process_group()


def _expert_parallel_worker(rank: int, size: int, port: int, q) -> None:
    _init(rank, size, port)
    from escha_mlx_b200 import sharding, synth
    from oracle import escha_oracle as oracle
    oracle.set_num_threads(2)
    rng = np.random.default_rng(9)
    E, H, I, T, top_k = 8, 256, 128, 5, 2
    w = synth.moe_weights(rng, E, H, I, 2, 2)
    x = synth.activations(rng, T, H)
    ids, scores = synth.topk_softmax(synth.router_logits(rng, T, E), top_k)
    full = oracle.moe_routed(x, ids, scores, w["gu_code"], w["gu_rin"], w["gu_rout"], 2,
                             w["dn_code"], w["dn_rin"], w["dn_rout"], 2)
    # this rank's experts; rows it does not own run on local expert 0 and are discarded
    lo, hi = sharding.expert_range(E, rank, size)
    gu = sharding.shard_experts(w["gu_code"], w["gu_rin"], w["gu_rout"], rank, size)
    dn = sharding.shard_experts(w["dn_code"], w["dn_rin"], w["dn_rout"], rank, size)
    re = ids.reshape(-1)
    owned = (re >= lo) & (re < hi)
    local = np.where(owned, re - lo, 0).astype(np.int32)
    rows = np.repeat(x, top_k, axis=0)
    gu16 = oracle.expert_linear(rows, gu[0], gu[1].astype(np.float32), gu[2].astype(np.float32), 2, local)
    h = oracle.swiglu(gu16)
    d16 = oracle.expert_linear(h, dn[0], dn[1].astype(np.float32), dn[2].astype(np.float32), 2, local)
    joined = sharding.all_gather_rows_by_owner(torch.from_numpy(d16),
                                               torch.from_numpy(owned)).numpy()
    # identical fixed slot-order combine on every rank
    acc = np.zeros((T, H), np.float32)
    for s in range(top_k):
        acc = acc + joined[s::top_k].astype(np.float32) * \
            scores[:, s].astype(np.float16).astype(np.float32)[:, None]
    y = acc.astype(np.float16)
    q.put((rank, bool(np.array_equal(y.view(np.uint16), full.view(np.uint16)))))
    dist.barrier()
    dist.destroy_process_group()


def _run(worker, port: int) -> None:
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=90) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)], results


@pytest.mark.timeout(300)
def test_split_n_shards_join_bit_exact():
    _run(_split_n_worker, 29541)


@pytest.mark.timeout(300)
def test_expert_parallel_join_bit_exact():
    _run(_expert_parallel_worker, 29542)


def test_partition_helpers_reject_uneven_splits():
    from escha_mlx_b200 import sharding
    assert sharding.block_range(48, 3, 8) == (18, 24)
    assert sharding.expert_range(256, 7, 8) == (224, 256)
    with pytest.raises(ValueError, match="do not split evenly"):
        sharding.block_range(40, 0, 3)
    with pytest.raises(ValueError, match="do not split evenly"):
        sharding.expert_range(10, 0, 4)
    with pytest.raises(ValueError, match="outside"):
        sharding.block_range(8, 8, 8)

#!/usr/bin/env python
"""Benchmark of the coded-projection hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch M] [--impl b200|reference]

Workload (the reference's published dense configuration): one layer of a 27B-class dense model at
decode batch M (default 1) -- seven trellis-coded projections, hidden 5120:
q/k/v/o 2-bit 5120x{6144,1024,1024,5120}, gate/up 3-bit 5120x17408, down 3-bit
17408x5120 = 117,309,440 bytes of code per layer.  A step is one pass of the
layer (input transform, coded GEMV, output transform per projection, SwiGLU
before down) over one batch of synthetic fp16 activations.  Several layers'
worth of distinct weights are resident and rotated step to step so every step's
code stream misses L2 (the reference's bench/p0_gates.py:111-116 draws fresh
experts per call for the same reason).

Metric: compressed-weight GB/s = code bytes per step / time per step, whole job.
  value  -- inputs resident in HBM, steps replayed as CUDA graphs, CUDA events.
  e2e    -- same, through the public Python API with pinned HOST activations copied
            in and the layer output copied back out for every step inside the timed
            region (uploads and downloads on copy streams, pipelined against compute).
  roofline -- the coded GEMV kernel alone (algorithmic = code bytes per launch).
  cpu_baseline -- the CPU oracle (C port of the reference's NumPy path) on the
            host cores, bounded sample of the same layer.

At N > 1 GPUs the projections are split-N tensor parallel (whole 128-channel
output blocks per rank); the GEMV epilogue stores each rank's columns into every
GPU's gathered row through peer-mapped memory and a bounded barrier kernel closes
each launch (NCCL only carries set-up and the timing reduction); total work is
fixed, so scaling is "strong".

`--impl reference` times the reference's CPU implementation of the path: its
NumPy module cannot be installed on the GPU machine (it needs mlx), so this arm
runs the C port under oracle/ with every host thread.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

LAYER = (  # name, IC, OC, K  (escha_mlx_b200.synth.DENSE_LAYER_27B)
    ("q_proj", 5120, 6144, 2), ("k_proj", 5120, 1024, 2), ("v_proj", 5120, 1024, 2),
    ("o_proj", 5120, 5120, 2), ("gate_proj", 5120, 17408, 3), ("up_proj", 5120, 17408, 3),
    ("down_proj", 17408, 5120, 3),
)
LAYER_BYTES = sum(ic * oc * k // 8 for _, ic, oc, k in LAYER)
HIDDEN = 5120
L2_BYTES = 126 * 1024 * 1024
METRIC = "coded GEMV compressed-weight GB/s"


def measured_peak_tflops() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    except Exception:
        return 1590.0, "fallback"


def measured_peak_gbs() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# --------------------------------------------------------------------------- clocks

class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpus, active: bool = True) -> None:
        """`gpus`: one index or a list (rank 0 of a multi-rank run samples every GPU of the job
        with one nvidia-smi; the other ranks pass active=False and start nothing: one
        nvidia-smi per rank took seconds to come up on an 8-GPU box and sampled nothing)."""
        self.gpus = [gpus] if isinstance(gpus, int) else list(gpus)
        self.active = active
        self.rows: list[list[str]] = []
        self.proc = None
        self.closing = False

    def __enter__(self):
        if not self.active:
            return self
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20", "-i", ",".join(str(g) for g in self.gpus)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
            # the timed region starts only once the sampler delivers (bounded: 10 s)
            t0 = time.time()
            while not self.rows and time.time() - t0 < 10.0 and self.proc.poll() is None:
                time.sleep(0.01)
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            if self.closing:
                break
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 8:
                self.rows.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            if len(self.rows) < 2 * len(self.gpus):
                time.sleep(0.05)          # a region shorter than the sampling period: one more sample
            self.closing = True
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                "sw_power_cap"), r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- CPU legs

def cpu_layer_inputs(batch: int, seed: int = 1234):
    from escha_mlx_b200 import synth
    rng = np.random.default_rng(seed)
    projs = {}
    for name, ic, oc, k in LAYER:
        code, rin, rout = synth.coded_projection(rng, ic, oc, k)
        projs[name] = (code, rin.astype(np.float32), rout.astype(np.float32), k)
    x = synth.activations(rng, batch, HIDDEN)
    return projs, x


def cpu_layer_pass(oracle, projs, x):
    """One layer pass on the CPU oracle, same dataflow as the GPU step."""
    out = {}
    for name in ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj"):
        code, rin, rout, k = projs[name]
        out[name] = oracle.dense_linear(x, code, rin, rout, k)
    h = oracle.swiglu(np.concatenate([out["gate_proj"], out["up_proj"]], axis=-1))
    code, rin, rout, k = projs["down_proj"]
    out["down_proj"] = oracle.dense_linear(h, code, rin, rout, k)
    return out


def time_cpu(batch: int, min_seconds: float, max_passes: int):
    from oracle import escha_oracle as oracle
    oracle.set_num_threads(os.cpu_count() or 1)
    projs, x = cpu_layer_inputs(batch)
    cpu_layer_pass(oracle, projs, x)  # warm (LUT, page-in)
    passes, t0 = 0, time.perf_counter()
    while True:
        cpu_layer_pass(oracle, projs, x)
        passes += 1
        dt = time.perf_counter() - t0
        if dt >= min_seconds or passes >= max_passes:
            break
    return LAYER_BYTES * passes / dt / 1e9, passes, dt, oracle.num_threads()


def run_reference(args, rank: int) -> None:
    """`--impl reference`: the reference's CPU path (C port), rank 0 only."""
    if rank != 0:
        return
    from oracle import escha_oracle as oracle
    oracle.set_num_threads(os.cpu_count() or 1)
    projs, x = cpu_layer_inputs(args.batch)
    for _ in range(max(1, min(args.warmup, 3))):
        cpu_layer_pass(oracle, projs, x)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_layer_pass(oracle, projs, x)
    dt = time.perf_counter() - t0
    value = LAYER_BYTES * args.steps / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16 weights, f32 accumulate", "data": "synthetic",
        "config": workload_config(args, 1),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": oracle.num_threads(),
                         "kind": "port",
                         "sample": f"{args.steps} full passes of the layer (7 projections, "
                                   f"{LAYER_BYTES} code bytes each pass), batch {args.batch}"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, n_sets: int) -> dict:
    return {"workload": (f"dense27b_layer_prefill_m{args.batch}" if args.workload == "prefill"
                         else f"dense27b_layer_decode_b{args.batch}"),
            "projections": "q/k/v/o 2-bit 5120x{6144,1024,1024,5120}; gate/up 3-bit 5120x17408; "
                           "down 3-bit 17408x5120",
            "batch": args.batch, "code_bytes_per_step": LAYER_BYTES,
            "parallelism": (f"tp{args.gpus} split-N" if args.gpus > 1 else "single GPU"),
            "l2_policy": f"{n_sets} distinct weight sets rotated per step "
                         f"({n_sets * LAYER_BYTES // args.gpus} B per GPU > L2)"}


# --------------------------------------------------------------------------- MoE workloads

MOE_LAYERS = 40


def run_moe(args, rank: int, world: int, local_rank: int) -> None:
    """`--workload moe`: the published MoE configuration, one 35B-A3B-class MoE decode layer
    (256 routed 2-bit experts, top-8, hidden 2048, expert width 512, int8 shared expert)
    at `--tokens` tokens.  `--workload step`: the published full-step configuration, the 40-layer decode step at
    batch 32 with the int8 attention projections in front of every MoE block.
    A step is one layer (moe) or one 40-layer pass (step); 40 layers of distinct
    weights are resident so no step finds its experts in L2.  N > 1: expert parallel,
    the router, shared expert and int8 projections replicated."""
    import torch
    import torch.distributed as dist
    from escha_mlx_b200 import graphs, sharding, workloads

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    args.warmup = max(args.warmup, 3)
    global MOE_LAYERS
    if args.layers > 0:
        MOE_LAYERS = args.layers
    full_step = args.workload == "step"
    T = 32 if full_step else args.tokens
    cfg = workloads.MOE_35B
    er = sharding.expert_range(cfg["experts"], rank, world) if world > 1 else None
    pg = None
    if world > 1:
        # expert rows travel through peer-mapped memory straight from the kernel epilogue
        from escha_mlx_b200 import peer
        try:
            pg = peer.PeerGroup()
        except peer.PeerUnavailable as e:       # raised on every rank together
            pg = None
            if rank == 0:
                print(f"bench.py: {e}; falling back to NCCL all-gathers", file=sys.stderr)
    layers = workloads.moe_stack(MOE_LAYERS, device, attention=full_step, expert_range=er, rank=rank,
                                 peer_group=pg)
    gen = torch.Generator(device=device)
    gen.manual_seed(99)
    x0 = torch.randn((T, cfg["hidden"]), device=device, generator=gen).half()

    def norm(h):
        return torch.nn.functional.rms_norm(h, (h.shape[-1],), eps=1e-6)

    if full_step:
        def pass_(x):
            for layer in layers:
                x = norm(x + layer(x))      # residual + RMS norm between layers (framework ops)
            return x
        steps_per_replay = 1
    else:
        def pass_(x):
            out = None
            for layer in layers:
                out = layer(x)
            return out
        steps_per_replay = MOE_LAYERS
    g = graphs.GraphedCall(pass_, [x0])

    # bytes a step touches on this GPU (distinct routed experts of the shard + int8 + router)
    with torch.no_grad():
        if full_step:
            xs, routed = x0, 0
            for layer in layers:
                routed += layer.routed_experts(xs)
                xs = norm(xs + layer(xs))
        else:
            routed = sum(layer.routed_experts(x0) for layer in layers)
    torch.cuda.synchronize()
    lay = layers[0]
    code_bytes = routed * lay.expert_bytes                       # per 40-layer pass, this GPU
    other_bytes = MOE_LAYERS * (lay.int8_bytes + lay.router_bytes)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    replays = max(1, -(-args.steps // steps_per_replay))
    steps = replays * steps_per_replay
    stream = torch.cuda.current_stream()
    for _ in range(max(1, -(-args.warmup // steps_per_replay))):
        g.replay()
    sync_all()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(list(range(world)) if world > 1 else local_rank, active=(rank == 0)) as clocks:
        sync_all()
        ev0.record(stream)
        for _ in range(replays):
            g.replay()
        ev1.record(stream)
        sync_all()
    ms_total = ev0.elapsed_time(ev1)

    x_host = torch.randn((T, cfg["hidden"])).half().pin_memory()
    y_host = torch.empty((T, cfg["hidden"]), dtype=torch.float16).pin_memory()
    for _ in range(2):
        y_host.copy_(g(x_host), non_blocking=True)
    sync_all()
    ee0, ee1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ee0.record(stream)
    for _ in range(replays):
        y_host.copy_(g(x_host), non_blocking=True)
    ee1.record(stream)
    sync_all()
    ms_e2e = ee0.elapsed_time(ee1)

    if world > 1:
        t = torch.tensor([ms_total, ms_e2e, float(code_bytes),
                          float(pg.status()) if pg is not None else 0.0], device=device,
                         dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, ms_e2e, max_code, gave_up = (float(v) for v in t.tolist())
        tot = torch.tensor([float(code_bytes)], device=device, dtype=torch.float64)
        dist.all_reduce(tot)
        sum_code = float(tot.item())
    else:
        max_code = sum_code = float(code_bytes)

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        tokens_per_s = T * steps / (ms_total * 1e-3)
        passes = replays
        gbs = (sum_code + world * other_bytes) * passes / (ms_total * 1e-3) / 1e9
        line = {
            "metric": "MoE decode-layer tokens/s" if not full_step else "MoE decode-step tokens/s",
            "value": tokens_per_s, "unit": "tokens/s", "n_gpus": world, "steps": steps,
            "warmup": args.warmup, "ms_per_step": ms_total / steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": "f16 weights, f32 accumulate", "data": "synthetic",
            "config": {
                "workload": (f"moe35b_step_decode_b{T}" if full_step else f"moe35b_layer_decode_t{T}"),
                "experts": "256 routed 2-bit (2048->1024, 512->2048), top-8, int8 shared expert"
                           + ("; int8 q/k/v/o 2048->{4096,512,512}, 4096->2048" if full_step else ""),
                "tokens": T, "layers_resident": MOE_LAYERS,
                "parallelism": (f"ep{world}, " + ("expert rows stored to every GPU from the kernel "
                                                  "epilogue (peer memory)" if pg is not None
                                                  else "NCCL all-gather of expert rows"))
                if world > 1 else "single GPU",
                "routed_experts_per_layer_avg": routed / MOE_LAYERS,
                "max_over_mean_code_bytes_per_gpu": (max_code * world / sum_code) if sum_code else None,
                "l2_policy": f"{MOE_LAYERS} layers of distinct weights "
                             f"({int(code_bytes + other_bytes)} B touched per pass per GPU > L2)"},
            "e2e": {"value": T * steps / (ms_e2e * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": T * cfg["hidden"] * 2 // steps_per_replay,
                    "d2h_bytes_per_step": T * cfg["hidden"] * 2 // steps_per_replay},
            "touched_gb_per_s": gbs, "pct_of_hbm_peak": 100.0 * gbs / (peak * world),
            # per layer: router, two expert legs, the shared expert's gate/up and the tail kernel
            # (+ the cross-GPU barrier under expert parallelism; + int8 q/k/v in one launch and o
            # in another for the full step)
            "gpu_launches": (5 + (1 if pg is not None else 0) + (2 if full_step else 0)) * MOE_LAYERS * passes,
            "roofline": {"bound": "hbm", "achieved": gbs / world, "peak": peak, "unit": "GB/s",
                         "frac": gbs / world / peak, "traffic": None,
                         "kernel": "whole step: bytes of routed expert streams, int8 matrices and "
                                   "router weights touched per GPU / step time",
                         "peak_source": f"MEASURED_PEAKS.json hbm_gbs ({peak_kind})"},
            "clocks": clocks.summary(),
        }
        if world > 1:
            line["peer_barrier_gave_up"] = bool(gave_up)   # must be false for a valid run
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.cuda.synchronize()
        g.close()
        for layer in layers:
            layer.block._peer_bufs = {}
        del layers, pass_, g
        if pg is not None:
            pg.close()
        dist.barrier()
        dist.destroy_process_group()
        sys.stdout.flush()
        sys.stderr.flush()


def moe_legs(device, token_counts=(1, 8, 64), replays: int = 10) -> dict:
    """Second half of the headline metric inside the default run: one 35B-A3B-class MoE
    decode layer at 1, 8 and 64 tokens (the `--workload moe` measurement, shortened): per
    token count the time per layer, the bytes of the distinct routed experts it streams and
    that rate as a fraction of the measured HBM peak."""
    import torch
    from escha_mlx_b200 import graphs, workloads
    cfg = workloads.MOE_35B
    layers = workloads.moe_stack(MOE_LAYERS, device)
    peak, _ = measured_peak_gbs()
    out = {"metric": "MoE decode-layer tokens/s", "layers_resident": MOE_LAYERS,
           "workload": "moe35b_layer_decode_t{1,8,64} (see --workload moe)"}
    for tokens in token_counts:
        gen = torch.Generator(device=device)
        gen.manual_seed(99)
        x0 = torch.randn((tokens, cfg["hidden"]), device=device, generator=gen).half()

        def pass_(x):
            y = None
            for layer in layers:
                y = layer(x)
            return y
        with torch.no_grad():
            routed = sum(layer.routed_experts(x0) for layer in layers)
        g = graphs.GraphedCall(pass_, [x0])
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (replays * MOE_LAYERS)
        g.close()
        lay = layers[0]
        code_bytes = routed * lay.expert_bytes / MOE_LAYERS
        touched = code_bytes + lay.int8_bytes + lay.router_bytes
        out[f"t{tokens}"] = {"us_per_layer": us, "tokens_per_s": tokens / (us * 1e-6),
                             "distinct_expert_code_bytes_per_layer": code_bytes,
                             "touched_gb_per_s": touched / (us * 1e-6) / 1e9,
                             "frac": touched / (us * 1e-6) / 1e9 / peak}
    return out


def c1_leg(device, reps: int = 5, e2e: bool = False) -> dict:
    """The single dense coded projection of the reference's own gate (4096x4096, 2-bit, one
    row; escha_mlx bench/p0_gates.py:111-118): 4 MiB of code, below launch latency and smaller
    than L2, so two figures, both from CUDA-graph replays of 128 back-to-back launches:
    HBM-resident (64 distinct weight buffers = 256 MiB rotated, every launch misses L2) and
    L2-resident (one buffer)."""
    import torch
    from escha_mlx_b200 import dense, graphs
    IC = OC = 4096
    K, nbuf, launches = 2, 64, 128
    gen = torch.Generator(device=device)
    gen.manual_seed(4096)

    def vec(n):
        scale = torch.randn(n, device=device, generator=gen).abs() * 0.02 + 1e-3
        sign = torch.randint(0, 2, (n,), device=device, generator=gen).float() * 2 - 1
        return (scale * sign).half().float()
    rin, rout = vec(IC), vec(OC)
    lins = [dense.EschaLinear(dense.EschaWeight.from_device(
        torch.randint(-2**31, 2**31 - 1, (IC // 16, OC // 16, 8 * K), dtype=torch.int32,
                      device=device, generator=gen), rin, rout)) for _ in range(nbuf)]
    x = torch.randn((1, IC), device=device, generator=gen).half()
    peak, _ = measured_peak_gbs()
    out = {"workload": "dense_c1_4096x4096_k2_b1", "code_bytes": IC * OC * K // 8,
           "launches_per_replay": launches}
    for name, pick in (("hbm_resident", lambda i: lins[i % nbuf]), ("l2_resident", lambda i: lins[0])):
        g = graphs.GraphedCall(lambda xx, pick=pick: [pick(i)(xx) for i in range(launches)][-1], [x])
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3 / launches)
        g.close()
        us = statistics.median(times)
        gbs = IC * OC * K // 8 / (us * 1e-6) / 1e9
        out[name] = {"us_per_launch": us, "gb_per_s": gbs, "frac_of_hbm_peak": gbs / peak,
                     "weight_buffers": nbuf if name == "hbm_resident" else 1}
    if e2e:
        # through the module call with a pinned host row in and the host result out, every
        # launch (one single-launch graph per weight buffer, copies on the launching stream)
        gs = [graphs.GraphedCall(lambda xx, lin=lin: lin(xx), [x]) for lin in lins]
        xh = torch.randn((1, IC)).half().pin_memory()
        yh = torch.empty((1, OC), dtype=torch.float16).pin_memory()
        for i in range(8):
            yh.copy_(gs[i % nbuf](xh), non_blocking=True)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n = 4 * launches
        e0.record()
        for i in range(n):
            yh.copy_(gs[i % nbuf](xh), non_blocking=True)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / n
        for g in gs:
            g.close()
        out["e2e"] = {"us_per_launch": us, "gb_per_s": IC * OC * K // 8 / (us * 1e-6) / 1e9,
                      "launches": n, "h2d_bytes_per_step": IC * 2, "d2h_bytes_per_step": OC * 2}
    return out


def run_c1(args, rank: int, world: int, local_rank: int) -> None:
    """`--workload c1`: the reference's simplest configuration as a line of its own.  A step
    is one launch of the 4096x4096 2-bit projection at one row (input transform, GEMV and
    output transform in the launch), replayed 128 at a time from a CUDA graph; `value` is the
    HBM-resident figure (64 rotating weight buffers), the L2-resident one rides along.  The
    path does not shard at this size: N > 1 runs independent replicas (rank 0 reports its own
    time; nothing is exchanged)."""
    import torch
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    reps = max(5, args.repeats)
    with ClockSampler(local_rank, active=(rank == 0)) as clocks:
        leg = c1_leg(device, reps=reps, e2e=True)
    if rank != 0:
        return
    peak, peak_kind = measured_peak_gbs()
    hbm, l2 = leg["hbm_resident"], leg["l2_resident"]
    launches = leg["launches_per_replay"] * reps
    line = {
        "metric": METRIC, "value": hbm["gb_per_s"] * world, "unit": "GB/s", "n_gpus": world,
        "steps": launches, "warmup": 3 * leg["launches_per_replay"],
        "ms_per_step": hbm["us_per_launch"] * 1e-3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 weights, f32 accumulate",
        "data": "synthetic",
        "config": {"workload": leg["workload"], "code_bytes_per_step": leg["code_bytes"],
                   "parallelism": "single GPU" if world == 1 else f"{world} independent replicas",
                   "l2_policy": "value: 64 weight buffers (256 MiB) rotated, every launch misses L2; "
                                "l2_resident: one buffer"},
        "l2_resident": l2,
        "e2e": {"value": leg["e2e"]["gb_per_s"] * world, "unit": "GB/s",
                "h2d_bytes_per_step": leg["e2e"]["h2d_bytes_per_step"],
                "d2h_bytes_per_step": leg["e2e"]["d2h_bytes_per_step"],
                "note": "one graph launch per step with the host row copied in and the result "
                        "copied out on the same stream: bound by three enqueues per step on the host"},
        "gpu_launches": 2 * launches,
        "roofline": {"bound": "hbm", "achieved": hbm["gb_per_s"], "peak": peak, "unit": "GB/s",
                     "frac": hbm["gb_per_s"] / peak, "traffic": None,
                     "kernel": "gemv_mma_kernel<2,1> (coded GEMV + fused transforms), one launch per step",
                     "peak_source": f"MEASURED_PEAKS.json hbm_gbs ({peak_kind})"},
        "clocks": clocks.summary(),
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU side

def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="dense", choices=["dense", "prefill", "moe", "step", "c1"],
                    help="dense: 27B-class layer at decode batch --batch (default, the headline); "
                         "prefill: the same layer at 256 rows on the tcgen05 GEMM, reported in "
                         "TFLOP/s; moe: one 35B-A3B-class MoE layer at --tokens; step: 40-layer "
                         "MoE decode step at batch 32; c1: the single 4096x4096 2-bit GEMV at one row, "
                         "HBM- and L2-resident")
    ap.add_argument("--tokens", type=int, default=8, help="tokens per step for --workload moe")
    ap.add_argument("--layers", type=int, default=0,
                    help="resident MoE layers for --workload moe/step (default 40; fewer only for "
                         "profiler captures, where less device memory must be saved and restored)")
    ap.add_argument("--cpu-seconds", type=float, default=10.0,
                    help="bounded CPU-baseline sample (rank 0, N=1)")
    ap.add_argument("--repeats", type=int, default=5,
                    help="how many times the --steps region is timed (median reported)")
    ap.add_argument("--wave", type=int, default=1,
                    help="1: split factors of a joint launch chosen for the launch as a whole "
                         "(dense.project_many(one_wave=True)); 0: every projection keeps the factor "
                         "it has alone (bit-identical to separate calls)")
    ap.add_argument("--group", default="layer", choices=["layer", "model"],
                    help="launch grouping at small batch: layer = the projections that read the "
                         "step input share one launch per rate (3 launches per step; 2 with the persistent "
                         "kernel, which mixes rates); model = q/k/v | o | "
                         "gate/up | SwiGLU+down (4 launches)")
    ap.add_argument("--no-moe-leg", action="store_true",
                    help="skip the short MoE-layer measurement appended to the default line")
    ap.add_argument("--only", default=None,
                    help="profiling aid: run just this projection's GEMV for --steps launches")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.workload == "c1":
        run_c1(args, rank, world, local_rank)
        return
    if args.workload in ("moe", "step"):
        run_moe(args, rank, world, local_rank)
        return
    prefill = args.workload == "prefill"
    if prefill and args.batch == 1:
        args.batch = 256

    import torch
    import torch.distributed as dist
    from escha_mlx_b200 import dense, graphs, msl

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path (use --impl reference "
                         "for the CPU baseline)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    args.warmup = max(args.warmup, 3)
    M = args.batch

    # From 32 rows on (the tcgen05 kernel) the rows are the independent unit: every rank holds the
    # full weights and runs its own `--batch` rows, with nothing to exchange (weak scaling: the
    # job's batch is N x --batch).  Below that, split-N tensor parallelism (strong scaling).
    replica = world > 1 and M >= 32
    shards = 1 if replica else world
    # weight sets: enough distinct layers that a step's per-GPU code bytes never sit in L2
    per_gpu = LAYER_BYTES // shards
    n_sets = max(2, -(-3 * L2_BYTES // per_gpu))
    gen = torch.Generator(device=device)
    gen.manual_seed(1234 + rank)

    def make_weight(ic: int, oc: int, k: int) -> dense.EschaWeight:
        oc_local = oc // shards
        code = torch.randint(-2**31, 2**31 - 1, (ic // 16, oc_local // 16, 8 * k),
                             dtype=torch.int32, device=device, generator=gen)

        def vec(n):
            scale = torch.randn(n, device=device, generator=gen).abs() * 0.02 + 1e-3
            sign = torch.randint(0, 2, (n,), device=device, generator=gen).float() * 2 - 1
            return (scale * sign).half().float()   # f16-representable, held as f32
        return dense.EschaWeight.from_device(code, vec(ic), vec(oc_local))

    for _, ic, oc, _ in LAYER:
        if (oc // 128) % shards:
            raise SystemExit(f"{oc // 128} output blocks do not split over {shards} GPUs")
    sets = [{name: dense.EschaLinear(make_weight(ic, oc, k)) for name, ic, oc, k in LAYER}
            for _ in range(n_sets)]

    ROW = sum(oc for _, _, oc, _ in LAYER)     # gathered halves per activation row and layer
    pg, arena, gathered = None, None, []
    if world > 1 and not replica:
        # split-N tensor parallel: the GEMV epilogue stores each rank's columns into every
        # GPU's gathered row (peer-mapped memory), one bounded cross-GPU barrier per launch.
        # One buffer set per weight set: a buffer is rewritten n_sets barriers later.
        from escha_mlx_b200 import peer, sharding
        try:
            pg = peer.PeerGroup()
            arena = pg.empty((n_sets * M * ROW,), torch.float16)
        except peer.PeerUnavailable as e:       # raised on every rank together
            pg = arena = None
            if rank == 0:
                print(f"bench.py: {e}; falling back to NCCL all-gathers", file=sys.stderr)
        for i in range(n_sets if pg is not None else 0):
            off, bufs = i * M * ROW, {}
            for name, _, oc, _ in LAYER:
                bufs[name] = arena.carve(off, (M, oc))
                off += M * oc
            gathered.append(bufs)

    def tp_launch(layer, bufs, names, x, x_up=None, join=True):
        """One fused launch of the named projections' shards into their gathered buffers,
        closed by the cross-GPU barrier unless a later launch's barrier covers it (a rank's
        barrier kernel runs after all its earlier launches, so one barrier completes the
        gathers of every launch before it)."""
        ws = [layer[n]._w for n in names]
        fuse_in = M <= msl.FUSE_INPUT_MAX_ROWS
        mode = (msl.INPUT_SWIGLU if x_up is not None else msl.INPUT_RAW) if fuse_in \
            else msl.INPUT_TRANSFORMED
        xs = None
        if not fuse_in:   # one launch: SwiGLU (if any) and every projection's input transform
            xs = msl.dense_scaled_had_many(x.contiguous(), [w.rin for w in ws], msl.RS,
                                           up=None if x_up is None else x_up.contiguous())
            x_up = None
        outs = msl.coded_projections(
            x if fuse_in else xs[0], [w.code for w in ws], [w.rin for w in ws] if fuse_in else None,
            [w.rout for w in ws], ws[0].K, ws[0].IC, [w.OC for w in ws], input_mode=mode,
            x_up=x_up, rs=msl.RS, xs=xs, gather=[(bufs[n], rank * w.OC) for n, w in zip(names, ws)],
            splits=msl.wave_splits(ws[0].IC, [w.OC for w in ws]) if args.wave else None)
        if join:
            pg.barrier()
        return outs

    tc_shards = False   # from 32 rows on ranks are row replicas (above); shards stay on the GEMV
    # launch grouping of the fused small-batch path: "layer" follows this step's own data flow
    # (q/k/v, o, gate, up all read the step input: one launch; SwiGLU + down: a second);
    # "model" keeps the four launches a transformer layer with attention between q/k/v and o
    # needs (q/k/v | o | gate/up | SwiGLU + down)
    joint_launches = args.group == "layer" and (world == 1 or replica) and M <= msl.FUSE_INPUT_MAX_ROWS

    def layer_step(layer, x, bufs=None, joint=None):
        joint = joint_launches if joint is None else joint
        if world > 1 and not replica and (pg is None or tc_shards):
            # NCCL form of the same exchange: an all-gather of every projection's f16 output
            # (also from 32 rows on, where each rank's shard runs on the tcgen05 kernel, whose
            # epilogue does not store to peers; measured on 2 GPUs: 16 rows 178 us through the
            # GEMV's peer stores, 32 rows 275 us that way and 247 us this way)
            ag = sharding.all_gather_columns
            q, k, v = (ag(t) for t in dense.project_many(
                [layer["q_proj"], layer["k_proj"], layer["v_proj"]], x))
            o = ag(layer["o_proj"](x))
            g, u = (ag(t) for t in dense.project_pair(layer["gate_proj"], layer["up_proj"], x))
            d = ag(dense.swiglu_project(layer["down_proj"], g, u))
            return q, k, v, o, d
        if world > 1 and not replica:
            # one launch (and one cross-GPU join) per rate among the projections of the input
            # q/k/v/o and gate/up read the same input: nobody needs q/k/v/o gathered before
            # gate/up has run, so the two launches share the second one's barrier
            q, k, v, o = tp_launch(layer, bufs, ("q_proj", "k_proj", "v_proj", "o_proj"), x, join=False)
            g, u = tp_launch(layer, bufs, ("gate_proj", "up_proj"), x)
            (d,) = tp_launch(layer, bufs, ("down_proj",), g, u)   # full-width SwiGLU input
            return q, k, v, o, d
        if joint:
            # every projection that reads the step's input in ONE launch (2-bit and 3-bit
            # streams side by side), SwiGLU + down in a second
            q, k, v, o, g, u = dense.project_many(
                [layer[n] for n in ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj")], x,
                one_wave=args.wave)
        else:
            q, k, v = dense.project_many([layer["q_proj"], layer["k_proj"], layer["v_proj"]], x)
            o = layer["o_proj"](x)
            g, u = dense.project_pair(layer["gate_proj"], layer["up_proj"], x)
        d = dense.swiglu_project(layer["down_proj"], g, u)
        return q, k, v, o, d

    # launches of this library's kernels per step: fused small-batch path = q/k/v, o,
    # gate/up, swiglu+down (4); larger batches add the separate input transforms
    if M <= msl.FUSE_INPUT_MAX_ROWS:
        # joint: one launch for all rates (persistent kernel) or one per rate
        per_step = (2 if msl.mixed_rates_supported() else 3) if joint_launches else 4
        launches_per_step = per_step if world == 1 else 5   # 3 fused GEMV + 2 peer barriers
    elif msl.use_prefill_kernel(M) and (world == 1 or replica):
        # four input-transform launches (q/k/v, o, gate/up, SwiGLU + down), the tcgen05 GEMMs,
        # and a plane sum + output transform for every projection split more than 4 ways along K
        from escha_mlx_b200._lib import lib as _lib
        def split(ic, oc):
            # splits of up to 4 are summed inside the GEMM by a cluster of CTAs; more need a
            # plane-sum launch
            return _lib.escha_coded_gemm_tc_splits(ic, oc, 0) > 4
        # a rank holds 1/world of every projection's output channels (split-N)
        dims = {name: (ic, oc // shards) for name, ic, oc, _k in LAYER}
        qkv_oc = sum(dims[n][1] for n in ("q_proj", "k_proj", "v_proj"))
        # q/k/v share one GEMM launch (their column blocks fit one wave) and, up to 128 rows,
        # one plane-sum launch
        gemms = 1 + 1 + 2 + 1
        sums = ((1 if M <= 128 else 3) if split(HIDDEN, qkv_oc) else 0) + sum(
            1 for n in ("o_proj", "gate_proj", "up_proj", "down_proj") if split(*dims[n]))
        launches_per_step = 4 + gemms + sums
    else:
        # q/k/v 1+1, o 1+1, gate/up 1+1, SwiGLU + down 1+1 (+ 4 barriers)
        launches_per_step = 8 if world == 1 else 12

    x0 = torch.randn((M, HIDDEN), device=device, generator=gen).half()

    # Split-N parity, once, before any timing: on a small projection every rank builds the
    # same full weight, runs its shard through the exchange the timed steps use and compares
    # the gathered rows with the unsharded product of the same kernel, bit for bit.
    tp_parity = None
    if world > 1 and not replica:
        pgen = torch.Generator(device=device)
        pgen.manual_seed(777)
        pic, poc, pk = 1024, 128 * world * 2, 2
        pcode = torch.randint(-2**31, 2**31 - 1, (pic // 16, poc // 16, 8 * pk), dtype=torch.int32,
                              device=device, generator=pgen)
        pvec = lambda n: (torch.randn(n, device=device, generator=pgen) * 0.02).half().float()
        full = dense.EschaWeight.from_device(pcode, pvec(pic), pvec(poc))
        px = torch.randn((1, pic), device=device, generator=pgen).half()
        want = dense.EschaLinear(full)(px)
        mine = full.shard_out(rank, world)
        if pg is not None:
            pbuf = pg.empty((1, poc), torch.float16)
            msl.coded_projections(px, [mine.code], [mine.rin], [mine.rout], pk, pic, [mine.OC],
                                  input_mode=msl.INPUT_RAW, rs=msl.RS,
                                  gather=[(pbuf, rank * mine.OC)])
            pg.barrier()
            got = pbuf.local
        else:
            from escha_mlx_b200 import sharding as _sh
            got = _sh.all_gather_columns(dense.EschaLinear(mine)(px))
        torch.cuda.synchronize()
        same = torch.tensor([1.0 if torch.equal(got, want) else 0.0], device=device)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        tp_parity = "bit-exact" if same.item() == 1.0 else "MISMATCH"

    if args.only:
        # profiling aid: K launches of one projection's product kernel, rotating weight sets
        lin = [s[args.only] for s in sets]
        ic = lin[0]._w.IC
        xh = msl.dense_scaled_had(torch.randn((M, ic), device=device, generator=gen).half(),
                                  lin[0]._w.rin, msl.RS)
        for i in range(args.warmup + args.steps):
            w = lin[i % n_sets]._w
            if msl.use_prefill_kernel(M):
                msl.dense_gemm_tc(xh, w.code, w.K, w.IC, w.OC)
            else:
                msl.dense_gemm_rows_direct_out(xh, w.code, w.rout, w.K, w.IC, w.OC, 8, msl.RS)
        torch.cuda.synchronize()
        print(json.dumps({"only": args.only, "rows": M, "launches": args.steps}))
        return

    step_graphs = [graphs.GraphedCall(
        lambda x, L=L, i=i: layer_step(L, x, gathered[i] if gathered else None), [x0])
        for i, L in enumerate(sets)]

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    stream = torch.cuda.current_stream()
    for i in range(args.warmup):
        step_graphs[i % n_sets].replay()
    sync_all()

    # ---- value: resident inputs, device-timed -----------------------------------------------
    # the K-step region is timed `--repeats` times back to back; the line reports the median
    # repeat and how far the first and the last lie from it (drift control)
    rep_ms = []
    with ClockSampler(list(range(world)) if world > 1 else local_rank, active=(rank == 0)) as clocks:
        for _ in range(max(1, args.repeats)):
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            sync_all()
            ev0.record(stream)
            for i in range(args.steps):
                step_graphs[i % n_sets].replay()
            ev1.record(stream)
            sync_all()
            rep_ms.append(ev0.elapsed_time(ev1))
    if world > 1:   # every rank must pick the same repeat: rank-wise maxima first
        t = torch.tensor(rep_ms, device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        rep_ms = [float(v) for v in t.tolist()]
    ms_total = statistics.median(rep_ms)

    # ---- e2e: pinned host activations in, layer output back out, every step -------------------
    # A serving loop pipelines its copies: step i+1's input is uploaded and step i's output is
    # downloaded on two copy streams while step i / i+1 computes.  Consecutive steps use
    # different graphs (weight sets), hence different static input and output buffers, so the
    # only ordering needed is per graph: upload after its previous replay has finished, replay
    # after the upload, download after the replay.
    x_host = [torch.randn((M, HIDDEN)).half().pin_memory() for _ in range(4)]
    y_host = [torch.empty((M, HIDDEN), dtype=torch.float16).pin_memory() for _ in range(n_sets)]
    up, down = torch.cuda.Stream(), torch.cuda.Stream()
    uploaded = [torch.cuda.Event() for _ in range(n_sets)]
    computed = [torch.cuda.Event() for _ in range(n_sets)]
    fetched = [torch.cuda.Event() for _ in range(n_sets)]

    def e2e_step(i):
        j = i % n_sets
        g = step_graphs[j]
        with torch.cuda.stream(up):
            up.wait_event(computed[j])            # the graph's previous replay has read its input
            g.inputs[0].copy_(x_host[i % 4], non_blocking=True)
            uploaded[j].record(up)
        stream.wait_event(uploaded[j])
        stream.wait_event(fetched[j])             # the previous output of this graph was downloaded
        g.replay()
        computed[j].record(stream)
        with torch.cuda.stream(down):
            down.wait_event(computed[j])
            y_host[j].copy_(g.outputs[4], non_blocking=True)
            fetched[j].record(down)

    for j in range(n_sets):
        computed[j].record(stream)
        fetched[j].record(stream)
    for i in range(args.warmup):
        e2e_step(i)
    sync_all()
    ee0, ee1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ee0.record(stream)
    up.wait_stream(stream)                        # no upload starts before the clock does
    for i in range(args.steps):
        e2e_step(i)
    stream.wait_stream(down)                      # the last output has reached the host buffer
    ee1.record(stream)
    sync_all()
    ms_e2e = ee0.elapsed_time(ee1)
    out = step_graphs[0].outputs

    # ---- roofline leg: the coded GEMV kernel alone --------------------------------------------
    tensor_leg = msl.use_prefill_kernel(M)

    def gemv_only(layer, xs):
        outs = []
        for name, _, _, _ in LAYER:
            w = layer[name]._w
            if tensor_leg:   # the tcgen05 GEMM alone (f32 mid out)
                outs.append(msl.dense_gemm_tc(xs[w.IC], w.code, w.K, w.IC, w.OC))
            else:
                outs.append(msl.dense_gemm_rows_direct_out(xs[w.IC], w.code, w.rout, w.K, w.IC,
                                                           w.OC, 8, msl.RS))
        return outs

    xs = {ic: msl.dense_scaled_had(torch.randn((M, ic), device=device, generator=gen).half(),
                                   sets[0]["q_proj" if ic == HIDDEN else "down_proj"]._w.rin, msl.RS)
          for ic in (HIDDEN, 17408)}
    gemv_graphs = [graphs.GraphedCall(lambda L=L: gemv_only(L, xs), []) for L in sets]
    for g in gemv_graphs:
        g.replay()
    sync_all()
    er0, er1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(1, args.steps)
    er0.record(stream)
    for i in range(reps):
        gemv_graphs[i % n_sets].replay()
    er1.record(stream)
    sync_all()
    ms_gemv = er0.elapsed_time(er1)

    def prefill_leg(rows: int = 256, steps: int = 12) -> dict:
        """The same layer at 256 rows on the tcgen05 GEMM (`--workload prefill`, shortened)."""
        xp = torch.randn((rows, HIDDEN), device=device, generator=gen).half()
        # launch grouping of the prefill workload (q/k/v | o | gate/up | SwiGLU + down), whatever
        # grouping the batch-1 step of this run uses
        pgraphs = [graphs.GraphedCall(lambda xx, L=L: layer_step(L, xx, joint=False), [xp]) for L in sets]
        for gph in pgraphs:
            gph.replay()
        torch.cuda.synchronize()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record(stream)
        for i in range(steps):
            pgraphs[i % n_sets].replay()
        p1.record(stream)
        torch.cuda.synchronize()
        ms = p0.elapsed_time(p1) / steps
        for gph in pgraphs:
            gph.close()
        tpeak, _ = measured_peak_tflops()
        tf = 2.0 * rows * sum(ic * oc for _, ic, oc, _ in LAYER) / (ms * 1e-3) / 1e12
        return {"workload": f"dense27b_layer_prefill_m{rows}", "ms_per_step": ms, "tflops": tf,
                "frac_of_bf16_peak": tf / tpeak}

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ms_total, ms_e2e, ms_gemv = (max_over_ranks(v) for v in (ms_total, ms_e2e, ms_gemv))
    barrier_gave_up = max_over_ranks(float(pg.status())) if (world > 1 and pg is not None) else 0.0

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        # replicas: every rank streams the whole layer for its own rows, so the job's bytes
        # and rows per step are `world` times one rank's
        job = world if replica else 1
        value = job * LAYER_BYTES * args.steps / (ms_total * 1e-3) / 1e9
        e2e = job * LAYER_BYTES * args.steps / (ms_e2e * 1e-3) / 1e9
        launches = 7 * reps
        achieved = (LAYER_BYTES / shards) * reps / (ms_gemv * 1e-3) / 1e9   # per GPU
        # DRAM bytes per GEMV launch from the ncu captures summarised under profiles/
        # (gemv_mma_gate_proj_k3_m1.md: 33,567,744 B read for 33,423,360 B of code, 1.004x;
        # gemv_mma_q_proj_k2_m1.md: 7,962,880 B for 7,864,320 B, 1.013x; no writes to DRAM).
        # Traffic grows with the code bytes, so the other projections are scaled by their rate's
        # factor; this is the average over the seven launches timed above, per GPU.
        traffic = (sum(ic * oc * k // 8 * (1.013 if k == 2 else 1.004) for _, ic, oc, k in LAYER)
                   / 7 / shards) if M == 1 else None
        flops_step = 2.0 * job * M * sum(ic * oc for _, ic, oc, _ in LAYER)
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_total / args.steps,
            "higher_is_better": True, "scaling": "weak" if replica else "strong", "vs_baseline": None,
            "dtype": "f16 weights, f32 accumulate", "data": "synthetic",
            "config": workload_config(args, n_sets),
            "pct_of_hbm_peak": 100.0 * value / (peak * world),
            "tokens_per_s": job * M * args.steps / (ms_total * 1e-3),
            "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": M * HIDDEN * 2,
                    "d2h_bytes_per_step": M * HIDDEN * 2},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic,
                         "kernel": "gemv_mma_kernel (coded GEMV + fused output transform)",
                         "launches_timed": launches,
                         "avg_launch_us": ms_gemv * 1e3 / launches,
                         "algorithmic_bytes_per_launch_avg": LAYER_BYTES / shards / 7,
                         "timed": "seven projections launched one by one (CUDA-graph replays)",
                         "peak_source": f"MEASURED_PEAKS.json hbm_gbs ({peak_kind})"},
            "clocks": clocks.summary(),
            "repeats": {"n": len(rep_ms), "ms_per_step": [m / args.steps for m in rep_ms],
                        "reported": "median",
                        "first_vs_median_pct": 100.0 * (rep_ms[0] / ms_total - 1.0),
                        "last_vs_median_pct": 100.0 * (rep_ms[-1] / ms_total - 1.0)},
        }
        if world == 1 and M <= msl.FUSE_INPUT_MAX_ROWS:
            # at these batch sizes the timed step is nothing but four launches of this kernel
            # (q/k/v, o, gate/up, SwiGLU+down, transforms fused), so the step itself is the
            # kernel's live measurement; the one-by-one leg above stays for comparison with
            # the per-projection profiler captures
            sep = dict(line["roofline"])
            line["roofline"].update({
                "achieved": value, "frac": value / peak,
                "launches_timed": launches_per_step * args.steps,
                "avg_launch_us": ms_total * 1e3 / (launches_per_step * args.steps),
                "algorithmic_bytes_per_launch_avg": LAYER_BYTES / launches_per_step,
                "traffic": (traffic * 7 / launches_per_step) if traffic else None,
                "timed": f"the timed steps themselves: {launches_per_step} fused launches per step",
                "traffic_source": "scaled from the captures under profiles/ (not measured in this run)",
                "separate_launches": {k: sep[k] for k in ("achieved", "frac", "launches_timed",
                                                          "avg_launch_us", "traffic")}})
        if not tensor_leg:
            # second fraction: warp instructions the decode cannot do without (41 per 16x16
            # tile at 2 bits, 46 at 3: profiles/issue_rates.md) over the issue slots the step
            # had, one per sub-partition and clock at the sampled SM clock
            tiles = {k: sum(ic * oc // 256 for _, ic, oc, kk in LAYER if kk == k) for k in (2, 3)}
            need = (41 * tiles[2] + 46 * tiles[3]) / shards
            mhz = line["clocks"].get("sm_mhz") or 1965.0
            have = 4 * 148 * mhz * 1e6 * (ms_total * 1e-3 / args.steps)
            line["roofline"]["issue_frac"] = need / have
            line["roofline"]["issue_note"] = ("minimal decode warp instructions per step / issue "
                                              "slots in the step time (4 per SM per clock)")
        if world > 1 and replica:
            line["config"]["parallelism"] = f"{world} row replicas (full weights per GPU, no exchange)"
            line["config"]["global_batch"] = world * M
        elif world > 1:
            line["config"]["exchange"] = ("GEMV epilogue stores into every GPU's gathered row "
                                          "(peer memory) + barrier kernel"
                                          if pg is not None and not tc_shards
                                          else "NCCL all-gather per projection")
            line["peer_barrier_gave_up"] = bool(barrier_gave_up)   # must be false for a valid run
            line["tp_parity"] = tp_parity
        if tensor_leg:
            tpeak, tkind = measured_peak_tflops()
            tf = flops_step / world * reps / (ms_gemv * 1e-3) / 1e12      # per GPU
            line["tflops"] = flops_step * args.steps / (ms_total * 1e-3) / 1e12
            line["roofline"] = {
                "bound": "tensor", "achieved": tf, "peak": tpeak, "unit": "TFLOP/s",
                "frac": tf / tpeak, "traffic": None,
                "kernel": "gemm_tcm_kernel (trellis decode into tensor memory + tcgen05.mma)",
                "launches_timed": launches, "avg_launch_us": ms_gemv * 1e3 / launches,
                "algorithmic_flops_per_launch_avg": flops_step / world / 7,
                "peak_source": f"MEASURED_PEAKS.json bf16_tflops burst ({tkind}); f16 and bf16 "
                               "share the tensor rate"}
        if prefill:
            line.update({"metric": "prefill coded GEMM TFLOP/s", "value": line["tflops"],
                         "unit": "TFLOP/s",
                         "e2e": {"value": flops_step * args.steps / (ms_e2e * 1e-3) / 1e12,
                                 "unit": "TFLOP/s", "h2d_bytes_per_step": M * HIDDEN * 2,
                                 "d2h_bytes_per_step": M * HIDDEN * 2}})
        if world == 1 and not prefill and not args.no_moe_leg:
            # the other configurations of the published table, as short legs of the same run
            line["prefill"] = prefill_leg()
            line["c1"] = c1_leg(device)
            for sg in step_graphs + gemv_graphs:
                sg.close()
            del sets[1:]
            torch.cuda.empty_cache()
            line["moe"] = moe_legs(device)
        if world == 1:
            cpu_rows = min(M, 16)
            cpu_gbs, passes, dt, cores = time_cpu(cpu_rows, args.cpu_seconds, 200)
            if prefill:
                cpu_gbs = cpu_gbs / LAYER_BYTES * (flops_step * cpu_rows / M) / 1e3   # GB/s -> TFLOP/s
                line["cpu_baseline"] = {
                    "value": cpu_gbs, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                    "sample": f"{passes} passes ({dt:.1f} s) of the same layer at {cpu_rows} rows on "
                              "the CPU oracle (C port of escha_mlx/ref.py)"}
                print(json.dumps(line), flush=True)
                return
            line["cpu_baseline"] = {
                "value": cpu_gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                "sample": f"{passes} full layer passes ({dt:.1f} s) of the same 7-projection "
                          f"layer at batch {cpu_rows} on the CPU oracle (C port of escha_mlx/ref.py)"}
        print(json.dumps(line), flush=True)
    if world > 1:
        # graphs that captured NCCL collectives pin the communicator: NCCL's teardown
        # waits for them to be destroyed, so release them before leaving the group
        torch.cuda.synchronize()
        for g in step_graphs + gemv_graphs:
            g.close()
        del out, gathered, arena
        if pg is not None:
            pg.close()  # unmap the other ranks' buffers while their owners are still alive
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()
        sys.stdout.flush()
        sys.stderr.flush()


if __name__ == "__main__":
    main()

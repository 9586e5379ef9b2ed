#!/usr/bin/env python3
"""Headline benchmark: Gemma-3-12B Q4_K_M target + Gemma-3-270M Q8_0 drafter, H1 speculative
decode (one drafted token, two-row verification, lossless acceptance), on synthetic random-init
weights of those geometries.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --workload streams [--streams S] [--prefix P] [--steps K] [--gpus N]
    torchrun ... bench.py --gpus N --workload tp [--h1] [--exchange peer|nccl]     one stream, the 12B target sharded over N GPUs
    python bench.py --horizon H [--conditional]                                   chains of H drafts per cycle
    python bench.py --case matmul <dtype 8|12|14> <K> <N> <rows> [launches]
    python bench.py --case attention <cached rows> <rows> <heads> <kv_heads> <window> <kv_f16 0|1> [launches]
    python bench.py --case prefill <12b|270m> <tokens> [tensor path 0|1]
    python bench.py --case prefill_matmul <dtype 8|12|14> <K> <N> <rows> [launches]
    python bench.py --case prefill_attention <cached rows> <rows> <heads> <kv_heads> <window> [launches]

A "step" is one H1 cycle: drafter proposal -> two-row target pass -> candidate selection ->
host acceptance -> publish / rollback.  Accept/reject control flow follows a seeded Bernoulli(0.7)
schedule (random weights give no natural draft agreement) while the real acceptance law runs on
the real logits and proposal law every cycle; tokens per cycle (1 + accepted) is therefore an
assumption of the workload, `ms_per_step` is the measured quantity.  The device-timed loop and the
end-to-end loop replay the same scheduled outcomes.  Each rank decodes its own independent stream
(data parallel, no collective); the reported value is all ranks' tokens over the slowest rank's
device time.

`--impl reference` times the reference's own CPU matmul (its compiled sources, one call per
column slice on every host core) on a bounded sample of the same cycle and scales it by
multiply-add count; where the compiled reference is absent it times the CPU restatement instead.

`--workload streams` is the second workload of the list (configs[4]): the Gemma-2-9B geometry (Q4_K body,
Q8_0 head, binary16 cache, softcaps), S independent conversation streams per GPU that share one replica of
the weights, each with a P-token seeded prefix ingested through the tensor-core prompt path, then K greedy
decode steps for all streams; streams are spread over the ranks with no collective.  Its line reports
whole-job decode tok/s and the HBM bytes a step reads (weights once per group of eight streams, every
stream's cache once).

`--case` runs one small single-kernel case a few times through the C ABI: the command to put
under a profiler.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONTEXT = 2048
TARGET, DRAFT = "gemma3-12b", "gemma3-270m"
ACCEPT_P = 0.7
PREFILL_ROWS = 8          # rows per prompt-ingestion pass (verification passes stay two rows wide)
# dram__bytes_read.sum + dram__bytes_write.sum over the weight bytes of one captured GEMV launch
# (profiles/weight_stream_kernel_q4k_k3840_n65536_rows2.md).
TRAFFIC_PER_ALGORITHMIC_BYTE = (141.66 + 3.08) / 141.56
SEEDS = dict(target=1201, draft=2701, prompt=31, sampler=41, schedule=7, shapes=17)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index, self.rows, self.proc = device_index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.device_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, sm_max, reasons = [], 0.0, set()
        for row in self.rows:
            try:
                sm.append(float(row[1]))
                sm_max = max(sm_max, float(row[2]))
            except (ValueError, IndexError):
                continue
            for name, value in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), row[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": sm_max or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def distributed():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return world, rank, local


def prompt_tokens(vocab: int, rank: int) -> np.ndarray:
    return np.random.default_rng(SEEDS["prompt"] + rank).integers(0, vocab, CONTEXT).astype(np.uint32)


def aggregate_streams(dist, tokens: float, tokens_e2e: float, device_ms: float, e2e_s: float, device=None):
    """Whole-job figures of N independent streams: tokens add up, time is the slowest rank's.
    `dist` is torch.distributed (any backend) or None for a single process."""
    if dist is None:
        return tokens, tokens_e2e, device_ms, e2e_s
    import torch
    totals = torch.tensor([tokens, tokens_e2e], dtype=torch.float64, device=device)
    slowest = torch.tensor([device_ms, e2e_s], dtype=torch.float64, device=device)
    dist.all_reduce(totals, op=dist.ReduceOp.SUM)
    dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
    return (*totals.tolist(), *slowest.tolist())


# ----------------------------------------------------------------------------------------- ours

L2_BYTES = 126 << 20
# configs[0] and configs[1] of the workload list: single dequant-GEMV shapes, one and two rows.
SHAPES = [("q4k_ffn_gate_15360x3840", 12, 3840, 15360), ("q6k_ffn_down_3840x15360", 14, 15360, 3840),
          ("q80_drafter_2048x640", 8, 640, 2048), ("q80_drafter_640x2048", 8, 2048, 640),
          ("q80_head_262144x640", 8, 640, 262144)]


def shape_rooflines(lib, syn, peak: float) -> list:
    """GB/s of weight bytes for each single-matrix shape at one and two rows: "isolated" = one
    product per submission (median of 20, events around each), "sustained" = 40 products back to
    back between one event pair.  Successive products read different copies of the matrix, more
    of them than fit in L2, so every byte comes from HBM."""
    L = lib.load()
    rng = np.random.default_rng(SEEDS["shapes"])
    out = []
    for name, dtype, k, n in SHAPES:
        native = syn.make_weight(rng, dtype, k, n)
        first = lib.PackedWeight(dtype, k, n, native)
        copies = max(2, -(-2 * L2_BYTES // first.nbytes) + 1)
        pool = lib.DeviceBuffer(copies * first.nbytes)
        for c in range(copies):
            lib.check(L.gf_copy(pool.ptr + c * first.nbytes, first.packed.ptr, first.nbytes, None))
        first.packed.free()
        nbytes = syn.weight_bytes(dtype, k, n)
        entry = {"shape": name, "weight_bytes": nbytes, "copies": copies}
        for rows in (1, 2):
            x = lib.DeviceBuffer.from_numpy(rng.standard_normal((rows, k)).astype(np.float32))
            y = lib.DeviceBuffer(rows * n * 4)
            ws_bytes = L.gf_matmul_workspace_bytes(dtype, rows, k, n)
            ws = lib.DeviceBuffer(ws_bytes) if ws_bytes else None

            def run(i):
                lib.check(L.gf_matmul(dtype, pool.ptr + (i % copies) * first.nbytes, x.ptr, y.ptr, rows, k, n,
                                      ws.ptr if ws else None, None))
            for i in range(copies + 3):
                run(i)
            lib.check(L.gf_stream_synchronize(None))
            isolated = []
            for i in range(20):
                e0, e1 = lib.Event(), lib.Event()
                e0.record(None)
                run(i)
                e1.record(None)
                e1.synchronize()
                isolated.append(e0.elapsed_ms(e1))
            e0, e1 = lib.Event(), lib.Event()
            e0.record(None)
            for i in range(40):
                run(i)
            e1.record(None)
            e1.synchronize()
            sustained = e0.elapsed_ms(e1) / 40
            lib.check(L.gf_matmul_check(None))
            iso = float(np.median(isolated))
            entry[f"rows{rows}"] = {"isolated_us": iso * 1e3, "isolated_gbs": nbytes / iso / 1e6,
                                    "sustained_us": sustained * 1e3, "sustained_gbs": nbytes / sustained / 1e6,
                                    "sustained_frac": nbytes / sustained / 1e6 / peak}
            for b in (x, y, ws):
                if b:
                    b.free()
        pool.free()
        out.append(entry)
    return out


def run_ours(args) -> dict:
    from guffin_b200 import engine as ge, lib, model as gm, synthetic as syn
    world, rank, local = distributed()
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    L = lib.load()
    lib.check(L.gf_set_device(local))
    steps, warmup = args.steps, max(args.warmup, 3)
    horizon = max(1, args.horizon)
    context = CONTEXT + (horizon + 1) * (warmup + 2 * steps) + 64          # at most horizon + 1 tokens per cycle, two timed loops

    t0 = time.time()
    tc, dc = syn.model_config(TARGET), syn.model_config(DRAFT)
    target = gm.Model(tc, syn.iter_model_weights(TARGET, SEEDS["target"]), context, PREFILL_ROWS)
    draft = gm.Model(dc, syn.iter_model_weights(DRAFT, SEEDS["draft"]), context, PREFILL_ROWS)
    load_s = time.time() - t0
    if args.schedule is not None:
        target.use_pass_kernel(args.schedule)
        draft.use_pass_kernel(args.schedule)
    options = ge.H1Options(ge.sampler_options(0.7, 40, 0.95, 0.05, 1.0, seed=SEEDS["sampler"] + rank), 1, 1, ACCEPT_P,
                           SEEDS["schedule"] + rank, 0, horizon, int(args.conditional))
    engine = ge.H1(target, draft, options)
    # Prompt ingestion of both plans, twice: the first call also allocates the 128-row arena and loads
    # the kernels, the second is what a session pays per prompt.
    prefill_times = []
    for _ in range(2):
        t0 = time.time()
        engine.prefill(prompt_tokens(tc["vocab"], rank))
        target.synchronize()
        draft.synchronize()
        prefill_times.append(time.time() - t0)
    prefill_first_s, prefill_s = prefill_times

    def barrier():
        target.synchronize()
        draft.synchronize()
        if dist is not None:
            dist.barrier()

    def launches_now():
        return target.kernel_launches() + draft.kernel_launches() + int(engine.stats().sampler_launches)

    # ---- warm-up, then K cycles timed on the device (events on the target's stream; the drafter's
    # work is ordered into it every cycle), bracketed by barrier + synchronise.  Both measured loops
    # restart the accept schedule from the same seed, so they see the same outcomes.
    token_room = lambda cycles: (horizon + 1) * cycles + 2          # a cycle emits at most horizon + 1 tokens
    engine.generate_steps(warmup, token_room(warmup))
    barrier()
    loop_seed = 1000 + SEEDS["schedule"] + rank
    engine.reseed_schedule(loop_seed)
    launches_before = launches_now()
    stats_before = engine.stats()
    start, end = lib.Event(), lib.Event()
    with ClockSampler(local) as clocks:
        start.record(target.stream)
        wall0 = time.perf_counter()
        tokens = engine.generate_steps(steps, token_room(steps))
        end.record(target.stream)
        end.synchronize()
        wall = time.perf_counter() - wall0
        device_ms = start.elapsed_ms(end)
        launches = launches_now() - launches_before          # kernels of the device-timed loop only, counted as launched
        stats_loop = engine.stats()
        # Same loop once more for the end-to-end figure: host wall clock around the public call,
        # which uploads the root token and selection requests and reads back candidates and the
        # drafter's receipt every cycle.
        barrier()
        engine.reseed_schedule(loop_seed)
        e2e0 = time.perf_counter()
        tokens_e2e = engine.generate_steps(steps, token_room(steps))
        target.synchronize()
        e2e_wall = time.perf_counter() - e2e0
        # ---- roofline of the dominant kernel: exactly one verify pass's weight GEMVs, alone.
        sweep_ms = []
        for i in range(5):
            s0, s1 = lib.Event(), lib.Event()
            s0.record(target.stream)
            sweep_launches, sweep_bytes = target.weight_sweep(2)
            s1.record(target.stream)
            s1.synchronize()
            if i >= 2:
                sweep_ms.append(s0.elapsed_ms(s1))
    barrier()
    cycles = stats_loop.cycles + stats_loop.ordinary_steps - stats_before.cycles - stats_before.ordinary_steps
    accepted = int(stats_loop.accepted - stats_before.accepted)
    status = target.status() | draft.status()
    weight_bytes = target.weight_bytes(True) + draft.weight_bytes(True)
    kv_bytes = target.kv_bytes_per_pass(2)

    produced, produced_e2e, elapsed_ms, e2e_s = aggregate_streams(
        dist, float(len(tokens)), float(len(tokens_e2e)), device_ms, e2e_wall, "cuda" if dist is not None else None)
    if rank != 0:
        return {}

    peak, peak_kind = load_peaks()
    sweep = float(np.mean(sweep_ms))
    achieved = sweep_bytes / (sweep * 1e-3) / 1e9
    result = {
        "metric": "Gemma3-12B Q4_K_M+270M H1 decode tok/s per GPU; dequant-GEMV HBM GB/s vs 8 TB/s",
        "value": produced / (elapsed_ms * 1e-3),            # whole job: every rank's stream
        "unit": "tok/s",
        "per_gpu_tok_s": produced / (elapsed_ms * 1e-3) / world,
        "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": elapsed_ms / steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u4/u6/u8 blocks -> f32",
        "data": "synthetic",
        "config": {"workload": ("configs[3]: Gemma-3-12B Q4_K_M + 270M Q8_0 drafter, H1, context 2048, T=0.7 top-k 40 "
                                "top-p 0.95 min-p 0.05, 2-row verification, seeded Bernoulli(0.7) accept schedule") if horizon == 1 else
                               (f"configs[3] with chains of {horizon} drafts per cycle ({horizon + 1}-row verification, one Bernoulli(0.7) "
                                "draw per draft): not the headline"),
                   "schedule": {None: "kernel per operator (default)", 0: "kernel per operator", 1: "decode pass kernel",
                                2: "decode pass kernel, attention launched separately"}[args.schedule],
                   "horizon": horizon, "verification": "conditional tiles" if args.conditional and horizon > 2 else "one pass",
                   "streams_per_gpu": 1, "parallelism": f"independent streams x{world} (no collective)",
                   "l2_policy": "inputs larger than L2: every pass streams 7.3 GB of distinct weights",
                   "assumed_accept_probability": ACCEPT_P,
                   "tokens_per_cycle_rank0": len(tokens) / max(cycles, 1),
                   "cycles_per_s_per_gpu": steps / (elapsed_ms * 1e-3),
                   "accepted": accepted, "cycles": int(cycles),
                   "law_agreements": int(stats_loop.law_agreements - stats_before.law_agreements),
                   "load_s": round(load_s, 1), "prefill_s": round(prefill_s, 3), "prefill_first_call_s": round(prefill_first_s, 3),
                   "prefill_tok_s": round(CONTEXT / prefill_s, 1),
                   "status_word": int(status)},
        "e2e": {"value": produced_e2e / e2e_s, "unit": "tok/s",
                "h2d_bytes_per_step": 4 + (horizon + 1) * 264, "d2h_bytes_per_step": (horizon + 1) * 3080 + horizon * 3096,
                "ms_per_step": e2e_s * 1e3 / steps, "wall_s_first_loop": wall},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": f"of {peak_kind}",
                     # DRAM bytes per launch: the read+write bytes ncu counted on one launch of the same kernel
                     # (Q4_K, K = 3840, N = 65536, two rows: 144.74 MB for 141.56 MB of weights), scaled by bytes.
                     "traffic": TRAFFIC_PER_ALGORITHMIC_BYTE * sweep_bytes / sweep_launches,
                     "kernel": "weight_stream_kernel (Q4_K/Q6_K, rows=2): one verify pass's weight products run alone",
                     "bytes_per_launch": sweep_bytes / sweep_launches, "launches": sweep_launches,
                     "avg_launch_us": sweep * 1e3 / sweep_launches,
                     "cycle_bytes": weight_bytes + kv_bytes,
                     "cycle_frac": (weight_bytes + kv_bytes) / (elapsed_ms / steps * 1e-3) / 1e9 / peak},
        "clocks": clocks.summary(),
    }
    if world == 1 and not args.no_shapes:
        result["roofline"]["per_shape"] = shape_rooflines(lib, syn, peak)
    if world == 1 and not args.no_cpu_baseline:
        result["cpu_baseline"], result["parity"] = cpu_baseline_with_parity(target)
    return result


def run_streams(args) -> dict:
    """configs[4]: independent streams of the Gemma-2-9B geometry, data parallel over the ranks."""
    from guffin_b200 import lib, model as gm, synthetic as syn
    world, rank, local = distributed()
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    L = lib.load()
    lib.check(L.gf_set_device(local))
    name = "gemma2-9b"
    config = syn.model_config(name)
    per_gpu, prefix = args.streams, args.prefix
    steps, warmup = args.steps, max(args.warmup, 3)
    context = prefix + warmup + steps + 8
    t0 = time.time()
    plan = gm.Model(config, syn.iter_model_weights(name, SEEDS["target"]), context, PREFILL_ROWS)
    load_s = time.time() - t0
    streams = gm.Streams(plan, per_gpu)
    if args.tensor_decode:
        streams.set_mode(1)
    t0 = time.time()
    for s in range(per_gpu):
        tokens = np.random.default_rng(SEEDS["prompt"] + 1000 * rank + s).integers(0, config["vocab"], prefix).astype(np.uint32)
        streams.prefill(s, tokens)
    plan.synchronize()
    prefill_s = time.time() - t0

    def barrier():
        plan.synchronize()
        if dist is not None:
            dist.barrier()

    def step():
        streams.decode(streams.greedy())            # one selection + readback, then one token per stream

    for _ in range(warmup):
        step()
    barrier()
    launches_before = plan.kernel_launches()
    kv_bytes = streams.kv_bytes_per_step()
    start, end = lib.Event(), lib.Event()
    with ClockSampler(local) as clocks:
        start.record(plan.stream)
        wall0 = time.perf_counter()
        for _ in range(steps):
            step()
        end.record(plan.stream)
        end.synchronize()
        wall = time.perf_counter() - wall0
        device_ms = start.elapsed_ms(end)
    launches = plan.kernel_launches() - launches_before
    barrier()
    status = plan.status()
    produced, produced_e2e, elapsed_ms, e2e_s = aggregate_streams(
        dist, float(per_gpu * steps), float(per_gpu * steps), device_ms, wall, "cuda" if dist is not None else None)
    if rank != 0:
        return {}
    peak, peak_kind = load_peaks()
    groups = 1 if args.tensor_decode else (per_gpu + PREFILL_ROWS - 1) // PREFILL_ROWS
    step_bytes = groups * plan.weight_bytes(True) + kv_bytes
    achieved = step_bytes / (elapsed_ms / steps * 1e-3) / 1e9
    return {
        "metric": "Gemma-2-9B Q4_K decode tok/s, independent streams (whole job)",
        "value": produced / (elapsed_ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": elapsed_ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u4/u8 blocks -> f32, binary16 cache", "data": "synthetic",
        "config": {"workload": f"configs[4]: Gemma-2-9B Q4_K body + Q8_0 head, {per_gpu} independent streams per GPU, "
                               f"{prefix}-token seeded prefixes (tensor-core ingestion), greedy decode",
                   "streams_per_gpu": per_gpu, "streams": per_gpu * world, "prefix": prefix,
                   "decode_projections": "one bf16 tensor-core pass over all streams" if args.tensor_decode
                   else "exact row passes in groups of eight streams",
                   "parallelism": f"independent streams x{world} ranks (no collective)",
                   "l2_policy": "inputs larger than L2: a step streams the weights once per group of eight streams and every stream's cache",
                   "load_s": round(load_s, 1), "prefill_s": round(prefill_s, 2),
                   "prefill_tok_s": round(per_gpu * prefix / prefill_s, 1), "status_word": int(status)},
        "e2e": {"value": produced_e2e / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": per_gpu * (4 + 264),
                "d2h_bytes_per_step": per_gpu * 3080, "ms_per_step": e2e_s * 1e3 / steps},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": f"of {peak_kind}", "traffic": None,
                     "kernel": "one decode step: weight_stream_kernel per group of streams + stream attention over every cache",
                     "step_bytes": step_bytes, "kv_bytes": kv_bytes, "weight_passes": groups},
        "clocks": clocks.summary(),
    }


def run_tensor_parallel_h1(args, plan, shard, dist, world, rank, local, context, prompt, load_s, prefill_s) -> dict:
    """The headline's H1 cycle with the target sharded over the ranks: every rank runs its own engine on its shard
    and its own replica of the drafter, with the same seeds; the shards' merged candidate rows are identical, so
    the engines stay in step and emit the same tokens."""
    from guffin_b200 import engine as ge, lib, model as gm, synthetic as syn
    steps, warmup = args.steps, max(args.warmup, 3)
    dc = syn.model_config(DRAFT)
    draft = gm.Model(dc, syn.iter_model_weights(DRAFT, SEEDS["draft"]), context, PREFILL_ROWS)
    if shard is not None:
        shard.global_selection()
    options = ge.H1Options(ge.sampler_options(0.7, 40, 0.95, 0.05, 1.0, seed=SEEDS["sampler"]), 1, 1, ACCEPT_P, SEEDS["schedule"], 0, 1)
    engine = ge.H1(plan, draft, options)
    engine.prefill(prompt)

    def barrier():
        plan.synchronize()
        draft.synchronize()
        if dist is not None:
            dist.barrier()

    engine.generate_steps(warmup, 2 * warmup + 2)
    barrier()
    engine.reseed_schedule(1000 + SEEDS["schedule"])
    before = engine.stats()
    launches_before = plan.kernel_launches() + draft.kernel_launches() + int(before.sampler_launches)
    start, end = lib.Event(), lib.Event()
    with ClockSampler(local) as clocks:
        start.record(plan.stream)
        wall0 = time.perf_counter()
        tokens = engine.generate_steps(steps, 2 * steps + 2)
        end.record(plan.stream)
        end.synchronize()
        wall = time.perf_counter() - wall0
        device_ms = start.elapsed_ms(end)
    after = engine.stats()
    launches = plan.kernel_launches() + draft.kernel_launches() + int(after.sampler_launches) - launches_before
    barrier()
    status = plan.status()
    digest = int(np.bitwise_xor.reduce(tokens.astype(np.uint64) * np.arange(1, tokens.size + 1, dtype=np.uint64)))
    if dist is not None:
        import torch
        slowest = torch.tensor([device_ms, wall], dtype=torch.float64, device="cuda")
        dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
        device_ms, wall = slowest.tolist()
        digests = [None] * world
        dist.all_gather_object(digests, digest)
        in_step = len(set(digests)) == 1
    else:
        in_step = True
    if rank != 0:
        return {}
    cycles = int(after.cycles - before.cycles)
    return {
        "metric": "Gemma3-12B Q4_K_M+270M H1 decode tok/s, one stream, target sharded over the GPUs", "value": tokens.size / (device_ms * 1e-3),
        "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": device_ms / steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u4/u6/u8 blocks -> f32", "data": "synthetic",
        "config": {"workload": "configs[3] (H1, context 2048, T=0.7 top-k 40 top-p 0.95 min-p 0.05, seeded Bernoulli(0.7) accept schedule) as ONE stream: "
                               + (f"the 12B target row-sharded over {world} GPUs (partial sums exchanged inside the projection launches), an engine and "
                                  "a drafter replica per GPU in step" if world > 1 else "unsharded target, one GPU"),
                   "parallelism": f"tp{world}", "l2_policy": "inputs larger than L2: every pass streams its weights once",
                   "tokens_per_cycle": round(tokens.size / max(cycles, 1), 3), "cycles": cycles, "engines_in_step": in_step,
                   "load_s": round(load_s, 1), "prefill_s": round(prefill_s, 3), "status_word": int(status)},
        "e2e": {"value": tokens.size / wall, "unit": "tok/s", "h2d_bytes_per_step": 4 + 2 * 264, "d2h_bytes_per_step": world * 2 * 3080 + 3096,
                "ms_per_step": wall * 1e3 / steps},
        "gpu_launches": int(launches),
        "roofline": None,
        "clocks": clocks.summary(),
    }


def run_tensor_parallel(args) -> dict:
    """One stream of the 12B target sharded over the ranks (guffin_b200.tensor_parallel): the latency of the
    two-row verification pass with an NCCL all-reduce behind every O and down projection.  One rank runs the
    unsharded plan, so the same command gives the single-GPU figure it is compared with."""
    from guffin_b200 import lib, model as gm, synthetic as syn, tensor_parallel as tp
    world, rank, local = distributed()
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    L = lib.load()
    lib.check(L.gf_set_device(local))
    name = "gemma3-12b"
    config = syn.model_config(name)
    steps, warmup = args.steps, max(args.warmup, 3)
    prefix = min(args.prefix, 2040)
    context = prefix + 2 * (warmup + steps) + 16
    rng = np.random.default_rng(SEEDS["prompt"])
    prompt = rng.integers(0, config["vocab"], prefix).astype(np.uint32)
    pairs = rng.integers(0, config["vocab"], (warmup + steps + 1, 2)).astype(np.uint32)
    reducer = None
    t0 = time.time()
    if world > 1:
        def exchange(ident):
            box = [ident]
            dist.broadcast_object_list(box, src=0)
            return box[0]
        if args.exchange == "nccl":
            reducer = tp.NcclReducer(rank, world, exchange)
            shard = tp.Shard(config, syn.iter_model_weights(name, SEEDS["target"]), context, rank, world, reducer.hook, PREFILL_ROWS)
        else:
            shard = tp.Shard(config, syn.iter_model_weights(name, SEEDS["target"]), context, rank, world, None, PREFILL_ROWS)
            handles = [None] * world
            dist.all_gather_object(handles, shard.exported())
            shard.connect_exported(handles)
            dist.barrier()                  # every shard is connected before any pass starts
        plan = shard.model
    else:
        plan = gm.Model(config, syn.iter_model_weights(name, SEEDS["target"]), context, PREFILL_ROWS)
    load_s = time.time() - t0
    def barrier():
        plan.synchronize()
        if dist is not None:
            dist.barrier()

    # Prompt ingestion twice: the first call also allocates the chunk arena and loads the kernels, the second is
    # what a session pays per prompt.
    t0 = time.time()
    plan.prefill(prompt)
    plan.synchronize()
    prefill_first_s = time.time() - t0
    plan.reset()
    barrier()
    t0 = time.time()
    plan.prefill(prompt)
    plan.synchronize()
    prefill_s = time.time() - t0

    if args.h1:
        return run_tensor_parallel_h1(args, plan, shard if world > 1 else None, dist, world, rank, local, context, prompt, load_s, prefill_s)

    def step(i):
        plan.forward(pairs[i])
        plan.publish(1)

    for i in range(warmup):
        step(i)
    barrier()
    launches_before = plan.kernel_launches()
    start, end = lib.Event(), lib.Event()
    with ClockSampler(local) as clocks:
        start.record(plan.stream)
        wall0 = time.perf_counter()
        for i in range(steps):
            step(warmup + i)
        end.record(plan.stream)
        end.synchronize()
        wall = time.perf_counter() - wall0
        device_ms = start.elapsed_ms(end)
    launches = plan.kernel_launches() - launches_before
    barrier()
    # the last pass once more with the logits read back: the shards' slices side by side are the full rows
    plan.forward(pairs[warmup + steps])
    logits = np.stack([plan.logits(0), plan.logits(1)])
    status = plan.status()
    checksum = None
    if dist is not None:
        import torch
        mine = torch.from_numpy(logits).cuda()
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        full = torch.cat(gathered, dim=1).cpu().numpy()
        slowest = torch.tensor([device_ms, wall], dtype=torch.float64, device="cuda")
        dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
        device_ms, wall = slowest.tolist()
    else:
        full = logits
    if rank != 0:
        return {}
    checksum = {"argmax": [int(v) for v in full.argmax(axis=1)], "l2": [float(np.linalg.norm(row)) for row in full]}
    peak, peak_kind = load_peaks()
    pass_bytes = plan.weight_bytes(True) * world
    achieved = pass_bytes / (device_ms / steps * 1e-3) / 1e9
    return {
        "metric": "Gemma3-12B Q4_K_M two-row verification passes/s, one stream sharded over the GPUs", "value": steps / (device_ms * 1e-3),
        "unit": "passes/s", "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": device_ms / steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u4/u8 blocks -> f32, binary16 cache",
        "data": "synthetic",
        "config": {"workload": f"one Gemma3-12B stream at {prefix} committed tokens, two-row pass + publish, "
                               + ((f"row-sharded over {world} GPUs, " + ("NCCL all-reduce behind every O and down projection" if args.exchange == "nccl"
                                  else "partial sums exchanged inside the projection launches over peer memory")) if world > 1 else "unsharded plan"),
                   "parallelism": f"tp{world}", "l2_policy": "inputs larger than L2: a pass streams every weight once",
                   "load_s": round(load_s, 1), "prefill_s": round(prefill_s, 3), "prefill_first_call_s": round(prefill_first_s, 2),
                   "prefill_tok_s": round(prefix / prefill_s, 1), "status_word": int(status),
                   "reductions_per_pass": 2 * config["layers"] if world > 1 else 0, "exchange": args.exchange if world > 1 else None, "last_pass_logits": checksum},
        "e2e": {"value": steps / wall, "unit": "passes/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 0, "ms_per_step": wall * 1e3 / steps},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak * world, "unit": "GB/s", "frac": achieved / (peak * world),
                     "peak_source": f"of {peak_kind} x {world} GPUs", "traffic": None, "kernel": "one two-row pass over every shard"},
        "clocks": clocks.summary(),
    }


# ----------------------------------------------------------------------------------------- CPU arm

def cpu_port_cycles(threads: int, cycles: int, warmup: int, gpu_target=None):
    """Times the CPU restatement of the reference's path for whole H1 cycles: one drafter row and two
    target rows through its scalar dequant-GEMV block schedule, the second target row dropped again
    (a rejected draft), at a context of a few tokens (a 2048-token CPU prefill would take over an
    hour; attention is a negligible share).  With `gpu_target` the same two rows run on the GPU plan
    from a reset cache and the logits of both sides are compared."""
    from guffin_b200 import synthetic as syn
    from oracle.pyoracle import Oracle, OracleModel, build
    build(reference=False)
    oracle = Oracle()
    oracle.set_threads(threads)
    tc, dc = syn.model_config(TARGET), syn.model_config(DRAFT)
    total = cycles + warmup
    target = OracleModel(oracle, tc, syn.make_model_weights(TARGET, SEEDS["target"]), context=total + 4)
    draft = OracleModel(oracle, dc, syn.make_model_weights(DRAFT, SEEDS["draft"]), context=total + 4)
    tokens = prompt_tokens(tc["vocab"], 0)
    if gpu_target is not None:
        gpu_target.reset()
    times, errors = [], []
    for i in range(total):
        t0 = time.perf_counter()
        draft.append(tokens[i], want_logits=True)
        want = [target.append(tokens[i], want_logits=True), target.append(tokens[i + 1], want_logits=True)]
        target.truncate(i + 1)                                # the rejected draft row is dropped
        times.append(time.perf_counter() - t0)
        if gpu_target is not None:
            gpu_target.forward(tokens[i:i + 2], logits=True)
            for row in range(2):
                got = gpu_target.logits(row)
                errors.append(float(np.linalg.norm(got - want[row]) / np.linalg.norm(want[row])))
            gpu_target.publish(1)
    return times[warmup:], errors


def cpu_baseline_with_parity(gpu_target):
    threads = os.cpu_count() or 1
    times, errors = cpu_port_cycles(threads, 2, 2, gpu_target)
    per_cycle = float(np.mean(times))
    baseline = {"value": (1.0 + ACCEPT_P) / per_cycle, "unit": "tok/s", "cores": threads, "kind": "port",
                "ms_per_step": per_cycle * 1e3,
                "sample": f"{len(times)} H1 cycles (1 drafter row + 2 target rows each) after 2 warm-up cycles at context <= "
                          f"{len(times) + 4} tokens, CPU restatement of the reference's scalar dequant-GEMV block schedule "
                          f"split over {threads} threads by output column, {1 + ACCEPT_P:.1f} tokens per cycle assumed"}
    parity = {"rel_l2": max(errors), "rows": len(errors), "what": "12B two-row verify logits, GPU plan against the CPU "
              "restatement on the same tokens from an empty cache"}
    return baseline, parity


def reference_layer_sample(threads: int, steps: int, warmup: int):
    """Times the reference's own backends::cpu::matmul_f32_quantized_gguf_weight (compiled from its
    sources into oracle/_ref) on the seven projections of two 12B layers at two rows -- one layer
    whose attn_v / ffn_down are Q6_K and one all-Q4_K, the two kinds a Q4_K_M file holds in equal
    number -- each matrix cut into column slices, one call per slice, `threads` calls in flight."""
    from concurrent.futures import ThreadPoolExecutor
    from guffin_b200 import synthetic as syn
    from oracle.pyoracle import Reference, build, BLOCK_BYTES, BLOCK_ELEMENTS
    build(reference=False)
    ref = Reference()
    config = syn.model_config(TARGET)
    rng = np.random.default_rng(SEEDS["target"])
    jobs, elements = [], 0
    for q6 in (True, False):
        for name, (k, n) in syn.matrix_shapes(config).items():
            dtype = syn.Q6_K if q6 and name in ("attn_v", "ffn_down") else syn.Q4_K
            weight = syn.make_weight(rng, dtype, k, n)
            x = rng.standard_normal((2, k)).astype(np.float32)
            column_bytes = (k // BLOCK_ELEMENTS[dtype]) * BLOCK_BYTES[dtype]
            slices = min(n, 4 * threads)
            for s in range(slices):
                begin, end = n * s // slices, n * (s + 1) // slices
                jobs.append((dtype, x, weight[begin * column_bytes:end * column_bytes], k, end - begin,
                             np.empty((2, end - begin), np.float32)))
            elements += 2 * k * n

    def run(job):
        dtype, x, weight, k, n, out = job
        assert ref.lib.ref_matmul_quantized(dtype, x, weight, 2, k, n, out) == 0

    times = []
    with ThreadPoolExecutor(threads) as pool:
        for i in range(steps + warmup):
            t0 = time.perf_counter()
            list(pool.map(run, jobs))
            times.append(time.perf_counter() - t0)
    return times[warmup:], elements


def cycle_multiply_adds() -> float:
    """Weight elements times rows of one H1 cycle: two target rows, and the drafter's 1 + 0.7 rows
    (the pending token of an accepted cycle rides along)."""
    from guffin_b200 import synthetic as syn

    def elements(name):
        config = syn.model_config(name)
        body = sum(k * n for k, n in syn.matrix_shapes(config).values()) * config["layers"]
        return body + config["hidden"] * config["vocab"]
    return 2.0 * elements(TARGET) + (1.0 + ACCEPT_P) * elements(DRAFT)


def run_reference(args) -> dict:
    from oracle.pyoracle import Reference
    world, rank, _ = distributed()
    if rank != 0:
        return {}
    threads = os.cpu_count() or 1
    steps, warmup = max(1, args.steps), max(2, args.warmup)
    if Reference.available():
        # A step is the bounded sample; the cycle time follows from it by multiply-add count.
        steps = min(steps, 8)
        times, sample_elements = reference_layer_sample(threads, steps, warmup)
        scale = cycle_multiply_adds() / sample_elements
        per_cycle = float(np.mean(times)) * scale
        kind = "reference"
        sample = (f"{len(times)} timed samples after {warmup} warm-up: the reference's matmul_f32_quantized_gguf_weight (its own "
                  f"sources, compiled) on the 7 projections of two 12B layers at 2 rows ({sample_elements / 2e6:.0f} M weights), "
                  f"column slices on {threads} threads, {np.mean(times):.2f} s per sample; scaled x{scale:.1f} by multiply-add count "
                  f"to one H1 cycle (2 target rows + {1 + ACCEPT_P:.1f} drafter rows; attention, norms and sampling left out), "
                  f"{1 + ACCEPT_P:.1f} tokens per cycle assumed")
    else:
        steps = min(steps, 6)
        times, _ = cpu_port_cycles(threads, steps, warmup)
        per_cycle = float(np.mean(times))
        kind = "port"
        sample = (f"{len(times)} H1 cycles (1 drafter row + 2 target rows each) after {warmup} warm-up cycles at context <= "
                  f"{len(times) + warmup + 4} tokens, CPU restatement of the reference's scalar dequant-GEMV (the compiled reference "
                  f"is not present), {threads} threads, {1 + ACCEPT_P:.1f} tokens per cycle assumed")
    value = (1.0 + ACCEPT_P) / per_cycle
    return {
        "impl": "reference",
        "metric": "Gemma3-12B Q4_K_M+270M H1 decode tok/s per GPU; dequant-GEMV HBM GB/s vs 8 TB/s",
        "value": value, "unit": "tok/s", "n_gpus": world, "steps": len(times), "warmup": warmup,
        "ms_per_step": per_cycle * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u4/u6/u8 blocks -> f32", "data": "synthetic",
        "config": {"workload": "configs[3]: Gemma-3-12B Q4_K_M + 270M Q8_0 drafter, H1 (CPU sample, see cpu_baseline.sample)",
                   "steps_requested": args.steps, "sample_s": float(np.mean(times))},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


# ----------------------------------------------------------------------------------------- single-kernel cases

def run_case(argv) -> int:
    """One small single-kernel case, a few launches through the C ABI (for a profiler)."""
    from guffin_b200 import lib, model, synthetic as syn  # noqa: F401  (model declares the operator signatures)
    L = lib.load()
    rng = np.random.default_rng(0)
    kind = argv[0]
    numbers = [int(a) for a in argv[1:]] if kind != "prefill" else []
    if kind == "matmul":
        dtype, k, n, rows = numbers[:4]
        launches = numbers[4] if len(numbers) > 4 else 3
        weight = lib.PackedWeight(dtype, k, n, syn.make_weight(rng, dtype, k, n))
        x = lib.DeviceBuffer.from_numpy(rng.standard_normal((rows, k)).astype(np.float32))
        y = lib.DeviceBuffer(rows * n * 4)
        ws_bytes = L.gf_matmul_workspace_bytes(dtype, rows, k, n)
        ws = lib.DeviceBuffer(ws_bytes) if ws_bytes else None
        for _ in range(launches):
            lib.check(L.gf_matmul(dtype, weight.packed.ptr, x.ptr, y.ptr, rows, k, n, ws.ptr if ws else None, None))
        lib.check(L.gf_matmul_check(None))
        print(f"ok: {launches} gf_matmul launches, dtype={dtype} K={k} N={n} rows={rows} ({weight.nbytes / 1e6:.1f} MB of weights)")
        return 0
    if kind == "attention":
        base, rows, heads, kv_heads, window, kv_f16 = numbers[:6]
        launches = numbers[6] if len(numbers) > 6 else 3
        ring_rows = 1 << max(1, int(np.ceil(np.log2(base + rows))))
        kv_dtype = np.float16 if kv_f16 else np.float32
        q = rng.standard_normal((rows, heads * 256)).astype(np.float32)
        arrays = [q] + [rng.standard_normal((ring_rows, kv_heads * 256)).astype(kv_dtype) for _ in range(2)] \
            + [rng.standard_normal((rows, kv_heads * 256)).astype(kv_dtype) for _ in range(2)]
        buffers = [lib.DeviceBuffer.from_numpy(a) for a in arrays]
        out = lib.DeviceBuffer(q.nbytes)
        workspace = lib.DeviceBuffer(L.gf_attention_workspace_bytes(rows, heads))
        position = lib.DeviceBuffer.from_numpy(np.array([base], np.uint32))
        for _ in range(launches):
            lib.check(L.gf_attention(buffers[0].ptr, buffers[1].ptr, buffers[2].ptr, buffers[3].ptr, buffers[4].ptr, out.ptr,
                                     workspace.ptr, position.ptr, rows, heads, kv_heads, 256, ring_rows, window,
                                     1.0 / 16.0, 0.0, kv_f16, None))
        result = out.download(np.float32)
        print(f"ok: {launches} gf_attention launches, base={base} rows={rows} heads={heads}/{kv_heads} window={window}, "
              f"|out| = {float(np.abs(result).mean()):.4f}")
        return 0
    if kind == "prefill_matmul":
        dtype, k, n, rows = numbers[:4]
        launches = numbers[4] if len(numbers) > 4 else 3
        weight = lib.PackedWeight(dtype, k, n, syn.make_weight(rng, dtype, k, n))
        x = lib.DeviceBuffer.from_numpy(rng.standard_normal((rows, k)).astype(np.float32))
        y = lib.DeviceBuffer((rows + 127) // 128 * 128 * n * 4)          # results come in whole halves of 128 rows
        ws = lib.DeviceBuffer(L.gf_prefill_workspace_bytes(k))
        for _ in range(launches):
            lib.check(L.gf_prefill_matmul(dtype, weight.packed.ptr, x.ptr, y.ptr, rows, k, n, ws.ptr, None))
        print(f"ok: {launches} gf_prefill_matmul launches, dtype={dtype} K={k} N={n} rows={rows} ({weight.nbytes / 1e6:.1f} MB of weights)")
        return 0
    if kind == "prefill_attention":
        base, rows, heads, kv_heads, window = numbers[:5]
        launches = numbers[5] if len(numbers) > 5 else 3
        ring_rows = 1 << max(1, int(np.ceil(np.log2(max(base, 2)))))
        q = rng.standard_normal((rows, heads * 256)).astype(np.float32)
        arrays = [q] + [rng.standard_normal((ring_rows, kv_heads * 256)).astype(np.float16) for _ in range(2)] \
            + [rng.standard_normal((rows, kv_heads * 256)).astype(np.float16) for _ in range(2)]
        buffers = [lib.DeviceBuffer.from_numpy(a) for a in arrays]
        out = lib.DeviceBuffer(q.nbytes)
        position = lib.DeviceBuffer.from_numpy(np.array([base], np.uint32))
        for _ in range(launches):
            lib.check(L.gf_prefill_attention(buffers[0].ptr, buffers[1].ptr, buffers[2].ptr, buffers[3].ptr, buffers[4].ptr, out.ptr,
                                             position.ptr, rows, heads, kv_heads, 256, ring_rows, window, 1.0 / 16.0, 0.0, None))
        result = out.download(np.float32)
        print(f"ok: {launches} gf_prefill_attention launches, base={base} rows={rows} heads={heads}/{kv_heads} window={window}, "
              f"|out| = {float(np.abs(result).mean()):.4f}")
        return 0
    if kind == "prefill":
        # prefill <12b|270m> <tokens> [tensor 0|1]: prompt ingestion alone on one synthetic model.
        name = {"12b": TARGET, "270m": DRAFT}[argv[1]]
        count = int(argv[2])
        tensor = int(argv[3]) if len(argv) > 3 else 1
        from guffin_b200 import model as gm
        config = syn.model_config(name)
        plan = gm.Model(config, syn.iter_model_weights(name, SEEDS["target"]), count + 16, PREFILL_ROWS)
        plan.use_tensor_prefill(bool(tensor))
        tokens = prompt_tokens(config["vocab"], 0)[:count]
        times = []
        for _ in range(2):
            plan.reset()
            plan.synchronize()
            t0 = time.perf_counter()
            plan.prefill(tokens)
            plan.synchronize()
            times.append(time.perf_counter() - t0)
        print(f"ok: {name} prefill of {count} tokens, tensor path {tensor}: {times[-1] * 1e3:.1f} ms ({count / times[-1]:.0f} tok/s), status {plan.status()}")
        return 0
    print(f"unknown case {kind!r}", file=sys.stderr)
    return 2


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=None)
    parser.add_argument("--warmup", type=int, default=None)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline / parity leg of the default arm")
    parser.add_argument("--no-shapes", action="store_true", help="skip the per-shape GB/s table of the default arm")
    parser.add_argument("--schedule", type=int, choices=(0, 1, 2), default=None,
                        help="0: one kernel per operator (CUDA graph, the default); 1: persistent decode pass kernel; "
                             "2: pass kernel with attention launched separately")
    parser.add_argument("--case", nargs="+", default=None, help="run one single-kernel case instead of the benchmark")
    parser.add_argument("--workload", choices=("h1", "streams", "tp"), default="h1",
                        help="h1: the headline (configs[3]); streams: configs[4]; tp: one 12B stream sharded over the GPUs")
    parser.add_argument("--horizon", type=int, default=1, help="drafts per cycle of the h1 workload (1 = the headline; 2..7 = chains)")
    parser.add_argument("--conditional", action="store_true",
                        help="h1 workload with --horizon > 2: verify the chain as a cascade of passes (the reference's conditional tiles)")
    parser.add_argument("--streams", type=int, default=8, help="streams per GPU of the streams workload (64 over eight GPUs)")
    parser.add_argument("--prefix", type=int, default=8192, help="prefix tokens per stream of the streams workload")
    parser.add_argument("--h1", action="store_true",
                        help="tp workload: the whole H1 cycle on the sharded target (an engine and a drafter replica per rank, in step) instead of bare passes")
    parser.add_argument("--exchange", choices=("peer", "nccl"), default="peer",
                        help="tp workload: partial sums exchanged inside the projection launches over peer memory, or by NCCL all-reduces between them")
    parser.add_argument("--tensor-decode", action="store_true",
                        help="streams workload: every step as one bf16 tensor-core pass over all streams instead of exact row passes")
    args = parser.parse_args()
    if args.case:
        sys.exit(run_case(args.case))
    if args.workload == "streams" and args.impl == "ours":
        args.steps = 64 if args.steps is None else args.steps
        args.warmup = 3 if args.warmup is None else args.warmup
        result = run_streams(args)
    elif args.workload == "tp" and args.impl == "ours":
        args.steps = 100 if args.steps is None else args.steps
        args.warmup = 5 if args.warmup is None else args.warmup
        result = run_tensor_parallel(args)
    elif args.impl == "reference":
        args.steps = 3 if args.steps is None else args.steps
        args.warmup = 2 if args.warmup is None else args.warmup
        result = run_reference(args)
    else:
        args.steps = 200 if args.steps is None else args.steps
        args.warmup = 10 if args.warmup is None else args.warmup
        result = run_ours(args)
    if result:
        print(json.dumps(result), flush=True)
    if "torch.distributed" in sys.modules:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    main()

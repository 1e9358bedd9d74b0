"""The disaggregated serving loop around the migration path, with the model
forward replaced by a stand-in: what matters here is *when* migrations run
relative to decode steps, not what the steps compute.

    python -m distserve_b200.e2e_loop [--gpus 1|2] [--steps 400] [--rate 4.0]

Requests arrive as a Poisson process (the reference's load generator,
evaluation/2-benchmark-serving/2-benchmark-serving.py:49-53), each with a
prompt whose KV blocks already sit in the context stage's pool (prefill itself
is outside this path).  The decoding stage runs steps back to back; between
steps it accepts arrived requests, which is where the reference migrates them
(decoding_stage_scheduler.py:247-260 via single_stage_engine.py:490-536, one
awaited call per request, the loop parked meanwhile).  Three runs are timed:

* ``decode_only``  — the steps alone;
* ``bookkeeping``  — steps plus the host work of accepting requests (block
  allocation, table building) but no copy: the part no data path can hide;
* ``serial``       — the reference's cadence: each accepted request is migrated
  with the awaited operator between two steps;
* ``overlapped``   — the migration is enqueued on a side stream with
  ``migrate_blocks_async`` and the next step starts at once; the request joins
  the batch at the first step boundary after its ticket has completed.

A decode step is memory-bound: it streams the worker's weight shard once.  The
stand-in does exactly that (``steps_bytes`` of HBM reads through a chain of
matrix-vector products over a weight-sized buffer), on the compute stream.
With 2 GPUs the context pool lives on GPU 0 and the decoding worker on GPU 1
(same process, peer access); with 1 GPU both live on it.
"""
from __future__ import annotations

import argparse
import json
import time
from dataclasses import dataclass
from typing import List

import numpy as np
import torch

from . import load_ops
from .config import CacheConfig, KVModelConfig, ParallelConfig
from .request import Request
from .stage import ContextStageEngine, DecodingStageEngine
from .worker import KVWorker
from .workloads import WORKLOADS


@dataclass
class LoopResult:
    mode: str
    total_ms: float
    steps: int
    migrations: int
    blocks: int
    p50_latency_ms: float
    max_latency_ms: float


class StandInDecoder:
    """Streams `weight_bytes` of HBM per step on the current stream."""

    def __init__(self, device: torch.device, weight_bytes: int, hidden: int = 4096) -> None:
        rows = max(1, weight_bytes // (2 * hidden))
        self.weights = torch.empty((rows, hidden), dtype=torch.float16, device=device).normal_(0, 0.02)
        self.x = torch.randn(hidden, 8, dtype=torch.float16, device=device)
        self.out = torch.empty((rows, 8), dtype=torch.float16, device=device)

    def step(self) -> None:
        torch.matmul(self.weights, self.x, out=self.out)


def _arrivals(rate_per_s: float, step_ms: float, steps: int, seed: int) -> List[int]:
    """Step index at which each request becomes visible to the decoding stage."""
    rng = np.random.default_rng(seed)
    horizon_s = steps * step_ms / 1e3
    t, out = 0.0, []
    while True:
        t += rng.exponential(1.0 / rate_per_s)
        if t >= horizon_s:
            return out
        out.append(int(t * 1e3 / step_ms))


# Kernel options for a migration that runs beside a decode step: 24 CTAs with deep rings (192 KiB each,
# about 4.5 MB in flight) keep the NVLink ingress as busy as the full grid does (685 vs 686 GB/s on awaited
# 168 MB calls) while leaving 124 of the 148 SMs to the step.
SIDE_BY_SIDE_OPTIONS = {"chunk_bytes": 32768, "stages": 6, "ctas_per_sm": 1, "max_ctas": 24}


def run(gpus: int = 1, steps: int = 400, rate: float = 4.0, workload: str = "c5", weight_gb: float = 6.7,
        pool_blocks: int = 1024, seed: int = 7, time_scale: float = 1.0, overlapped_options: dict = None) -> dict:
    """`time_scale` > 1 compresses arrival times so that a short run still sees many requests."""
    load_ops()
    from . import capi

    options = dict(SIDE_BY_SIDE_OPTIONS if overlapped_options is None else overlapped_options)
    saved = {k: capi.get_option(k) for k in options}
    try:
        with torch.cuda.device(1 if gpus >= 2 else 0):
            return _run(gpus, steps, rate, workload, weight_gb, pool_blocks, seed, time_scale, options, saved)
    finally:
        for k, v in saved.items():
            capi.set_option(k, v)


def _run(gpus, steps, rate, workload, weight_gb, pool_blocks, seed, time_scale, options, defaults) -> dict:
    from . import capi

    w = WORKLOADS[workload]
    model = KVModelConfig(w.model.num_layers, w.model.num_kv_heads // w.dec_tp, w.model.head_dim)   # one tp shard
    cache = CacheConfig(w.block_size, 1 << 20)
    ctx_dev, dec_dev = 0, (1 if gpus >= 2 else 0)
    pc = ParallelConfig()
    ctx_worker = KVWorker(0, "context", model, cache, pc, device=ctx_dev)
    dec_worker = KVWorker(1, "decoding", model, cache, pc, device=dec_dev)
    ctx_engine = ContextStageEngine(model, pc, cache, [[ctx_worker]])
    dec_engine = DecodingStageEngine(model, pc, cache, [[dec_worker]],
                                     clear_migrated_blocks_callback=ctx_engine.clear_migrated_blocks)
    handles = ctx_engine.init_kvcache(pool_blocks, 1)
    dec_engine.init_kvcache(pool_blocks, 1)
    ctx_worker.k_cache.normal_()
    ctx_worker.v_cache.normal_()
    dec_engine.register_kvcache_mem_handles(pc, handles)
    decoder = StandInDecoder(torch.device("cuda", dec_dev), int(weight_gb * 1e9))
    compute = torch.cuda.current_stream()
    side = torch.cuda.Stream(device=dec_dev)

    # step time alone
    for _ in range(5):
        decoder.step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(50):
        decoder.step()
    b.record()
    torch.cuda.synchronize()
    step_ms = a.elapsed_time(b) / 50

    rng = np.random.default_rng(seed)
    arrivals = _arrivals(rate * time_scale, step_ms, steps, seed)
    dist = w.length_dist
    lens = [int(min(dist[3], max(1, round(x)))) for x in rng.lognormal(np.log(dist[1]), dist[2], size=len(arrivals))]
    block_bytes = 2 * model.block_bytes(pc, w.block_size)

    def loop(mode: str) -> LoopResult:
        for k, v in (options if mode == "overlapped" else defaults).items():
            capi.set_option(k, v)
        # fresh bookkeeping for every run
        for eng in (ctx_engine, dec_engine):
            bm = eng.block_manager
            for rid in list(bm.block_table):
                bm.free_blocks(rid)
        pending, lat, blocks, resident = [], [], 0, []
        nxt = 0
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for step in range(steps):
            if mode != "decode_only":
                # retire finished tickets: the request joins the running batch
                still = []
                for ticket, started, rid in pending:
                    if step >= started + 1:
                        dec_worker.migrate_wait(ticket)
                        lat.append(time.perf_counter() - started_wall[rid])
                        ctx_engine.clear_migrated_blocks(migrating[rid])
                    else:
                        still.append((ticket, started, rid))
                pending = still
                while nxt < len(arrivals) and arrivals[nxt] <= step:
                    rid = nxt
                    req = Request.of_length(rid, lens[rid])
                    need = -(-lens[rid] // w.block_size)
                    while dec_engine.block_manager.get_num_avail_gpu_blocks() < need:
                        dec_engine.block_manager.free_blocks(resident.pop(0))
                    m = ctx_engine.finish_prefill(req)
                    migrating[rid] = m
                    blocks += need
                    resident.append(rid)
                    if mode == "bookkeeping":
                        dec_engine.block_manager.allocate_blocks(req)
                        ctx_engine.clear_migrated_blocks(m)
                        lat.append(0.0)
                    elif mode == "serial":
                        t1 = time.perf_counter()
                        dec_engine.migrate_blocks(m)              # awaited; frees the context blocks itself
                        lat.append(time.perf_counter() - t1)
                    else:
                        dec_engine.block_manager.allocate_blocks(req)
                        target = dec_engine.block_manager.get_block_table(rid)
                        started_wall[rid] = time.perf_counter()
                        ticket = dec_worker.migrate_blocks_async(m.block_indexes, pc, target, stream=side)
                        pending.append((ticket, step, rid))
                    nxt += 1
            decoder.step()
            compute.synchronize()          # a real step returns sampled tokens to the host
        for ticket, _, rid in pending:
            dec_worker.migrate_wait(ticket)
            lat.append(time.perf_counter() - started_wall[rid])
            ctx_engine.clear_migrated_blocks(migrating[rid])
        torch.cuda.synchronize()
        total = (time.perf_counter() - t0) * 1e3
        lat.sort()
        return LoopResult(mode, total, steps, len(lat), blocks, (lat[len(lat) // 2] * 1e3) if lat else 0.0,
                          (lat[-1] * 1e3) if lat else 0.0)

    migrating, started_wall = {}, {}
    results = {}
    for mode in ("decode_only", "bookkeeping", "serial", "overlapped") * 2:
        migrating.clear()
        started_wall.clear()
        r = loop(mode)
        if mode not in results or r.total_ms < results[mode].total_ms:
            results[mode] = r                                         # best of two passes

    # the last overlapped pass left every accepted request's blocks in the decoding pool: check them
    verified = True
    bm = dec_engine.block_manager
    for rid in list(bm.block_table)[-8:]:
        src = torch.tensor(migrating[rid].block_indexes, device=ctx_worker.device)
        dst = torch.tensor(bm.get_block_table(rid), device=dec_worker.device)
        # context blocks were recycled after the ticket completed, but nothing rewrote them in this harness
        verified &= bool(torch.equal(dec_worker.k_cache[dst].cpu(), ctx_worker.k_cache[src].cpu()))
        verified &= bool(torch.equal(dec_worker.v_cache[dst].cpu(), ctx_worker.v_cache[src].cpu()))

    base, bk, ser, ov = results["decode_only"], results["bookkeeping"], results["serial"], results["overlapped"]
    n = max(1, ov.migrations)
    added_serial = (ser.total_ms - bk.total_ms) / max(1, ser.migrations)
    added_overlap = (ov.total_ms - bk.total_ms) / n
    return {
        "workload": w.name, "gpus": gpus, "steps": steps, "decode_step_ms": step_ms,
        "stand_in_bytes_per_step": decoder.weights.numel() * 2, "arrival_rate_per_s": rate, "time_scale": time_scale,
        "migrations": ov.migrations, "blocks_migrated": ov.blocks, "mean_request_MB": ov.blocks * block_bytes / n / 1e6,
        "loop_ms": {"decode_only": base.total_ms, "bookkeeping": bk.total_ms, "serial": ser.total_ms,
                    "overlapped": ov.total_ms},
        "added_ms_per_migration_over_bookkeeping": {"serial": added_serial, "overlapped": added_overlap},
        "hidden_fraction": None if added_serial <= 0 else max(0.0, 1.0 - added_overlap / added_serial),
        "p50_migrate_latency_ms": {"serial": ser.p50_latency_ms, "overlapped": ov.p50_latency_ms},
        "overlapped_kernel_options": options,
        "verified": verified,
    }


def run_swap(steps: int = 300, weight_gb: float = 6.7, workload: str = "c5", pool_blocks: int = 1024,
             request_blocks: int = 32, every: int = 10, seed: int = 11) -> dict:
    """Decode steps with a request swapped out to pinned host memory and back in every `every` steps, the
    way the decoding scheduler does under memory pressure (distserve/decoding_stage_scheduler.py:183-223 via
    distserve/block_manager.py:288-315, which fires the copies and never awaits them).

    * ``awaited``    — the loop waits for each swap before the next step (what a blocking copy would cost);
    * ``overlapped`` — the copies run on the worker's swap streams beside the steps; as in the reference,
      the swapped-in request is in the very next batch, whose step therefore waits for the swap-in
      (``prepare_step`` makes the compute stream wait for it), so only swap-outs are hidden;
    * ``deferred``   — as above, but the request rejoins the batch at the first step boundary at which its
      swap-in event has completed, so swap-ins are hidden too.
    Returns the loop times and the swapped data's integrity check."""
    load_ops()
    from .block_manager import BlockManager

    with torch.cuda.device(0):
        w = WORKLOADS[workload]
        model = KVModelConfig(w.model.num_layers, w.model.num_kv_heads // w.dec_tp, w.model.head_dim)
        cache = CacheConfig(w.block_size, 1 << 20)
        worker = KVWorker(0, "decoding", model, cache, ParallelConfig(), device=0)
        worker.init_kvcache_and_swap(pool_blocks, 4 * request_blocks)
        worker.k_cache.normal_()
        worker.v_cache.normal_()
        bm = BlockManager("decoding", pool_blocks, 4 * request_blocks, model, ParallelConfig(), cache,
                          lambda name, *args: [getattr(worker, name)(*args)])
        req = Request.of_length(0, request_blocks * w.block_size)
        bm.allocate_blocks(req)
        first_ids = list(bm.get_block_table(0))
        want_k, want_v = worker.k_cache[first_ids].clone(), worker.v_cache[first_ids].clone()
        decoder = StandInDecoder(torch.device("cuda", 0), int(weight_gb * 1e9))
        compute = torch.cuda.current_stream()
        swap_bytes = 2 * request_blocks * model.block_bytes(ParallelConfig(), w.block_size)

        def loop(mode: str) -> float:
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            away = False
            rejoin_pending = False
            for step in range(steps):
                if mode != "decode_only" and step % every == every - 1:
                    if not away:
                        bm.swap_out_requests([req])
                        if mode == "awaited":
                            worker.wait_for_all_swap_out()
                    else:
                        bm.swap_in_requests([req])
                        if mode == "awaited":
                            worker.wait_for_all_swap_in()
                        if mode == "deferred":
                            rejoin_pending = True
                        else:
                            worker.prepare_step([0])       # the request's next step waits for its swap-in
                    away = not away
                if rejoin_pending and worker.swap_finished(0):
                    worker.prepare_step([0])               # already complete: rejoins without stalling the step
                    rejoin_pending = False
                decoder.step()
                compute.synchronize()
            if away:
                bm.swap_in_requests([req])
                worker.prepare_step([0])
            worker.wait_for_all_swap_out()
            worker.wait_for_all_swap_in()
            torch.cuda.synchronize()
            return (time.perf_counter() - t0) * 1e3

        times = {}
        for mode in ("decode_only", "awaited", "overlapped", "deferred") * 2:
            t = loop(mode)
            times[mode] = min(t, times.get(mode, t))
        ids = list(bm.get_block_table(0))
        intact = bool(torch.equal(worker.k_cache[ids], want_k) and torch.equal(worker.v_cache[ids], want_v))
        n = max(1, steps // every)
        return {"steps": steps, "swap_every_steps": every, "bytes_per_swap": swap_bytes, "swaps": n,
                "loop_ms": times,
                "added_ms_per_swap": {m: (times[m] - times["decode_only"]) / n for m in ("awaited", "overlapped", "deferred")},
                "hidden_fraction": {m: max(0.0, 1.0 - (times[m] - times["decode_only"]) /
                                           max(1e-9, times["awaited"] - times["decode_only"]))
                                    for m in ("overlapped", "deferred")},
                "data_intact_after_round_trips": intact}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--swap", action="store_true", help="measure swap-out/in beside decode steps instead of migration")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--rate", type=float, default=4.0)
    ap.add_argument("--workload", default="c5")
    ap.add_argument("--weight-gb", type=float, default=6.7)
    ap.add_argument("--time-scale", type=float, default=50.0)
    ap.add_argument("--opt", action="append", default=None, metavar="NAME=VALUE",
                    help="kernel option for the overlapped run (replaces the side-by-side defaults)")
    args = ap.parse_args()
    if args.swap:
        print(json.dumps(run_swap(steps=args.steps, weight_gb=args.weight_gb, workload=args.workload)))
        return
    options = None if args.opt is None else {k: int(v) for k, v in (pair.split("=") for pair in args.opt)}
    print(json.dumps(run(args.gpus, args.steps, args.rate, args.workload, args.weight_gb, time_scale=args.time_scale,
                         overlapped_options=options)))


if __name__ == "__main__":
    main()

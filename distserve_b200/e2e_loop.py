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
from typing import List, Optional

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
    return poisson_arrival_steps(rate_per_s, step_ms, steps, seed)


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


# ----------------------------------------------------------------------------------------------------------
# The same loop at its stated layout: one worker process per GPU, driven by a controller
# ----------------------------------------------------------------------------------------------------------

class LoopWorker(KVWorker):
    """A stage worker living in its own process (``actors.ActorPool``), with what the loop needs on top of the KV
    methods: a stand-in decode step, and ONE method per iteration that carries the iteration's scheduling
    decisions — the way the reference's ``step`` call carries the batch's block tables — so that every mode of
    the loop costs the same number of calls into the worker."""

    def fill_pools(self, seed: int) -> None:
        g = torch.Generator(device=self.device).manual_seed(seed)
        for pool in (self.k_cache, self.v_cache):
            pool.normal_(generator=g)
        torch.cuda.synchronize(self.device)

    def setup_decoder(self, weight_bytes: int) -> float:
        """Build the stand-in and return its step time in ms (50 steps after warm-up)."""
        with torch.cuda.device(self.device):
            self.decoder = StandInDecoder(self.device, weight_bytes)
            self.side = torch.cuda.Stream(device=self.device)
            for _ in range(5):
                self.decoder.step()
            torch.cuda.synchronize(self.device)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(50):
                self.decoder.step()
            b.record()
            torch.cuda.synchronize(self.device)
            return a.elapsed_time(b) / 50

    def set_options(self, options: dict) -> dict:
        from . import capi

        saved = {k: capi.get_option(k) for k in options}
        for k, v in options.items():
            capi.set_option(k, v)
        return saved

    def loop_iteration(self, mode: str, migrations, context_parallel_config, wait_tickets):
        """One iteration of the decoding loop on this worker.  `migrations` = [(source ids, target ids)] of the
        requests accepted at this step boundary; `wait_tickets` = tickets of copies enqueued at an earlier
        boundary whose requests join the batch now.  serial: each accepted request is pulled with the awaited
        operator before the step; overlapped: the pulls are enqueued on the side stream and the step starts at
        once.  Returns (tickets of the copies enqueued now, seconds spent in awaited pulls)."""
        with torch.cuda.device(self.device):
            for t in wait_tickets:
                self.migrate_wait(t)
            tickets, awaited = [], 0.0
            for src, dst in migrations:
                if mode == "serial":
                    t0 = time.perf_counter()
                    self.migrate_blocks(src, context_parallel_config, dst)
                    awaited += time.perf_counter() - t0
                elif mode == "overlapped":
                    tickets.append(self.migrate_blocks_async(src, context_parallel_config, dst, stream=self.side))
            self.decoder.step()
            torch.cuda.current_stream().synchronize()      # a real step returns sampled tokens to the host
            return tickets, awaited

    def read_blocks(self, block_ids):
        """The listed blocks of both pools as bit patterns on the host (for the controller's check)."""
        idx = torch.as_tensor(list(block_ids), dtype=torch.int64, device=self.device)
        torch.cuda.synchronize(self.device)
        return (self.k_cache.view(torch.int16).index_select(0, idx).cpu().numpy(),
                self.v_cache.view(torch.int16).index_select(0, idx).cpu().numpy())


def make_loop_worker(worker_id: int, stage: str, model: KVModelConfig, cache: CacheConfig, pc_list, device: int) -> LoopWorker:
    """Factory run inside the worker process.  On a machine with fewer GPUs than workers the workers share them."""
    device = device % torch.cuda.device_count()
    torch.cuda.set_device(device)
    tp, t, pp, p = pc_list
    return LoopWorker(worker_id, stage, model, cache, ParallelConfig(tp, t, pp, p), device=device)


def poisson_arrival_steps(rate_per_s: float, step_ms: float, steps: int, seed: int) -> List[int]:
    """Step index at which each request becomes visible to the decoding stage.  Inter-arrival times are
    gamma(shape 1, scale 1/rate) draws, the reference load generator's Poisson process
    (evaluation/2-benchmark-serving/2-benchmark-serving.py:49-53)."""
    rng = np.random.default_rng(seed)
    horizon_s = steps * step_ms / 1e3
    t, out = 0.0, []
    while True:
        t += rng.gamma(shape=1.0, scale=1.0 / rate_per_s)
        if t >= horizon_s:
            return out
        out.append(int(t * 1e3 / step_ms))


def _one_shard_of(w):
    """The workload as ONE tensor-parallel rank of each stage sees it (equal layouts only): that rank's share of the
    KV heads, tp = 1 on both sides.  Two worker processes instead of 2 x tp."""
    from dataclasses import replace

    assert w.ctx_tp == w.dec_tp and w.ctx_pp == w.dec_pp == 1, "a single shard stands for the stage only with equal layouts"
    model = KVModelConfig(w.model.num_layers, w.model.num_kv_heads // w.dec_tp, w.model.head_dim, w.model.dtype)
    return replace(w, name=w.name + "-one-shard", model=model, ctx_tp=1, dec_tp=1)


def _run_replica(pool, devices, w, steps, rate, weight_gb, pool_blocks, seed, time_scale, options, passes, tag) -> dict:
    """Context tp x pp workers on the first devices, decoding tp x pp workers on the next ones; one replica."""
    cache = CacheConfig(w.block_size, 1 << 20)
    n_ctx, n_dec = w.ctx_tp * w.ctx_pp, w.dec_tp * w.dec_pp
    ctx_pc, dec_pc = w.ctx_config(), w.dec_config()
    # the worker processes come up side by side (each spends most of its start-up importing torch)
    from concurrent.futures import ThreadPoolExecutor

    with ThreadPoolExecutor(max_workers=n_ctx + n_dec) as starter:
        ctx_starting = [[starter.submit(pool.spawn, make_loop_worker, p * w.ctx_tp + t, "context", w.model, cache,
                                        [w.ctx_tp, t, w.ctx_pp, p], devices[(p * w.ctx_tp + t) % len(devices)])
                         for t in range(w.ctx_tp)] for p in range(w.ctx_pp)]
        dec_starting = [[starter.submit(pool.spawn, make_loop_worker, n_ctx + p * w.dec_tp + t, "decoding", w.model, cache,
                                        [w.dec_tp, t, w.dec_pp, p], devices[(n_ctx + p * w.dec_tp + t) % len(devices)])
                         for t in range(w.dec_tp)] for p in range(w.dec_pp)]
        ctx_workers = [[f.result() for f in row] for row in ctx_starting]
        dec_workers = [[f.result() for f in row] for row in dec_starting]
    ctx_engine = ContextStageEngine(w.model, ctx_pc, cache, ctx_workers)
    dec_engine = DecodingStageEngine(w.model, dec_pc, cache, dec_workers,
                                     clear_migrated_blocks_callback=ctx_engine.clear_migrated_blocks)
    handles = ctx_engine.init_kvcache(pool_blocks, 1)
    dec_engine.init_kvcache(pool_blocks, 1)
    flat_ctx = [x for row in ctx_workers for x in row]
    flat_dec = [x for row in dec_workers for x in row]
    for i, worker in enumerate(flat_ctx):
        worker.fill_pools(seed * 100 + i).result()
    dec_engine.register_kvcache_mem_handles(ctx_pc, handles)
    # a decode step streams the worker's weight shard once
    step_ms = max(f.result() for f in [worker.setup_decoder(int(weight_gb * 1e9)) for worker in flat_dec])

    arrivals = poisson_arrival_steps(rate * time_scale, step_ms, steps, seed)
    rng = np.random.default_rng(seed)
    dist = w.length_dist
    lens = [int(min(dist[3], max(1, round(x)))) for x in rng.lognormal(np.log(dist[1]), dist[2], size=len(arrivals))]
    block_bytes = w.dec_block_bytes()
    migrating = {}

    def loop(mode: str) -> LoopResult:
        defaults = [f.result() for f in [worker.set_options(options if mode == "overlapped" else {}) for worker in flat_dec]]
        for eng in (ctx_engine, dec_engine):
            bm = eng.block_manager
            for rid in list(bm.block_table):
                bm.free_blocks(rid)
        migrating.clear()
        pending, awaited, blocks, resident, done = [], [], 0, [], 0
        nxt = 0
        t0 = time.perf_counter()
        for step in range(steps):
            accepted = []
            if mode != "decode_only":
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
                    dec_engine.block_manager.allocate_blocks(req)
                    if mode != "bookkeeping":
                        accepted.append((list(m.block_indexes), list(dec_engine.block_manager.get_block_table(rid))))
                    if mode != "overlapped":
                        ctx_engine.clear_migrated_blocks(m)      # awaited inside this iteration (or no copy at all)
                    done += 1
                    nxt += 1
            # copies enqueued at the previous boundary are awaited now: their requests join this batch
            waits, pending_rids = [p[0] for p in pending], [p[1] for p in pending]
            futures = [worker.loop_iteration(mode, accepted, ctx_pc, [wt[i] for wt in waits])
                       for i, worker in enumerate(flat_dec)]
            results = [f.result() for f in futures]
            for rids in pending_rids:
                for rid in rids:
                    ctx_engine.clear_migrated_blocks(migrating[rid])
            pending = []
            if mode == "overlapped" and accepted:
                tickets_per_worker = [r[0] for r in results]                       # [worker][migration]
                per_migration = [[tw[j] for tw in tickets_per_worker] for j in range(len(accepted))]
                first = done - len(accepted)
                pending = [(per_migration[j], [first + j]) for j in range(len(accepted))]
            if mode == "serial" and accepted:
                awaited.append(max(r[1] for r in results) / len(accepted))
        # copies still in flight after the last step
        if pending:
            for i, worker in enumerate(flat_dec):
                for tickets, _ in pending:
                    worker.migrate_wait(tickets[i]).result()
            for _, rids in pending:
                for rid in rids:
                    ctx_engine.clear_migrated_blocks(migrating[rid])
        total = (time.perf_counter() - t0) * 1e3
        for worker, saved in zip(flat_dec, defaults):
            worker.set_options(saved).result()
        awaited.sort()
        return LoopResult(mode, total, steps, done, blocks, (awaited[len(awaited) // 2] * 1e3) if awaited else 0.0,
                          (awaited[-1] * 1e3) if awaited else 0.0)

    results = {}
    for mode in ("decode_only", "bookkeeping", "serial", "overlapped") * passes:
        r = loop(mode)
        if mode not in results or r.total_ms < results[mode].total_ms:
            results[mode] = r                                         # best pass per mode

    # The last pass was an overlapped one: its accepted requests' blocks are still in the decoding pools, and nothing
    # rewrote the context blocks they came from.  A decoding worker's block must equal what the oracle-free
    # geometry says: with equal layouts on both sides, the whole block of the context worker at the same position.
    verified = None
    bm = dec_engine.block_manager
    if (w.ctx_tp, w.ctx_pp) == (w.dec_tp, w.dec_pp):
        verified = True
        for rid in list(bm.block_table)[-8:]:
            src_ids, dst_ids = migrating[rid].block_indexes, bm.get_block_table(rid)
            picks = sorted(set(range(0, len(src_ids), max(1, len(src_ids) // 4))))[:4]
            for cw, dw in zip(flat_ctx, flat_dec):
                sk, sv = cw.read_blocks([src_ids[i] for i in picks]).result()
                dk, dv = dw.read_blocks([dst_ids[i] for i in picks]).result()
                verified &= bool(np.array_equal(sk, dk) and np.array_equal(sv, dv))

    base, bk, ser, ov = results["decode_only"], results["bookkeeping"], results["serial"], results["overlapped"]
    n = max(1, ov.migrations)
    added_serial = (ser.total_ms - bk.total_ms) / max(1, ser.migrations)
    added_overlap = (ov.total_ms - bk.total_ms) / n
    return {
        "replica": tag, "devices": list(devices), "decode_step_ms": step_ms, "migrations": ov.migrations,
        "blocks_migrated": ov.blocks, "mean_request_MB_per_dest": ov.blocks * block_bytes / n / 1e6,
        "loop_ms": {"decode_only": base.total_ms, "bookkeeping": bk.total_ms, "serial": ser.total_ms, "overlapped": ov.total_ms},
        "added_us_per_migration_awaited": added_serial * 1e3, "added_us_per_migration_overlapped": added_overlap * 1e3,
        "hidden_fraction": None if added_serial <= 0 else max(0.0, 1.0 - added_overlap / added_serial),
        "p50_awaited_call_ms": ser.p50_latency_ms, "verified": verified,
    }


def run_actors(n_gpus: int = 4, steps: int = 400, rate: float = 4.0, workload: str = "c5", weight_gb: float = 6.7,
               pool_blocks: int = 1024, seed: int = 7, time_scale: float = 50.0, overlapped_options: dict = None,
               passes: int = 2, device_offset: int = 0, deadline_s: float = 600.0, one_shard: bool = False) -> dict:
    """The loop at the stated layout of the end-to-end configuration: every worker in its own process on its own
    GPU (context tp=2 on the first two GPUs, decoding tp=2 on the next two), driven from this process, which
    needs no GPU itself; with 8 GPUs a second, independent replica runs at the same time on GPUs 4-7.  With
    fewer than 4 GPUs the workers share the GPUs that exist; `one_shard` runs one tensor-parallel rank of each stage
    instead (two worker processes: what a 2-GPU machine can run without two workers sharing a GPU).  `deadline_s`
    bounds the whole run.  Arrivals are the reference generator's Poisson
    process at `rate` requests per second per replica, compressed by `time_scale` so that a short run sees
    many requests; prompt lengths follow the workload's distribution."""
    import threading

    from .actors import ActorPool

    w = _one_shard_of(WORKLOADS[workload]) if one_shard else WORKLOADS[workload]
    per_replica = w.ctx_tp * w.ctx_pp + w.dec_tp * w.dec_pp
    n_replicas = max(1, n_gpus // per_replica)
    options = dict(SIDE_BY_SIDE_OPTIONS if overlapped_options is None else overlapped_options)
    outs: List[Optional[dict]] = [None] * n_replicas
    errors: List[BaseException] = []
    with ActorPool() as pool:
        def one(r: int) -> None:
            try:
                if n_gpus >= per_replica:
                    devices = [device_offset + r * per_replica + i for i in range(per_replica)]
                else:
                    devices = [device_offset + i for i in range(max(1, n_gpus))]
                outs[r] = _run_replica(pool, devices, w, steps, rate, weight_gb, pool_blocks, seed + r, time_scale,
                                       options, passes, r)
            except BaseException as e:      # surfaced below, after the other replica has ended
                errors.append(e)

        threads = [threading.Thread(target=one, args=(r,), daemon=True) for r in range(n_replicas)]
        started = time.perf_counter()
        for t in threads:
            t.start()
        for t in threads:
            t.join(max(0.0, deadline_s - (time.perf_counter() - started)))
        if any(t.is_alive() for t in threads):
            # A worker process that no longer answers must not hold the caller for ever: stopping the pool ends the
            # worker processes this call started, which makes every pending call fail and the threads return.
            pool.stop(timeout=2.0)
            for t in threads:
                t.join(30)
            raise TimeoutError(f"the serving loop did not finish within {deadline_s:.0f} s")
    if errors:
        raise errors[0]
    fractions = [o["hidden_fraction"] for o in outs if o["hidden_fraction"] is not None]
    return {
        "workload": w.name, "layout": f"context tp{w.ctx_tp}pp{w.ctx_pp} -> decoding tp{w.dec_tp}pp{w.dec_pp}, one process per GPU",
        "gpus": n_gpus, "replicas": n_replicas, "steps": steps, "arrival_rate_per_s_per_replica": rate, "time_scale": time_scale,
        "stand_in_bytes_per_step": int(weight_gb * 1e9), "overlapped_kernel_options": options,
        "hidden_fraction": min(fractions) if fractions else None,
        "added_us_per_migration_awaited": max(o["added_us_per_migration_awaited"] for o in outs),
        "added_us_per_migration_overlapped": max(o["added_us_per_migration_overlapped"] for o in outs),
        "verified": all(o["verified"] is True for o in outs), "per_replica": outs,
    }


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--swap", action="store_true", help="measure swap-out/in beside decode steps instead of migration")
    ap.add_argument("--actors", action="store_true", help="one worker process per GPU, context tp2 -> decoding tp2 per 4 GPUs")
    ap.add_argument("--pool-blocks", type=int, default=1024)
    ap.add_argument("--one-shard", action="store_true", help="with --actors: one tensor-parallel rank of each stage (2 processes)")
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
    if args.actors:
        print(json.dumps(run_actors(args.gpus, args.steps, args.rate, args.workload, args.weight_gb, pool_blocks=args.pool_blocks,
                                    time_scale=args.time_scale, overlapped_options=options, one_shard=args.one_shard)))
        return
    print(json.dumps(run(args.gpus, args.steps, args.rate, args.workload, args.weight_gb, time_scale=args.time_scale,
                         overlapped_options=options)))


if __name__ == "__main__":
    main()

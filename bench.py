#!/usr/bin/env python
"""KV-block migration benchmark.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" migrates every request of the workload once.  After W warm-up steps,
regions of K steps each are timed on the device (CUDA events on the launching
stream, barrier + synchronize on both sides, max over ranks):

* ``value``       — one launch per request, enqueued back to back through the
  asynchronous C-ABI entry point; KV pools resident in HBM.  The launches run
  back to back on one stream, so the roofline figure uses region time / launches
  as the average launch duration (an event between launches would serialise
  launches that the library lets overlap).
* ``e2e``         — the call a DistServe worker makes, at the reference's
  cadence (distserve/single_stage_engine.py:490-536): one awaited
  ``torch.ops.block_migration_ops.migrate_blocks`` per request with Python
  block-index lists, returning only when the source blocks may be recycled.
  The host->device traffic of this path is the block tables, the device->host
  traffic the kernel's status words; the KV payload is device-resident by the
  operator's contract (it takes CUDA tensors).
* ``batched``     — the C ABI with the concatenated lists of consecutive
  requests (up to 4096 blocks, distinct targets) per launch.
* ``e2e_batched`` — the same cadence through the package's own host API with
  plain Python lists: ``DecodingStageFCFSScheduler.post_process_pipelined`` ->
  ``DecodingStageEngine.begin/finish_migrate_blocks_batched`` ->
  ``KVWorker.migrate_blocks_async``; the scheduler decides how many requests
  each launch carries, the block manager hands out the target blocks.

After the timed regions the result is checked: on one GPU the whole-request
read-back below runs in-process; on several GPUs every contributing context
rank copies sampled requests' source blocks from its own pool to the host and
sends them over gloo, the decoding rank copies its own target blocks to the
host, the CPU oracle re-executes the migration on those slices and the two are
compared bit for bit; target blocks that no request names must still hold what
they held before warm-up.  A mismatch ends the run with a non-zero status.

Workload by GPU count (override with --workload):
  1  c2 shapes, context and decoding pools on the same GPU (HBM-bound)
  2  c2: GPU0 -> GPU1
  4  c3: context tp=2 on GPUs 0-1 -> two decoding tp=1 replicas on GPUs 2, 3
  8  c4: context tp=4,pp=1 on GPUs 0-3 -> decoding tp=2,pp=2 on GPUs 4-7
On 4 and 8 GPUs the serving loop of the end-to-end configuration (context tp=2
-> decoding tp=2, one worker process per GPU, stand-in decode steps) then runs
from rank 0 and its result is reported as ``overlap``.
Each rank prints nothing except rank 0's single JSON line.
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
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "kv_migration_GBps_whole_job"
UNIT = "GB/s"
NVLINK_NOMINAL_GBS = 900.0      # per direction per GPU
HBM_FALLBACK_GBS = 6650.0

DEFAULT_WORKLOAD = {1: "c2", 2: "c2", 4: "c3", 8: "c4"}


def parse_args(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, help="c1..c5 (default depends on --gpus)")
    ap.add_argument("--requests", type=int, default=None, help="use only the first R requests of the workload")
    ap.add_argument("--pool-blocks", type=int, default=None, help="override both pool sizes (small captures)")
    ap.add_argument("--kernel", type=int, default=None, help="0 auto, 1 vector, 2 bulk")
    ap.add_argument("--chunk-bytes", type=int, default=None)
    ap.add_argument("--stages", type=int, default=None)
    ap.add_argument("--ctas-per-sm", type=int, default=None)
    ap.add_argument("--opt", action="append", default=[], metavar="NAME=VALUE", help="any kvmig_set_option pair")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="budget of the CPU baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-swap", action="store_true")
    ap.add_argument("--no-other-workloads", action="store_true", help="N=1: skip the short c1 and c5 runs")
    ap.add_argument("--no-overlap", action="store_true", help="N=4/8: skip the serving loop with stand-in decode steps")
    ap.add_argument("--only-value", action="store_true", help="time the value region only (profiler captures)")
    ap.add_argument("--wave-blocks", type=int, default=4096, help="most blocks one launch of the `batched` leg carries")
    ap.add_argument("--peer-in-process", action="store_true",
                    help="one process, two GPUs: every context worker on GPU 0, decoding worker (0,0) on GPU 1 "
                         "(a single-process cross-GPU case, e.g. for a profiler capture)")
    return ap.parse_args(argv)


# ----------------------------------------------------------------------------------------------
# helpers
# ----------------------------------------------------------------------------------------------

def hbm_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return HBM_FALLBACK_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []          # (arrival time, cells)
        self.proc = None
        self.thread = None
        self.window = [None, None]

    def mark(self, which: int):
        """0: the timed region starts, 1: it ends."""
        self.window[which] = time.perf_counter()

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        t0, t1 = self.window
        inside = [r for t, r in self.rows if t0 is not None and t1 is not None and t0 <= t <= t1 + 0.05]
        for r in inside or [r for _, r in self.rows[-3:]]:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                smax.append(float(r[1]))
            except ValueError:
                continue
            for name, cell in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "samples_inside_timed_region": len(inside), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------------------------
# CPU arm: the oracle's torch gather/scatter on the host cores
# ----------------------------------------------------------------------------------------------

CPU_SAMPLE_REQUESTS = 8
CPU_SAMPLE_POOL_BLOCKS = 256


def cpu_sample(workload, trace):
    """The bounded sample the CPU arms run: the first requests of the trace that fit the compact pools, block
    ids folded into them (targets made distinct again where folding collides)."""
    sample = []
    for item in trace:
        if len(item.src_blocks) <= CPU_SAMPLE_POOL_BLOCKS:
            src = [i % CPU_SAMPLE_POOL_BLOCKS for i in item.src_blocks]
            dst = [i % CPU_SAMPLE_POOL_BLOCKS for i in item.dst_blocks]
            seen, s2, d2 = set(), [], []
            for a, b in zip(src, dst):
                if b not in seen:
                    seen.add(b)
                    s2.append(a)
                    d2.append(b)
            sample.append((s2, d2))
        if len(sample) == CPU_SAMPLE_REQUESTS:
            break
    return sample


def cpu_baseline(workload, trace, same_device: bool, seconds: float = None, passes: int = None, warmup_passes: int = 1):
    """The oracle's torch gather/scatter on host tensors with every host thread, one call per request, on the
    sample of :func:`cpu_sample`.  Either `passes` timed passes of the sample, or as many as fit `seconds`."""
    import torch

    from oracle import kv_oracle as O

    # every host core, also under torchrun (which exports OMP_NUM_THREADS=1 to its ranks)
    torch.set_num_threads(os.cpu_count() or 1)
    w = workload
    sample = cpu_sample(w, trace)
    dt = w.model.get_torch_dtype()
    ctx_pools = {}
    for p in range(w.ctx_pp):
        for t in range(w.ctx_tp):
            pc = w.ctx_config(p, t)
            shape = (CPU_SAMPLE_POOL_BLOCKS, w.model.get_num_layers(pc), w.model.get_num_heads(pc), w.block_size, w.model.head_dim)
            ctx_pools[(p, t)] = (torch.randn(shape, dtype=torch.float32).to(dt), torch.randn(shape, dtype=torch.float32).to(dt))
    pc = w.dec_config()
    dshape = (CPU_SAMPLE_POOL_BLOCKS, w.model.get_num_layers(pc), w.model.get_num_heads(pc), w.block_size, w.model.head_dim)
    dec_pools = {(p, t): (torch.zeros(dshape, dtype=dt), torch.zeros(dshape, dtype=dt))
                 for p in range(w.dec_pp) for t in range(w.dec_tp)}
    factor = 2 if same_device else 1
    sample_blocks = sum(len(d) for _, d in sample)

    def one_pass(migrate):
        moved = 0
        for s2, d2 in sample:
            for (p, t), (k, v) in dec_pools.items():
                migrate(ctx_pools, w.ctx_tp, w.ctx_pp, s2, w.dec_tp, t, w.dec_pp, p, d2, k, v,
                        w.model.num_layers, w.model.num_kv_heads)
                moved += len(d2) * w.dec_block_bytes()
        return moved

    def timed_passes(fn, budget, fixed, warm):
        for _ in range(max(1, warm)):
            one_pass(fn)   # warm-up: pages in the pools
        t0 = time.perf_counter()
        moved, done = 0, 0
        while True:
            moved += one_pass(fn)
            done += 1
            if (fixed is not None and done >= fixed) or (fixed is None and time.perf_counter() - t0 >= budget):
                break
        return moved, done, time.perf_counter() - t0

    moved, done, dt_s = timed_passes(O.migrate_blocks_torch, seconds, passes, warmup_passes)
    out = {"value": factor * moved / dt_s / 1e9, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
           "ms_per_sample_pass": dt_s * 1e3 / done, "passes": done, "warmup_passes": max(1, warmup_passes),
           "sample_requests": len(sample), "sample_blocks": sample_blocks, "sample_pool_blocks": CPU_SAMPLE_POOL_BLOCKS,
           "sample": f"first {len(sample)} requests of {w.name} ({sample_blocks} blocks), ids folded into "
                     f"{CPU_SAMPLE_POOL_BLOCKS}-block host pools, {done} passes in {dt_s:.1f} s, torch "
                     f"index_select/index_copy_ on {torch.get_num_threads()} threads"}
    # the same semantics as plain C (one memcpy per run, OpenMP over blocks x layers): a stronger CPU arm, for context
    try:
        from oracle import kv_oracle_c as OC

        budget_c = max(2.0, (seconds or dt_s) / 4)
        moved_c, passes_c, dt_c = timed_passes(OC.migrate_blocks_c, budget_c, None, 1)
        out["c_openmp"] = {"value": factor * moved_c / dt_c / 1e9, "unit": UNIT, "cores": os.cpu_count(),
                           "sample": f"same sample, {passes_c} passes in {dt_c:.1f} s, oracle/kv_oracle.c"}
    except Exception as e:   # gcc missing on the box: the torch arm stands alone
        out["c_openmp"] = {"unavailable": str(e)[:200]}
    return out


def reference_arm(args, w, trace, config, same_device):
    """``--impl reference``: the CPU restatement of the reference's semantics for this path, timed on the host
    cores.  A step of this arm is one pass over the bounded sample; --warmup / --steps are passes."""
    from distserve_b200.workloads import trace_blocks

    base = cpu_baseline(w, trace, same_device, passes=max(1, args.steps), warmup_passes=max(1, args.warmup))
    full_step_ms = base["ms_per_sample_pass"] * trace_blocks(trace) / max(1, base["sample_blocks"])
    assert (config["sample_requests"], config["sample_blocks"]) == (base["sample_requests"], base["sample_blocks"])
    return {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": base["passes"], "warmup": base["warmup_passes"], "ms_per_step": full_step_ms,
            "ms_per_step_basis": "extrapolated: time of one sample pass x (blocks of a full step / blocks of the sample)",
            "ms_per_sample_pass": base["ms_per_sample_pass"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": config, "step_is": "one pass over config.sample_requests requests, not over all requests of the workload",
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "the reference's native copy (SwiftTransformer) is not in its tree; this arm is the CPU "
                    "restatement of its semantics (oracle/kv_oracle.py), torch host-tensor gather/scatter"}


# ----------------------------------------------------------------------------------------------
# the checker: oracle on read-back slices
# ----------------------------------------------------------------------------------------------

def check_readbacks(workload, readbacks):
    """Re-execute each sampled request's migration with the CPU oracle on the read-back source slices and compare
    the result with the blocks the decoding worker holds, by bit pattern.  Returns (samples, blocks, mismatches)."""
    import numpy as np

    from oracle import kv_oracle as O

    w = workload
    blocks, bad = 0, []
    for rb in readbacks:
        s = rb.sample
        n = len(s.src_blocks)
        got_k, got_v = rb.target
        want_k, want_v = np.zeros_like(got_k), np.zeros_like(got_v)
        O.migrate_blocks_numpy(rb.ctx_pools, w.ctx_tp, w.ctx_pp, list(range(n)), w.dec_tp, s.dec_tp_rank, w.dec_pp, s.dec_pp_rank,
                               list(range(n)), want_k, want_v, w.model.num_layers, w.model.num_kv_heads)
        blocks += n
        if not (np.array_equal(got_k, want_k) and np.array_equal(got_v, want_v)):
            bad.append((s.dec_rank, s.request_id))
    return len(readbacks), blocks, bad


def untouched_checksum(worker, block_ids):
    """Sum of the bit patterns of the listed blocks of both pools (exact, 64-bit wrap-around)."""
    import torch

    width = {1: torch.int8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[worker.k_cache.element_size()]
    total = 0
    for pool in (worker.k_cache, worker.v_cache):
        view = pool.view(width)
        for i in range(0, len(block_ids), 32):
            idx = torch.as_tensor(block_ids[i:i + 32], dtype=torch.int64, device=pool.device)
            total += int(view.index_select(0, idx).to(torch.int64).sum().item())
    return total & ((1 << 64) - 1)


class _DrivenElsewhere:
    """Stands in the engine's worker grid for a decoding worker that another rank's process drives (every
    decoding rank runs the same engine over the same seeded requests and acts only on its own worker)."""

    def __getattr__(self, name):
        return lambda *a, **k: None


# ----------------------------------------------------------------------------------------------
# one workload on the GPU(s)
# ----------------------------------------------------------------------------------------------

def peer_copy_ceiling(src_device, dst_device, nbytes=1 << 30, repeats=10):
    """GB/s of one plain device-to-device copy (copy engines, no kernel of this library) between two GPUs of this
    process: the practical ceiling of the link for a single stream of large transfers."""
    import torch

    src = torch.empty(nbytes, dtype=torch.uint8, device=f"cuda:{src_device}")
    dst = torch.empty(nbytes, dtype=torch.uint8, device=f"cuda:{dst_device}")
    times = []
    with torch.cuda.device(dst_device):
        for _ in range(repeats + 2):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            dst.copy_(src, non_blocking=True)
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
    best = min(times[2:])
    return {"GBps": nbytes / (best / 1e3) / 1e9, "bytes": nbytes, "repeats": repeats,
            "call": "torch.Tensor.copy_ between two devices of one process (a driver peer copy on the copy engines), "
                    "CUDA events on the destination's stream, best of the repeats after 2 warm-up copies"}


def run_workload(args, w, world, rank, local_rank, dist, steps, warmup, primary=True):
    import torch

    from distserve_b200 import capi, spotcheck
    from distserve_b200.block_manager import BlockManager
    from distserve_b200.config import CacheConfig
    from distserve_b200.launch import Role, exchange_handles, num_replicas, plan_roles, shard_trace
    from distserve_b200.request import MigratingRequest, Request
    from distserve_b200.scheduler import DecodingStageFCFSScheduler, DecodingStageSchedConfig
    from distserve_b200.stage import DecodingStageEngine
    from distserve_b200.worker import KVWorker
    from distserve_b200.workloads import make_trace, trace_blocks

    trace = make_trace(w)
    peer = bool(args.peer_in_process) and world == 1
    same_device = world == 1 and not peer
    ctx_device, dec_device = (0, 1) if peer else (local_rank, local_rank)
    torch.cuda.set_device(dec_device)
    capi.reset_registry()

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()

    roles = None if world == 1 else plan_roles(w, world)
    cache = CacheConfig(w.block_size, 1 << 20)
    ctx_workers = {}          # (pp_rank, tp_rank) -> worker; a multi-rank run holds at most one per rank
    dec_worker = None
    role = Role("both") if roles is None else roles[rank]

    def fill(worker, salt):
        g = torch.Generator(device=worker.device).manual_seed(w.seed * 1000 + salt)
        for pool in (worker.k_cache, worker.v_cache):
            pool.normal_(generator=g)

    handles = None
    if role.stage == "both":
        # one process holds the whole context stage and decoding worker (0, 0)
        table = []
        for p in range(w.ctx_pp):
            row = []
            for t in range(w.ctx_tp):
                cw = KVWorker(p * w.ctx_tp + t, "context", w.model, cache, w.ctx_config(p, t), device=ctx_device)
                row.append(cw.init_kvcache_and_swap(w.ctx_pool_blocks, 1))
                fill(cw, p * w.ctx_tp + t)
                ctx_workers[(p, t)] = cw
            table.append(row)
    elif role.stage == "ctx":
        cw = KVWorker(rank, "context", w.model, cache, w.ctx_config(role.pp_rank, role.tp_rank), device=ctx_device)
        handles = cw.init_kvcache_and_swap(w.ctx_pool_blocks, 1)
        fill(cw, rank)
        ctx_workers[(role.pp_rank, role.tp_rank)] = cw
    if role.stage in ("dec", "both"):
        pc = w.dec_config(role.pp_rank, role.tp_rank)
        dec_worker = KVWorker(rank, "decoding", w.model, cache, pc, device=dec_device)
        dec_worker.init_kvcache_and_swap(w.dec_pool_blocks, 1)
        dec_worker.k_cache.zero_()
        dec_worker.v_cache.zero_()
    for d in {ctx_device, dec_device}:
        torch.cuda.synchronize(d)

    # handle table [pp][tp] of the context stage, gathered the way the engine gathers it
    if dist is not None:
        table = exchange_handles(w, roles, handles)
    ctx_pc = w.ctx_config()
    n_replicas = 1 if roles is None else num_replicas(roles)
    my_trace = []
    if dec_worker is not None:
        dec_worker.register_kvcache_mem_handles(ctx_pc, table)
        my_trace = list(trace) if roles is None else shard_trace(trace, role, n_replicas)
    barrier()

    stream = torch.cuda.current_stream()
    pc = dec_worker.parallel_config if dec_worker else None
    shape = dec_worker._pool_shape() if dec_worker else None
    bytes_per_block = w.dec_block_bytes()
    my_bytes_per_step = sum(len(t.src_blocks) for t in my_trace) * bytes_per_block
    factor = 2 if same_device else 1

    # target blocks that no request names: their contents must survive the whole run
    untouched = spotcheck.never_written_blocks(my_trace, w.dec_pool_blocks) if dec_worker is not None else []
    untouched = untouched[:: max(1, len(untouched) // 256)][:256]
    untouched_before = untouched_checksum(dec_worker, untouched) if untouched else None

    # the block lists of the `value` region are converted to C arrays once: its inputs are resident by definition
    c_lists = [(capi.I64List(item.src_blocks), capi.I64List(item.dst_blocks)) for item in my_trace]

    def enqueue(src, dst):
        return capi.migrate_blocks_async(
            ctx_pc.pipeline_parallel_size, ctx_pc.tensor_parallel_size, src,
            pc.pipeline_parallel_size, pc.tensor_parallel_size, pc.pipeline_parallel_rank, pc.tensor_parallel_rank,
            dst, dec_worker.k_cache.data_ptr(), dec_worker.v_cache.data_ptr(), shape, stream.cuda_stream)

    def step_async():
        tickets = [enqueue(src, dst) for src, dst in c_lists]
        for t in tickets:
            capi.migrate_wait(t)

    # several requests per launch: waves of consecutive requests whose target blocks are all distinct
    waves, cur_src, cur_dst, seen_dst = [], [], [], set()
    for item in my_trace:
        if cur_src and (seen_dst.intersection(item.dst_blocks) or len(cur_src) + len(item.src_blocks) > args.wave_blocks):
            waves.append((capi.I64List(cur_src), capi.I64List(cur_dst)))
            cur_src, cur_dst, seen_dst = [], [], set()
        cur_src += item.src_blocks
        cur_dst += item.dst_blocks
        seen_dst.update(item.dst_blocks)
    if cur_src:
        waves.append((capi.I64List(cur_src), capi.I64List(cur_dst)))

    def step_batched():
        tickets = [enqueue(src, dst) for src, dst in waves]
        for t in tickets:
            capi.migrate_wait(t)

    # what the worker receives from the engine: plain Python lists in host memory (an actor call delivers them so)
    py_lists = [(list(item.src_blocks), list(item.dst_blocks)) for item in my_trace]

    def step_e2e():
        migrate = dec_worker.migrate_blocks
        for src, dst in py_lists:
            migrate(src, ctx_pc, dst)

    def step_e2e_latencies(latencies):
        """The same calls with a host clock around each (kept out of the throughput region)."""
        for item in my_trace:
            t0 = time.perf_counter()
            dec_worker.migrate_blocks(list(item.src_blocks), ctx_pc, list(item.dst_blocks))
            latencies.append(time.perf_counter() - t0)

    # ---- the package's own host API at the batched cadence ----------------------------------------------
    engine = sched = None
    engine_records = []
    if dec_worker is not None:
        stage_pc = w.dec_config()
        grid = [[_DrivenElsewhere() for _ in range(w.dec_tp)] for _ in range(w.dec_pp)]
        grid[role.pp_rank][role.tp_rank] = dec_worker
        engine = DecodingStageEngine(w.model, stage_pc, cache, grid)
        engine.block_manager = BlockManager("decoding", w.dec_pool_blocks, 1, w.model, stage_pc, cache,
                                            engine._remote_call_all_workers_async)
        sched = DecodingStageFCFSScheduler(DecodingStageSchedConfig(), stage_pc, engine.block_manager, engine.migrate_blocks,
                                           engine.migrate_blocks_batched, engine.begin_migrate_blocks_batched,
                                           engine.finish_migrate_blocks_batched)

    def retire_oldest(fraction):
        """Stand-in for requests that finish decoding: the oldest running requests leave and free their blocks."""
        running = sorted((r for q in sched.batch_queues for r in q.requests), key=lambda r: r.request_id)
        for r in running[:max(1, int(len(running) * fraction))]:
            r.is_finished = True
        for q in sched.batch_queues:
            for r in q.pop_finished_requests():
                engine.block_manager.free_blocks(r.request_id)

    sources = {}
    steps_built = [0]

    def arrivals_of_one_step():
        """What the context stage hands over in one step: a MigratingRequest per request of the trace.  The engine
        runs on from step to step (requests of earlier steps are still decoding), so ids are unique across steps."""
        base = steps_built[0] * 1_000_000
        steps_built[0] += 1
        out = []
        for item in my_trace:
            req = Request.of_length(base + item.request_id, item.prompt_len)
            req.append_token()                                  # the token the prefill step produced
            out.append(MigratingRequest(req, list(item.src_blocks), ctx_pc))
            sources[base + item.request_id] = item.src_blocks
        return out

    # built ahead of the timed region: they are the step's input, produced by the context stage, not by this path
    prepared_arrivals = [arrivals_of_one_step() for _ in range(max(1, warmup) + steps)] if dec_worker is not None else []

    engine_error = []

    def step_engine():
        """One step through scheduler and engine.  A failure of this leg is reported in its own entry of the line; it
        must not keep this rank from the collectives the other ranks are waiting in."""
        if engine_error:
            return
        try:
            run_engine_step()
        except Exception as e:
            engine_error.append(f"{type(e).__name__}: {e}"[:300])

    def run_engine_step():
        bm = engine.block_manager
        sched.unaccepted_queue.extend(prepared_arrivals.pop(0) if prepared_arrivals else arrivals_of_one_step())
        engine.lifetime_events.clear()
        floor = int(0.15 * w.dec_pool_blocks)
        # the step ends when its last group has been enqueued; that group is awaited by the next step's first call
        while sched.unaccepted_queue:
            while bm.get_num_avail_gpu_blocks() < floor and sched.get_processing_num_requests():
                retire_oldest(0.25)
            ready = sched.post_process_pipelined()
            sched.get_next_batch()
            if not ready and sched._in_flight is None and sched.unaccepted_queue:
                if sched.get_processing_num_requests() == 0:
                    raise RuntimeError("the decoding pool cannot hold the next request")
                retire_oldest(0.5)

    def engine_drain():
        """Await the group still on the wire and note which blocks each resident request holds."""
        sched.flush_pipeline()
        engine_records[:] = [(rid, tuple(sources[rid]), tuple(ids)) for rid, ids in engine.block_manager.block_table.items()]

    def timed(step_fn, n_steps, **kw):
        """K steps between barriers; device time by CUDA events on the launching stream.  Returns the
        max over ranks and this rank's own time.  No event is recorded between launches: a timing event
        there would serialise launches that the library lets overlap."""
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(n_steps):
            if dec_worker is not None:
                step_fn(**kw)
        b.record(stream)
        barrier()
        mine = a.elapsed_time(b)
        ms = mine
        if dist is not None:
            t = torch.tensor([ms], dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, mine

    host_counters = ("migrate_calls", "plan_cache_hits", "ns_prepare", "ns_validate", "ns_order", "ns_launch", "ns_wait")

    def snapshot():
        return {k: capi.get_counter(k) for k in host_counters}

    sampler = ClockSampler(dec_device)
    if primary and (rank == 0 or (roles is not None and roles[rank] == Role("dec", 0, 0, 0))):
        sampler.start()
    for _ in range(warmup):
        if dec_worker is not None:
            step_async()
            if not args.no_e2e and not args.only_value:
                step_e2e()
    sampler.mark(0)
    launches0 = capi.get_counter("kernel_launches")
    ms_value, my_ms_value = timed(step_async, steps)
    value_launches = capi.get_counter("kernel_launches") - launches0
    latencies = []
    ms_e2e = ms_batched = ms_engine = None
    host_us = None
    engine_launches = 0
    if not args.only_value:
        if not args.no_e2e:
            c0 = snapshot()
            ms_e2e = timed(step_e2e, steps)[0]
            c1 = snapshot()
            if dec_worker is not None:
                step_e2e_latencies(latencies)
                torch.cuda.synchronize()
            calls = max(1, c1["migrate_calls"] - c0["migrate_calls"])
            host_us = {k[3:]: (c1[k] - c0[k]) / calls / 1e3 for k in host_counters if k.startswith("ns_")}
            host_us["plan_reused"] = (c1["plan_cache_hits"] - c0["plan_cache_hits"]) / calls
        if dec_worker is not None:
            step_batched()
        ms_batched = timed(step_batched, steps)[0]
    launches = capi.get_counter("kernel_launches") - launches0
    sampler.mark(1)
    clocks = sampler.stop() if sampler.proc is not None or (primary and rank == 0) else None

    # ---- correctness of what the timed regions left in the pools ----------------------------------------
    def verify(records_by_rank=None):
        """Sampled requests re-executed by the oracle on read-back slices (see the module docstring)."""
        if records_by_rank is None:
            samples = spotcheck.plan_samples(w, roles, trace)
        else:
            samples = spotcheck.plan_samples(w, roles, trace, traces_by_rank=records_by_rank)
        read_source = {key: spotcheck.torch_pool_reader(cw.k_cache, cw.v_cache) for key, cw in ctx_workers.items()} or None
        read_target = spotcheck.torch_pool_reader(dec_worker.k_cache, dec_worker.v_cache) if dec_worker is not None else None
        for d in {ctx_device, dec_device}:
            torch.cuda.synchronize(d)
        readbacks = spotcheck.exchange_samples(samples, rank, read_source, read_target, dist)
        n_samples, n_blocks, bad = check_readbacks(w, readbacks)
        stats = torch.tensor([float(n_samples), float(n_blocks), float(len(bad))], dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(stats)
        return int(stats[0].item()), int(stats[1].item()), int(stats[2].item()), bad

    verified = None
    verification = None
    if not args.only_value:
        n_samples, n_blocks, n_bad, bad = verify()
        untouched_ok = True
        if untouched:
            untouched_ok = untouched_checksum(dec_worker, untouched) == untouched_before
        flag = torch.tensor([0.0 if untouched_ok else 1.0], dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(flag)
        verified = n_bad == 0 and flag.item() == 0 and n_samples > 0
        verification = {"checker": "CPU oracle (numpy) on per-request read-back slices, bit patterns compared",
                        "sampled_requests": n_samples, "sampled_blocks": n_blocks, "mismatching_requests": n_bad,
                        "untouched_blocks_checked_per_dest": len(untouched) if dist is None else None,
                        "untouched_blocks_unchanged": bool(flag.item() == 0)}
        if not verified:
            print(f"bench: rank {rank}: verification failed: {verification} {bad}", file=sys.stderr)
            raise SystemExit(3)

    # ---- the package's own API at the batched cadence (after the check: it allocates its own target blocks) -----
    engine_verification = None
    if not args.only_value and not args.no_e2e:
        for _ in range(max(1, warmup)):
            if dec_worker is not None:
                step_engine()
        l0 = capi.get_counter("kernel_launches")
        w0, t0 = capi.get_counter("ns_wait"), time.perf_counter()
        ms_engine = timed(step_engine, steps)[0]
        engine_wall_ms = (time.perf_counter() - t0) * 1e3 / steps
        engine_waited_ms = (capi.get_counter("ns_wait") - w0) / 1e6 / steps
        engine_launches = capi.get_counter("kernel_launches") - l0
        if dec_worker is not None and not engine_error:
            try:
                engine_drain()
            except Exception as e:
                engine_error.append(f"{type(e).__name__}: {e}"[:300])
        failed = torch.tensor([1.0 if engine_error else 0.0], dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(failed)
        if failed.item() > 0:
            ms_engine = None
            if not engine_error:
                engine_error.append("this leg failed on another rank")
        launches += engine_launches
        if ms_engine is not None:
            records = [spotcheck.TraceItem(rid, 0, src, dst) for rid, src, dst in engine_records]
            if dist is not None:
                gathered = [None] * world
                dist.all_gather_object(gathered, records)
                by_rank = {r: recs for r, recs in enumerate(gathered)}
            else:
                by_rank = {0: records}
            n_samples, n_blocks, n_bad, bad = verify(by_rank)
            engine_verification = {"sampled_requests": n_samples, "sampled_blocks": n_blocks, "mismatching_requests": n_bad}
            if n_bad or not n_samples:
                print(f"bench: rank {rank}: verification of the engine-driven leg failed: {engine_verification} {bad}", file=sys.stderr)
                raise SystemExit(3)

    # block swap (decoding stage only): scattered GPU blocks <-> pinned host blocks through the worker's protocol
    swap_info = None
    if primary and same_device and dec_worker is not None and not args.no_swap and not args.only_value:
        n_swap = min(64, w.dec_pool_blocks)
        dtype = dec_worker.k_cache.dtype
        dec_worker.k_swap = torch.empty((n_swap,) + tuple(dec_worker.k_cache.shape[1:]), dtype=dtype, pin_memory=True)
        dec_worker.v_swap = torch.empty_like(dec_worker.k_swap).pin_memory()
        gpu_ids = [int(x) for x in torch.randperm(w.dec_pool_blocks)[:n_swap]]
        host_ids = [int(x) for x in torch.randperm(n_swap)]
        swap_bytes = n_swap * bytes_per_block
        res = {}
        for direction, is_in in (("out", False), ("in", True)):
            times = []
            for _ in range(4):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                if is_in:
                    dec_worker.swap_blocks([0], host_ids, gpu_ids, True)
                    dec_worker.wait_for_all_swap_in()
                else:
                    dec_worker.swap_blocks([0], gpu_ids, host_ids, False)
                    dec_worker.wait_for_all_swap_out()
                times.append(time.perf_counter() - t0)
            res[direction] = swap_bytes / min(times[1:]) / 1e9
        # the host link's own ceiling in this run: ONE contiguous pinned copy of the same number of bytes
        host_flat = dec_worker.k_swap.view(torch.uint8).reshape(-1)
        half = host_flat.numel()
        dev_flat = torch.empty(half, dtype=torch.uint8, device="cuda")
        peak = {}
        for direction in ("out", "in"):
            times = []
            for _ in range(4):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for _ in range(2):                                  # K-sized and V-sized halves, as the swap moves
                    if direction == "in":
                        dev_flat.copy_(host_flat, non_blocking=True)
                    else:
                        host_flat.copy_(dev_flat, non_blocking=True)
                torch.cuda.synchronize()
                times.append(time.perf_counter() - t0)
            peak[direction] = 2 * half / min(times[1:]) / 1e9
        del dev_flat
        swap_info = {"out_GBps": res["out"], "in_GBps": res["in"], "blocks": n_swap, "bytes_per_direction": swap_bytes,
                     "peak_GBps": {"out": peak["out"], "in": peak["in"]},
                     "frac": {"out": res["out"] / peak["out"], "in": res["in"] / peak["in"]},
                     "peak_source": "contiguous pinned<->device copies of the same bytes (two halves), same run, best of 3",
                     "api": "KVWorker.swap_blocks -> torch.ops.swapping_ops.swap, scattered ids, pinned host pool, "
                            "best of 3 after warm-up, wall clock around enqueue + flush"}

    # ---- aggregate over ranks ------------------------------------------------------------------------
    totals = torch.tensor([float(my_bytes_per_step), float(launches), float(dec_worker is not None)], dtype=torch.float64)
    # launches of the `value` region run back to back on one stream: average launch duration = region / launches
    kern = torch.tensor([my_ms_value if dec_worker is not None else 0.0, float(my_bytes_per_step * steps),
                         float(value_launches)], dtype=torch.float64)
    lat = sorted(latencies)
    p50 = torch.tensor([lat[len(lat) // 2] if lat else 0.0, float(len(waves)), float(engine_launches) / max(1, steps)],
                       dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(totals)
        gathered_kern = [None] * world
        dist.all_gather_object(gathered_kern, kern.tolist())
        dist.all_reduce(p50, op=dist.ReduceOp.MAX)
        clk = [None] * world
        dist.all_gather_object(clk, clocks)
        hosts = [None] * world
        dist.all_gather_object(hosts, host_us)
        dec_clk = [c for r, c in enumerate(clk) if c and roles[r].stage == "dec" and c.get("sm_mhz")]
        if dec_clk:
            clocks = dec_clk[0]
        host_us = next((h for r, h in enumerate(hosts) if h and roles[r].stage == "dec"), None)
        # the engine-driven leg's host times likewise come from a decoding rank (rank 0 holds a context worker)
        engine_hosts = [None] * world
        mine = None if ms_engine is None or dec_worker is None else {"wall_per_step": engine_wall_ms,
                                                                     "waiting_for_the_gpu_per_step": engine_waited_ms}
        dist.all_gather_object(engine_hosts, mine)
        engine_host_ms = next((h for r, h in enumerate(engine_hosts) if h and roles[r].stage == "dec"), None)
    else:
        engine_host_ms = None if ms_engine is None else {"wall_per_step": engine_wall_ms,
                                                         "waiting_for_the_gpu_per_step": engine_waited_ms}
        gathered_kern = [kern.tolist()]

    total_bytes_per_step = totals[0].item()
    n_dest = int(totals[2].item())

    def gbs(ms):
        return None if ms is None else factor * total_bytes_per_step * steps / (ms / 1e3) / 1e9

    # roofline of the dominant kernel: the slowest destination rank's per-launch average
    worst = None
    for k_ms, k_bytes, k_n in gathered_kern:
        if k_n:
            rate = factor * k_bytes / (k_ms / 1e3) / 1e9
            if worst is None or rate < worst[0]:
                worst = (rate, k_ms / k_n, k_bytes / k_n)
    longest = max(len(t.src_blocks) for t in trace)
    if capi.get_option("kernel") == 1:
        kernel_label = "kv_migrate_vec<16>"
    elif capi.get_option("inline_tables") and longest <= 256:
        kernel_label = "kv_migrate_bulk_inline<256>"
    else:
        kernel_label = "kv_migrate_bulk / kv_migrate_bulk_inline"
    if same_device:
        peak, peak_kind = hbm_peak()
        # ncu on a small case of this kernel: DRAM reads equal the algorithmic read bytes, DRAM
        # writes fall short of the algorithmic write bytes by the ~48.8 MB still dirty in L2 at kernel end.
        alg = factor * worst[2]
        traffic = alg / 2 + max(0.0, alg / 2 - 48.8e6) if capi.get_option("kernel") in (0, 2) else None
        roof = {"bound": "hbm", "achieved": worst[0], "peak": peak, "unit": "GB/s", "frac": worst[0] / peak,
                "traffic": traffic, "peak_source": f"{peak_kind} copy bandwidth (MEASURED_PEAKS.json)" if peak_kind == "measured"
                else "fallback 6650 GB/s", "avg_launch_us": worst[1] * 1e3, "algorithmic_bytes_per_launch": factor * worst[2],
                "kernel": kernel_label}
    else:
        roof = {"bound": "nvlink", "achieved": worst[0], "peak": NVLINK_NOMINAL_GBS, "unit": "GB/s",
                "frac": worst[0] / NVLINK_NOMINAL_GBS, "traffic": None,
                "peak_source": "nominal NVLink 5 ingress per GPU per direction (a measured peer-copy ceiling of the same "
                               "box, where one was taken, is in profiles/)",
                "avg_launch_us": worst[1] * 1e3,
                "algorithmic_bytes_per_launch": worst[2], "per": "slowest destination GPU",
                "kernel": kernel_label}

    peer_copy = peer_copy_ceiling(ctx_device, dec_device) if peer and primary and not args.only_value else None
    out = {
        "workload": w, "trace": trace, "same_device": same_device, "n_dest": n_dest, "n_replicas": n_replicas,
        "value": gbs(ms_value), "ms_value": ms_value, "e2e_value": gbs(ms_e2e), "ms_e2e": ms_e2e,
        "batched_value": gbs(ms_batched), "engine_value": gbs(ms_engine), "ms_engine": ms_engine,
        "waves": int(p50[1].item()), "engine_launches_per_step": p50[2].item(),
        "p50_ms": p50[0].item() * 1e3 if lat or dist is not None else None,
        "roofline": roof, "launches": int(totals[1].item()), "clocks": clocks, "verified": verified,
        "verification": verification, "engine_verification": engine_verification, "swap": swap_info, "host_us": host_us,
        "engine_error": engine_error[0] if engine_error else None,
        "engine_host_ms": engine_host_ms,
        "peer_copy": peer_copy,
    }
    # release the pools before another workload is set up in this process
    del ctx_workers, dec_worker, engine, sched
    capi.reset_registry()
    torch.cuda.empty_cache()
    return out


# ----------------------------------------------------------------------------------------------
# main
# ----------------------------------------------------------------------------------------------

def describe(w, trace, same_device):
    from distserve_b200.workloads import trace_blocks

    sample = cpu_sample(w, trace)
    return {
        "workload": f"{w.name}" + (" (context and decoding pools on one GPU)" if same_device else ""),
        "layers": w.model.num_layers, "kv_heads": w.model.num_kv_heads, "head_dim": w.model.head_dim,
        "block_size": w.block_size, "context": f"tp{w.ctx_tp}pp{w.ctx_pp}", "decoding": f"tp{w.dec_tp}pp{w.dec_pp}",
        "requests": len(trace), "blocks_per_step": trace_blocks(trace), "length_dist": list(w.length_dist),
        "pool_blocks": [w.ctx_pool_blocks, w.dec_pool_blocks], "seed": w.seed,
        "bytes_per_block_per_dest_gpu": w.dec_block_bytes(),
        "l2": "each step moves far more than the 126 MB L2 (no reuse between steps' blocks)",
        "bytes_counted": "read+write (same GPU)" if same_device else "payload once (into the destination GPU)",
        # the bounded sample the CPU arms run (cpu_baseline in this line; every timed step of --impl reference)
        "sample_requests": len(sample), "sample_blocks": sum(len(d) for _, d in sample),
        "sample_pool_blocks": CPU_SAMPLE_POOL_BLOCKS,
        "sample_note": "CPU arms only: one pass = these requests, ids folded into compact host pools; the GPU arm runs "
                       "all requests at full pool size",
    }


def main():
    args = parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != max(1, args.gpus) and world != 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")

    from distserve_b200.workloads import WORKLOADS, make_trace, trace_blocks

    name = args.workload or DEFAULT_WORKLOAD.get(args.gpus, "c2")
    w = WORKLOADS[name]
    if args.pool_blocks:
        w = w.scaled(ctx_pool_blocks=args.pool_blocks, dec_pool_blocks=args.pool_blocks)
    if args.requests:
        w = w.scaled(num_requests=args.requests)
    same_device = args.gpus == 1 and not args.peer_in_process

    if args.impl == "reference":
        if rank != 0:
            return
        trace = make_trace(w)
        print(json.dumps(reference_arm(args, w, trace, describe(w, trace, same_device), same_device)))
        return

    import torch

    import distserve_b200
    from distserve_b200 import capi

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the migration path has no CPU implementation")
    distserve_b200.load_ops()
    # one GPU per rank; on a machine with fewer GPUs than ranks (functional runs only) the ranks share them
    local_rank = local_rank % torch.cuda.device_count()
    torch.cuda.set_device(local_rank)
    for opt in ("kernel", "chunk_bytes", "stages", "ctas_per_sm"):
        v = getattr(args, opt)
        if v is not None:
            capi.set_option(opt, v)
    for pair in args.opt:
        k, v = pair.split("=")
        capi.set_option(k, int(v))

    dist = None
    if world > 1:
        import datetime

        import torch.distributed as dist
        dist.init_process_group(backend="gloo", timeout=datetime.timedelta(minutes=20))

    r = run_workload(args, w, world, rank, local_rank, dist, args.steps, args.warmup, primary=True)
    trace = r["trace"]
    n_dest, n_replicas = r["n_dest"], r["n_replicas"]

    # N = 1: the launch-bound regimes (small requests) beside the headline workload, a few steps each
    others = None
    if same_device and world == 1 and not args.no_other_workloads and not args.only_value and args.workload is None:
        others = {}
        for other in ("c1", "c5"):
            o = run_workload(args, WORKLOADS[other], world, rank, local_rank, dist, max(3, min(args.steps, 10)), 3, primary=False)
            others[other] = {"workload": WORKLOADS[other].name, "value": o["value"], "e2e": o["e2e_value"],
                             "batched": o["batched_value"], "e2e_batched": o["engine_value"], "unit": UNIT,
                             "p50_migrate_latency_ms": o["p50_ms"], "avg_launch_us": o["roofline"]["avg_launch_us"],
                             "verified_on_device": o["verified"], "steps": max(3, min(args.steps, 10)),
                             "note": "the whole context stage -> decoding worker (0, 0) of the layout, all pools on this GPU"}

    # N = 4 / 8: the serving loop of the end-to-end configuration, one worker process per GPU, driven from rank 0
    overlap = None
    if world in (4, 8) and not args.no_overlap and not args.only_value:
        dist.barrier()
        if rank == 0:
            try:
                from distserve_b200 import e2e_loop

                full = e2e_loop.run_actors(n_gpus=world, steps=600, time_scale=50.0, passes=3, deadline_s=360.0)
                overlap = {k: full[k] for k in ("workload", "layout", "replicas", "hidden_fraction",
                                                "added_us_per_migration_awaited", "added_us_per_migration_overlapped",
                                                "verified", "steps", "time_scale", "overlapped_kernel_options")}
                overlap["decode_step_ms"] = [o["decode_step_ms"] for o in full["per_replica"]]
                overlap["migrations"] = [o["migrations"] for o in full["per_replica"]]
                overlap["loop_ms"] = [o["loop_ms"] for o in full["per_replica"]]
                overlap["hidden_fraction_per_replica"] = [o["hidden_fraction"] for o in full["per_replica"]]
                overlap["note"] = "hidden_fraction is the smaller of the replicas' fractions; best of 3 passes per mode"
            except Exception as e:          # reported, not fatal: the migration figures above stand on their own
                overlap = {"error": f"{type(e).__name__}: {e}"[:400]}
        dist.barrier()

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    value = r["value"]
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": r["ms_value"] / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u8", "data": "synthetic", "config": describe(w, trace, same_device),
        "per_dest_gpu_GBps": value / max(1, n_dest), "dest_gpus": n_dest,
        "scaling_note": "N = 1 is bound by HBM (bytes counted read + write), N >= 2 by the NVLink ingress of each destination "
                        "GPU (payload counted once): compare per_dest_gpu_GBps across N >= 2, not value across N",
        "frac_of_nvlink_900_per_dest": None if same_device else value / max(1, n_dest) / NVLINK_NOMINAL_GBS,
        "p50_migrate_latency_ms": r["p50_ms"],
        "roofline": r["roofline"], "gpu_launches": r["launches"], "clocks": r["clocks"],
        "verified_on_device": r["verified"], "verification": r["verification"],
        "options": {k: capi.get_option(k) for k in ("kernel", "chunk_bytes", "stages", "ctas_per_sm", "inline_tables",
                                                   "overlap_launches")},
    }
    per_dest = lambda v: None if v is None else v / max(1, n_dest)
    if r["e2e_value"] is not None:
        n_calls = len(trace) * n_dest // max(1, n_replicas) if not same_device else len(trace)
        line["e2e"] = {"value": r["e2e_value"], "unit": UNIT, "ms_per_step": r["ms_e2e"] / args.steps,
                       "per_dest_gpu_GBps": per_dest(r["e2e_value"]),
                       "frac_of_nvlink_900_per_dest": None if same_device else per_dest(r["e2e_value"]) / NVLINK_NOMINAL_GBS,
                       "h2d_bytes_per_step": 8 * trace_blocks(trace) * (n_dest // max(1, n_replicas) if not same_device else 1),
                       "d2h_bytes_per_step": 16 * n_calls,
                       "host_us_per_call": r["host_us"],
                       "api": "torch.ops.block_migration_ops.migrate_blocks, one awaited call per request"}
    if r["batched_value"] is not None:
        line["batched"] = {"value": r["batched_value"], "unit": UNIT, "per_dest_gpu_GBps": per_dest(r["batched_value"]),
                           "launches_per_step_per_dest": r["waves"],
                           "api": "kvmig_migrate_blocks_async with the concatenated block lists of consecutive requests "
                                  f"(up to {args.wave_blocks} blocks, distinct targets) per launch"}
    if r["engine_value"] is not None:
        line["e2e_batched"] = {"value": r["engine_value"], "unit": UNIT, "ms_per_step": r["ms_engine"] / args.steps,
                               "per_dest_gpu_GBps": per_dest(r["engine_value"]),
                               "frac_of_nvlink_900_per_dest": None if same_device else per_dest(r["engine_value"]) / NVLINK_NOMINAL_GBS,
                               "launches_per_step_per_dest": r["engine_launches_per_step"],
                               "verification": r["engine_verification"],
                               "host_ms_decoding_rank": r["engine_host_ms"],
                               "api": "DecodingStageFCFSScheduler.post_process_pipelined -> DecodingStageEngine."
                                      "begin/finish_migrate_blocks_batched -> KVWorker.migrate_blocks_async, Python lists, "
                                      "target blocks from the block manager"}
    elif r["engine_error"]:
        line["e2e_batched"] = {"error": r["engine_error"]}
    if r["swap"] is not None:
        line["swap"] = r["swap"]
    if r["peer_copy"] is not None:
        line["roofline"]["measured_peer_copy"] = r["peer_copy"]
        line["roofline"]["frac_of_measured_peer_copy"] = r["roofline"]["achieved"] / r["peer_copy"]["GBps"]
        line["config"]["workload"] += " (one process: context stage on GPU 0, decoding worker (0,0) on GPU 1)"
    if others is not None:
        line["other_workloads"] = others
    if overlap is not None:
        line["overlap"] = overlap
    if not args.no_cpu_baseline and args.gpus == 1 and not args.only_value:
        line["cpu_baseline"] = cpu_baseline(w, trace, same_device, seconds=args.cpu_seconds)
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

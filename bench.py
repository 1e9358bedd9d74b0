#!/usr/bin/env python
"""KV-block migration benchmark.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" migrates every request of the workload once, one call per request
(the reference's cadence, distserve/single_stage_engine.py:490-536).  Two timed
regions of K steps each follow W warm-up steps:

* ``value`` — requests enqueued back to back through the asynchronous C-ABI
  entry point; KV pools resident in HBM; timed with CUDA events on the
  launching stream around the whole region.  The launches run back to back on
  that stream, so the roofline figure uses region time / launches as the
  average launch duration (an event between launches would serialise launches
  that the library lets overlap).
* ``e2e``   — the call a DistServe worker makes: ``torch.ops.block_migration_ops
  .migrate_blocks`` with Python block-index lists, returning only when the
  source blocks may be recycled.  The host->device traffic of this path is the
  block tables, the device->host traffic the kernel's status words; the KV
  payload is device-resident by the operator's contract (it takes CUDA
  tensors).

Workload by GPU count (override with --workload):
  1  c2 shapes, context and decoding pools on the same GPU (HBM-bound)
  2  c2: GPU0 -> GPU1
  4  c3: context tp=2 on GPUs 0-1 -> two decoding tp=1 replicas on GPUs 2, 3
  8  c4: context tp=4,pp=1 on GPUs 0-3 -> decoding tp=2,pp=2 on GPUs 4-7
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
NVLINK_MEASURED_P2P_GBS = 770.0  # peer copy measured on this pool
HBM_FALLBACK_GBS = 6650.0

DEFAULT_WORKLOAD = {1: "c2", 2: "c2", 4: "c3", 8: "c4"}


def parse_args():
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
    return ap.parse_args()


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


def cpu_baseline(workload, trace, same_device: bool, seconds: float):
    """The oracle's torch gather/scatter on host tensors with every host thread,
    on the first requests of the trace, block ids folded into compact pools."""
    import torch

    from oracle import kv_oracle as O

    # every host core, also under torchrun (which exports OMP_NUM_THREADS=1 to its ranks)
    torch.set_num_threads(os.cpu_count() or 1)
    w = workload
    max_pool = 256
    sample = []
    for item in trace:
        if len(item.src_blocks) <= max_pool:
            sample.append(item)
        if len(sample) == 8:
            break
    remap = lambda ids: [i % max_pool for i in ids]
    dt = w.model.get_torch_dtype()
    ctx_pools = {}
    for p in range(w.ctx_pp):
        for t in range(w.ctx_tp):
            pc = w.ctx_config(p, t)
            shape = (max_pool, w.model.get_num_layers(pc), w.model.get_num_heads(pc), w.block_size, w.model.head_dim)
            ctx_pools[(p, t)] = (torch.randn(shape, dtype=torch.float32).to(dt), torch.randn(shape, dtype=torch.float32).to(dt))
    pc = w.dec_config()
    dshape = (max_pool, w.model.get_num_layers(pc), w.model.get_num_heads(pc), w.block_size, w.model.head_dim)
    dec_pools = {(p, t): (torch.zeros(dshape, dtype=dt), torch.zeros(dshape, dtype=dt))
                 for p in range(w.dec_pp) for t in range(w.dec_tp)}
    factor = 2 if same_device else 1

    def one_pass(migrate):
        moved = 0
        for item in sample:
            src, dst = remap(item.src_blocks), remap(item.dst_blocks)
            # distinct targets are required; folding may collide, so de-duplicate while keeping order
            seen, s2, d2 = set(), [], []
            for a, b in zip(src, dst):
                if b not in seen:
                    seen.add(b)
                    s2.append(a)
                    d2.append(b)
            for (p, t), (k, v) in dec_pools.items():
                migrate(ctx_pools, w.ctx_tp, w.ctx_pp, s2, w.dec_tp, t, w.dec_pp, p, d2, k, v,
                        w.model.num_layers, w.model.num_kv_heads)
                moved += len(d2) * w.dec_block_bytes()
        return moved

    def timed_passes(fn, budget):
        one_pass(fn)   # warm-up: page in the pools
        t0 = time.perf_counter()
        moved, passes = 0, 0
        while True:
            moved += one_pass(fn)
            passes += 1
            if time.perf_counter() - t0 >= budget:
                break
        return moved, passes, time.perf_counter() - t0

    moved, passes, dt_s = timed_passes(O.migrate_blocks_torch, seconds)
    out = {"value": factor * moved / dt_s / 1e9, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
           "ms_per_sample_pass": dt_s * 1e3 / passes,
           "sample": f"first {len(sample)} requests of {w.name}, ids folded into {max_pool}-block host pools, "
                     f"{passes} passes in {dt_s:.1f} s, torch index_select/index_copy_ on {torch.get_num_threads()} threads"}
    # the same semantics as plain C (one memcpy per run, OpenMP over blocks x layers): a stronger CPU arm, for context
    try:
        from oracle import kv_oracle_c as OC

        moved_c, passes_c, dt_c = timed_passes(OC.migrate_blocks_c, max(2.0, seconds / 4))
        out["c_openmp"] = {"value": factor * moved_c / dt_c / 1e9, "unit": UNIT, "cores": os.cpu_count(),
                           "sample": f"same sample, {passes_c} passes in {dt_c:.1f} s, oracle/kv_oracle.c"}
    except Exception as e:   # gcc missing on the box: the torch arm stands alone
        out["c_openmp"] = {"unavailable": str(e)[:200]}
    return out


# ----------------------------------------------------------------------------------------------
# main
# ----------------------------------------------------------------------------------------------

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
    trace = make_trace(w)
    same_device = args.gpus == 1
    config = {
        "workload": f"{w.name}" + (" (context and decoding pools on one GPU)" if same_device else ""),
        "layers": w.model.num_layers, "kv_heads": w.model.num_kv_heads, "head_dim": w.model.head_dim,
        "block_size": w.block_size, "context": f"tp{w.ctx_tp}pp{w.ctx_pp}", "decoding": f"tp{w.dec_tp}pp{w.dec_pp}",
        "requests": len(trace), "blocks_per_step": trace_blocks(trace), "length_dist": list(w.length_dist),
        "pool_blocks": [w.ctx_pool_blocks, w.dec_pool_blocks], "seed": w.seed,
        "bytes_per_block_per_dest_gpu": w.dec_block_bytes(),
        "l2": "each step moves far more than the 126 MB L2 (no reuse between steps' blocks)",
        "bytes_counted": "read+write (same GPU)" if same_device else "payload once (into the destination GPU)",
    }

    if args.impl == "reference":
        if rank != 0:
            return
        base = cpu_baseline(w, trace, same_device, max(args.cpu_seconds, 5.0) * max(1, min(args.steps, 3)))
        line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_sample_pass"], "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
                "config": config, "cpu_baseline": base,
                "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "note": "the reference's native copy (SwiftTransformer) is not in its tree; this arm is the CPU "
                        "restatement of its semantics (oracle/kv_oracle.py), torch host-tensor gather/scatter"}
        print(json.dumps(line))
        return

    import torch

    import distserve_b200
    from distserve_b200 import capi
    from distserve_b200.config import CacheConfig
    from distserve_b200.worker import KVWorker

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the migration path has no CPU implementation")
    distserve_b200.load_ops()
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
        import torch.distributed as dist
        dist.init_process_group(backend="gloo")

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()

    from distserve_b200.launch import Role, exchange_handles, num_replicas, plan_roles, shard_trace

    roles = None if world == 1 else plan_roles(w, world)
    cache = CacheConfig(w.block_size, 1 << 20)
    ctx_worker = dec_worker = None
    role = Role("both") if roles is None else roles[rank]

    def fill(worker):
        g = torch.Generator(device="cuda").manual_seed(w.seed * 1000 + rank)
        for pool in (worker.k_cache, worker.v_cache):
            pool.normal_(generator=g)

    handles = None
    if role.stage in ("ctx", "both"):
        pc = w.ctx_config(role.pp_rank, role.tp_rank)
        ctx_worker = KVWorker(rank, "context", w.model, cache, pc, device=local_rank)
        handles = ctx_worker.init_kvcache_and_swap(w.ctx_pool_blocks, 1)
        fill(ctx_worker)
    if role.stage in ("dec", "both"):
        pc = w.dec_config(role.pp_rank, role.tp_rank)
        dec_worker = KVWorker(rank, "decoding", w.model, cache, pc, device=local_rank)
        dec_worker.init_kvcache_and_swap(w.dec_pool_blocks, 1)
        dec_worker.k_cache.zero_()
        dec_worker.v_cache.zero_()
    torch.cuda.synchronize()

    # handle table [pp][tp] of the context stage, gathered the way the engine gathers it
    table = [[handles]] if dist is None else exchange_handles(w, roles, handles)
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

    # the block lists of the `value` region are converted to C arrays once: its inputs are resident by definition
    c_lists = [(capi.I64List(item.src_blocks), capi.I64List(item.dst_blocks)) for item in my_trace]

    def step_async():
        tickets = [capi.migrate_blocks_async(
            ctx_pc.pipeline_parallel_size, ctx_pc.tensor_parallel_size, src,
            pc.pipeline_parallel_size, pc.tensor_parallel_size, pc.pipeline_parallel_rank, pc.tensor_parallel_rank,
            dst, dec_worker.k_cache.data_ptr(), dec_worker.v_cache.data_ptr(), shape, stream.cuda_stream)
            for src, dst in c_lists]
        for t in tickets:
            capi.migrate_wait(t)

    # several requests per launch: waves of consecutive requests whose target blocks are all distinct
    waves, cur_src, cur_dst, seen_dst = [], [], [], set()
    for item in my_trace:
        if seen_dst.intersection(item.dst_blocks) or len(cur_src) + len(item.src_blocks) > 4096:
            waves.append((capi.I64List(cur_src), capi.I64List(cur_dst)))
            cur_src, cur_dst, seen_dst = [], [], set()
        cur_src += item.src_blocks
        cur_dst += item.dst_blocks
        seen_dst.update(item.dst_blocks)
    if cur_src:
        waves.append((capi.I64List(cur_src), capi.I64List(cur_dst)))

    def step_batched():
        tickets = [capi.migrate_blocks_async(
            ctx_pc.pipeline_parallel_size, ctx_pc.tensor_parallel_size, src,
            pc.pipeline_parallel_size, pc.tensor_parallel_size, pc.pipeline_parallel_rank, pc.tensor_parallel_rank,
            dst, dec_worker.k_cache.data_ptr(), dec_worker.v_cache.data_ptr(), shape, stream.cuda_stream)
            for src, dst in waves]
        for t in tickets:
            capi.migrate_wait(t)

    def step_e2e(latencies=None):
        for item in my_trace:
            t0 = time.perf_counter()
            dec_worker.migrate_blocks(list(item.src_blocks), ctx_pc, list(item.dst_blocks))
            if latencies is not None:
                latencies.append(time.perf_counter() - t0)

    def timed(step_fn, steps, **kw):
        """K steps between barriers; device time by CUDA events on the launching stream.  Returns the
        max over ranks and this rank's own time.  No event is recorded between launches: a timing event
        there would serialise launches that the library lets overlap."""
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(steps):
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

    sampler = ClockSampler(local_rank)
    if rank == 0 or (roles is not None and roles[rank] == Role("dec", 0, 0, 0)):
        sampler.start()
    for _ in range(args.warmup):
        if dec_worker is not None:
            step_async()
            if not args.no_e2e:
                step_e2e()
    sampler.mark(0)
    launches0 = capi.get_counter("kernel_launches")
    ms_value, my_ms_value = timed(step_async, args.steps)
    value_launches = capi.get_counter("kernel_launches") - launches0
    latencies = []
    ms_e2e = None if args.no_e2e else timed(step_e2e, args.steps, latencies=latencies)[0]
    launches = capi.get_counter("kernel_launches") - launches0
    sampler.mark(1)
    if dec_worker is not None:
        step_batched()
    ms_batched = timed(step_batched, args.steps)[0]
    clocks = sampler.stop() if sampler.proc is not None or rank == 0 else None

    # spot check on the device: three requests' target blocks equal their source blocks
    verified = None
    if same_device and dec_worker is not None:
        verified = True
        last_writer = {}
        for item in trace:
            for s, d in zip(item.src_blocks, item.dst_blocks):
                last_writer[d] = s
        some = list(last_writer.items())[:: max(1, len(last_writer) // 64)]
        d_ids = torch.tensor([d for d, _ in some], device="cuda")
        s_ids = torch.tensor([s for _, s in some], device="cuda")
        verified = bool(torch.equal(dec_worker.k_cache[d_ids], ctx_worker.k_cache[s_ids]) and
                        torch.equal(dec_worker.v_cache[d_ids], ctx_worker.v_cache[s_ids]))
        if not verified:
            raise SystemExit("bench: migrated blocks differ from their sources")

    # block swap (decoding stage only): scattered GPU blocks <-> pinned host blocks through the worker's protocol
    swap_info = None
    if same_device and dec_worker is not None and not args.no_swap:
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
        swap_info = {"out_GBps": res["out"], "in_GBps": res["in"], "blocks": n_swap, "bytes_per_direction": swap_bytes,
                     "api": "KVWorker.swap_blocks -> torch.ops.swapping_ops.swap, scattered ids, pinned host pool, "
                            "best of 3 after warm-up, wall clock around enqueue + flush"}

    # aggregate over ranks
    totals = torch.tensor([float(my_bytes_per_step), float(launches), float(dec_worker is not None)], dtype=torch.float64)
    # launches of the `value` region run back to back on one stream: average launch duration = region / launches
    kern = torch.tensor([my_ms_value if dec_worker is not None else 0.0, float(my_bytes_per_step * args.steps),
                         float(value_launches)], dtype=torch.float64)
    lat = sorted(latencies)
    p50 = torch.tensor([lat[len(lat) // 2] if lat else 0.0, float(len(waves))], dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(totals)
        gathered_kern = [None] * world
        dist.all_gather_object(gathered_kern, kern.tolist())
        dist.all_reduce(p50, op=dist.ReduceOp.MAX)
    else:
        gathered_kern = [kern.tolist()]
    if rank != 0:
        if dist is not None:
            clk = [None] * world
            dist.all_gather_object(clk, clocks)
            dist.destroy_process_group()
        return
    if dist is not None:
        clk = [None] * world
        dist.all_gather_object(clk, clocks)
        dec_clk = [c for r, c in enumerate(clk) if c and roles[r].stage == "dec" and c.get("sm_mhz")]
        if dec_clk:
            clocks = dec_clk[0]

    total_bytes_per_step = totals[0].item()
    n_dest = int(totals[2].item())
    value = factor * total_bytes_per_step * args.steps / (ms_value / 1e3) / 1e9
    e2e_value = None if ms_e2e is None else factor * total_bytes_per_step * args.steps / (ms_e2e / 1e3) / 1e9
    # roofline of the dominant kernel: the slowest destination rank's per-launch average
    worst = None
    for k_ms, k_bytes, k_n in gathered_kern:
        if k_n:
            gbs = factor * k_bytes / (k_ms / 1e3) / 1e9
            if worst is None or gbs < worst[0]:
                worst = (gbs, k_ms / k_n, k_bytes / k_n)
    if capi.get_option("kernel") == 1:
        kernel_label = "kv_migrate_vec<16>"
    elif capi.get_option("inline_tables") and max(len(t.src_blocks) for t in trace) <= 256:
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
                "peak_source": "nominal NVLink 5 ingress per GPU per direction",
                "frac_of_measured_p2p_770": worst[0] / NVLINK_MEASURED_P2P_GBS, "avg_launch_us": worst[1] * 1e3,
                "algorithmic_bytes_per_launch": worst[2], "per": "slowest destination GPU",
                "kernel": kernel_label}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_value / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u8", "data": "synthetic", "config": config,
        "per_dest_gpu_GBps": value / max(1, n_dest), "dest_gpus": n_dest,
        "frac_of_nvlink_900_per_dest": None if same_device else value / max(1, n_dest) / NVLINK_NOMINAL_GBS,
        "p50_migrate_latency_ms": p50[0].item() * 1e3 if lat or dist is not None else None,
        "roofline": roof, "gpu_launches": int(totals[1].item()), "clocks": clocks, "verified_on_device": verified,
        "options": {k: capi.get_option(k) for k in ("kernel", "chunk_bytes", "stages", "ctas_per_sm", "inline_tables",
                                                   "overlap_launches")},
    }
    if e2e_value is not None:
        n_calls = len(trace) * n_dest // max(1, n_replicas) if not same_device else len(trace)
        line["e2e"] = {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
                       "h2d_bytes_per_step": 8 * trace_blocks(trace) * (n_dest // max(1, n_replicas) if not same_device else 1),
                       "d2h_bytes_per_step": 16 * n_calls,
                       "api": "torch.ops.block_migration_ops.migrate_blocks, one awaited call per request"}
    line["batched"] = {"value": factor * total_bytes_per_step * args.steps / (ms_batched / 1e3) / 1e9, "unit": UNIT,
                       "launches_per_step_per_dest": int(p50[1].item()),
                       "api": "kvmig_migrate_blocks_async with the concatenated block lists of consecutive requests "
                              "(up to 4096 blocks, distinct targets) per launch"}
    if swap_info is not None:
        line["swap"] = swap_info
    if not args.no_cpu_baseline and args.gpus == 1:
        line["cpu_baseline"] = cpu_baseline(w, trace, same_device, args.cpu_seconds)
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

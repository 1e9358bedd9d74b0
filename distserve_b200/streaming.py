"""Layer-wise streaming of a request's KV from the context stage to the decoding
stage while prefill is still running.

The reference publishes a request to the decoding stage only after the whole
prefill batch has returned (distserve/single_stage_engine.py:393-401) and frees
its blocks only on the migration callback (405-410), so the whole transfer sits
between the end of prefill and the first decoding step.  Here the two halves of
the alternative are built:

* **producer** (context side, ``StreamingWorker.begin_layerwise_prefill`` /
  ``wait_layer_group``): a stand-in prefill that writes the request's KV layer
  group by layer group on its own stream — busy time standing for the group's
  compute, then the group's K/V written into the request's blocks — with an
  event after each group.  ``wait_layer_group(i)`` returns once group *i*'s
  event has completed; that return, travelling over the host channel to the
  controller (the actor pipe when the worker lives in another process), is the
  per-layer completion signal.  No device-side flag or wait is involved.
* **consumer** (decoding side, ``pull_layer_group`` / ``finish_pulls``): for each
  signalled group, ``migrate_layers_async`` of that window of global layers on a
  side stream; windows of one request are disjoint, so they overlap on the GPU.

``stream_request`` is the controller: it starts the prefill, relays each signal
to every decoding worker, and reports the *tail* — the time from the moment the
last group's KV is written to the moment the decoding workers hold everything —
which is what is left of the transfer on the request's critical path.
``whole_request`` measures the reference's order for comparison: the complete
prefill first, then one awaited ``migrate_blocks``.

    python -m distserve_b200.streaming [--workload c2|c4|...] [--gpus 1|2] [--groups 8]
"""
from __future__ import annotations

import argparse
import json
import time
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .config import CacheConfig, KVModelConfig, ParallelConfig
from .worker import KVWorker
from .workloads import WORKLOADS


def _resolve(x):
    return x.result() if hasattr(x, "result") else x


def layer_groups(num_layers: int, groups: int) -> List[Tuple[int, int]]:
    """`groups` contiguous windows of global layers covering [0, num_layers), sizes differing by at most one."""
    groups = max(1, min(groups, num_layers))
    edges = [round(i * num_layers / groups) for i in range(groups + 1)]
    return [(edges[i], edges[i + 1]) for i in range(groups) if edges[i] < edges[i + 1]]


class StreamingWorker(KVWorker):
    """A stage worker with the producer and consumer halves of layer-wise streaming."""

    # ---- context side ------------------------------------------------------------------------------------
    def stage_request_kv(self, block_ids: Sequence[int], seed: int) -> None:
        """Prepare what prefill will produce for this request: seeded K/V for the request's blocks, kept in a
        staging buffer until the stand-in prefill writes it into the pool group by group."""
        with torch.cuda.device(self.device):
            n = len(block_ids)
            g = torch.Generator(device=self.device).manual_seed(seed)
            shape = (n,) + tuple(self.k_cache.shape[1:])
            self._staged = (torch.empty(shape, dtype=self.k_cache.dtype, device=self.device).normal_(generator=g),
                            torch.empty(shape, dtype=self.k_cache.dtype, device=self.device).normal_(generator=g))
            self._staged_ids = torch.as_tensor(list(block_ids), dtype=torch.int64, device=self.device)
            if not hasattr(self, "prefill_stream"):
                self.prefill_stream = torch.cuda.Stream(device=self.device)
            torch.cuda.synchronize(self.device)

    def begin_layerwise_prefill(self, windows: Sequence[Tuple[int, int]], compute_us_per_group: float = 0.0) -> None:
        """Enqueue the whole stand-in prefill: per window of GLOBAL layers, `compute_us_per_group` of busy time, then
        the window's K/V written into the request's blocks (the part of the window this worker holds), then an
        event.  Returns at once; the stream runs on."""
        lo = self.parallel_config.pipeline_parallel_rank * self.k_cache.shape[1]
        hi = lo + self.k_cache.shape[1]
        self._group_events = []
        with torch.cuda.device(self.device), torch.cuda.stream(self.prefill_stream):
            for l0, l1 in windows:
                if compute_us_per_group > 0:
                    torch.cuda._sleep(int(compute_us_per_group * 1e3 * 1.9))      # about 1.9 cycles per ns
                a, b = max(l0, lo) - lo, min(l1, hi) - lo
                if a < b:
                    for pool, staged in zip((self.k_cache, self.v_cache), self._staged):
                        pool[:, a:b].index_copy_(0, self._staged_ids, staged[:, a:b])
                event = torch.cuda.Event()
                event.record(self.prefill_stream)
                self._group_events.append(event)

    def wait_layer_group(self, index: int) -> float:
        """Block until group `index` of the prefill in flight has been written; returns the host time of that
        moment.  This return is the completion signal."""
        self._group_events[index].synchronize()
        return time.time()

    def read_request_kv(self):
        """Bit patterns of the staged K/V (for a checker)."""
        return tuple(x.view(torch.int16).cpu().numpy() for x in self._staged)

    def pool_bits(self):
        torch.cuda.synchronize(self.device)
        return self.k_cache.view(torch.int16).cpu().numpy(), self.v_cache.view(torch.int16).cpu().numpy()

    def fill_pools(self, seed: int) -> None:
        g = torch.Generator(device=self.device).manual_seed(seed)
        for pool in (self.k_cache, self.v_cache):
            pool.normal_(generator=g)
        torch.cuda.synchronize(self.device)

    # ---- decoding side -----------------------------------------------------------------------------------
    def pull_layer_group(self, context_block_indexes, context_parallel_config, decoding_block_indexes,
                         layer_begin: int, layer_end: int) -> int:
        """Enqueue the pull of one signalled window on this worker's side stream; returns the ticket."""
        if not hasattr(self, "pull_stream"):
            with torch.cuda.device(self.device):
                self.pull_stream = torch.cuda.Stream(device=self.device)
        return self.migrate_layers_async(context_block_indexes, context_parallel_config, decoding_block_indexes,
                                         layer_begin, layer_end, stream=self.pull_stream)

    def finish_pulls(self, tickets: Sequence[int]) -> float:
        """Wait for the listed pulls; returns the host time at which the last one had finished."""
        for t in tickets:
            self.migrate_wait(t)
        return time.time()

    def migrate_blocks_timed(self, context_block_indexes, context_parallel_config, decoding_block_indexes) -> float:
        self.migrate_blocks(context_block_indexes, context_parallel_config, decoding_block_indexes)
        return time.time()


def make_streaming_worker(worker_id: int, stage: str, model: KVModelConfig, cache: CacheConfig, pc_list, device: int) -> StreamingWorker:
    """Factory for a worker process (``actors.ActorPool.spawn``)."""
    torch.cuda.set_device(device)
    tp, t, pp, p = pc_list
    return StreamingWorker(worker_id, stage, model, cache, ParallelConfig(tp, t, pp, p), device=device)


def stream_request(ctx_workers: Sequence, dec_workers: Sequence, ctx_pc: ParallelConfig, src: Sequence[int], dst: Sequence[int],
                   windows: Sequence[Tuple[int, int]], compute_us_per_group: float, observe=None) -> dict:
    """Run one request through the streamed order.  `ctx_workers` / `dec_workers` are the flattened stages (local
    objects, or actor proxies whose calls return futures).  `observe(k)` is called after window k's pulls have
    finished when given (tests look at the pools there; it serialises the windows, so timing runs pass None)."""
    src, dst = list(src), list(dst)
    for f in [w.begin_layerwise_prefill(list(windows), compute_us_per_group) for w in ctx_workers]:
        _resolve(f)
    tickets = [[] for _ in dec_workers]
    written = 0.0
    for k, (l0, l1) in enumerate(windows):
        # the signal: every context worker reports that it has written this group
        written = max(_resolve(f) for f in [w.wait_layer_group(k) for w in ctx_workers])
        for i, f in enumerate([w.pull_layer_group(src, ctx_pc, dst, l0, l1) for w in dec_workers]):
            tickets[i].append(_resolve(f))
        if observe is not None:
            for i, w in enumerate(dec_workers):
                _resolve(w.finish_pulls(tickets[i]))
            observe(k)
    done = max(_resolve(f) for f in [w.finish_pulls(tickets[i]) for i, w in enumerate(dec_workers)])
    return {"tail_ms": (done - written) * 1e3, "windows": len(windows)}


def whole_request(ctx_workers: Sequence, dec_workers: Sequence, ctx_pc: ParallelConfig, src: Sequence[int], dst: Sequence[int],
                  windows: Sequence[Tuple[int, int]], compute_us_per_group: float) -> dict:
    """The reference's order: the whole prefill, then one awaited migration per decoding worker."""
    src, dst = list(src), list(dst)
    for f in [w.begin_layerwise_prefill(list(windows), compute_us_per_group) for w in ctx_workers]:
        _resolve(f)
    written = max(_resolve(f) for f in [w.wait_layer_group(len(windows) - 1) for w in ctx_workers])
    done = max(_resolve(f) for f in [w.migrate_blocks_timed(src, ctx_pc, dst) for w in dec_workers])
    return {"tail_ms": (done - written) * 1e3, "windows": 1}


def measure(workload: str = "c2", gpus: int = 1, groups: int = 8, request_blocks: Optional[int] = None, pool_blocks: int = 512,
            compute_us_per_layer: float = 100.0, repeats: int = 20, seed: int = 3) -> dict:
    """Tail latency of a typical request of the workload, streamed in `groups` windows vs migrated whole, with
    every worker in this process: the context stage on GPU 0, decoding worker (0, 0) on GPU `gpus - 1`."""
    from . import load_ops

    load_ops()
    w = WORKLOADS[workload]
    cache = CacheConfig(w.block_size, 1 << 20)
    ctx_dev, dec_dev = 0, max(0, gpus - 1)
    if request_blocks is None:
        dist = w.length_dist
        typical = dist[1] if dist[0] == "lognormal" else (dist[1] + dist[2]) // 2
        request_blocks = -(-int(typical) // w.block_size)
    ctx_pc = w.ctx_config()
    ctx_workers = []
    for p in range(w.ctx_pp):
        for t in range(w.ctx_tp):
            ctx_workers.append(StreamingWorker(len(ctx_workers), "context", w.model, cache, w.ctx_config(p, t), device=ctx_dev))
    handles_flat = [cw.init_kvcache_and_swap(pool_blocks, 1) for cw in ctx_workers]
    table = [handles_flat[p * w.ctx_tp:(p + 1) * w.ctx_tp] for p in range(w.ctx_pp)]
    dec = StreamingWorker(100, "decoding", w.model, cache, w.dec_config(0, 0), device=dec_dev)
    dec.init_kvcache_and_swap(pool_blocks, 1)
    dec.register_kvcache_mem_handles(ctx_pc, table)
    rng = np.random.default_rng(seed)
    windows = layer_groups(w.model.num_layers, groups)
    per_group_us = compute_us_per_layer * w.model.num_layers / len(windows)
    tails = {"streamed": [], "whole": []}
    with torch.cuda.device(dec_dev):
        for r in range(repeats + 2):
            src = [int(x) for x in rng.permutation(pool_blocks)[:request_blocks]]
            dst = [int(x) for x in rng.permutation(pool_blocks)[:request_blocks]]
            for i, cw in enumerate(ctx_workers):
                cw.stage_request_kv(src, seed * 1000 + r * 10 + i)
            for mode, fn in (("streamed", stream_request), ("whole", whole_request)):
                out = fn(ctx_workers, [dec], ctx_pc, src, dst, windows, per_group_us)
                if r >= 2:
                    tails[mode].append(out["tail_ms"])
    med = {k: float(np.median(v)) for k, v in tails.items()}
    bytes_per_request = request_blocks * w.dec_block_bytes()
    return {"workload": w.name, "gpus": gpus, "request_blocks": request_blocks, "MB_per_request_per_dest": bytes_per_request / 1e6,
            "groups": len(windows), "layers_per_group": w.model.num_layers / len(windows),
            "stand_in_compute_us_per_layer": compute_us_per_layer, "repeats": repeats,
            "tail_ms_whole_request_p50": med["whole"], "tail_ms_streamed_p50": med["streamed"],
            "tail_removed_fraction": 1.0 - med["streamed"] / med["whole"] if med["whole"] > 0 else None,
            "tail_ms_streamed_min_max": [float(min(tails["streamed"])), float(max(tails["streamed"]))],
            "tail_ms_whole_min_max": [float(min(tails["whole"])), float(max(tails["whole"]))]}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="c2")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--groups", type=int, default=8)
    ap.add_argument("--pool-blocks", type=int, default=512)
    ap.add_argument("--compute-us-per-layer", type=float, default=100.0)
    ap.add_argument("--repeats", type=int, default=20)
    args = ap.parse_args()
    print(json.dumps(measure(args.workload, args.gpus, args.groups, None, args.pool_blocks, args.compute_us_per_layer, args.repeats)))


if __name__ == "__main__":
    main()

"""Seeded synthetic migration workloads with the shapes of the benchmark
configurations: model geometry, stage layouts, request counts and prompt-length
distributions.  Only prompt *lengths* reach this path (a request moves
``ceil(len / block_size)`` whole blocks), so length distributions stand in for
the public prompt datasets the reference serves.

A trace is produced by running two block managers — one per stage — the way
the engines do: the context stage allocates a prompt's blocks, the decoding
stage reserves the same number, the blocks move, the context stage recycles
its blocks at once (distserve/single_stage_engine.py:536).  When the decoding
pool cannot hold the next request, its oldest resident requests are released
first (they stand for requests that finished decoding).  Both free lists start
as seeded permutations, the state a long-running server's lists are in after
many frees (distserve/block_manager.py:44,82-83,158).
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Dict, List, Tuple

import numpy as np

from .block_manager import BlockManager
from .config import CacheConfig, KVModelConfig, ParallelConfig
from .request import Request


@dataclass(frozen=True)
class Workload:
    name: str
    model: KVModelConfig
    block_size: int
    ctx_tp: int
    ctx_pp: int
    dec_tp: int
    dec_pp: int
    num_requests: int
    length_dist: Tuple          # ("uniform", lo, hi) or ("lognormal", median, sigma, cap)
    ctx_pool_blocks: int
    dec_pool_blocks: int
    seed: int
    note: str = ""

    def ctx_config(self, pp_rank: int = 0, tp_rank: int = 0) -> ParallelConfig:
        return ParallelConfig(self.ctx_tp, tp_rank, self.ctx_pp, pp_rank)

    def dec_config(self, pp_rank: int = 0, tp_rank: int = 0) -> ParallelConfig:
        return ParallelConfig(self.dec_tp, tp_rank, self.dec_pp, pp_rank)

    def dec_block_bytes(self) -> int:
        """Bytes written into one decoding worker per migrated block, K and V
        together — the algorithmic bytes of the path."""
        return 2 * self.model.block_bytes(self.dec_config(), self.block_size)

    def scaled(self, num_requests: int = None, ctx_pool_blocks: int = None, dec_pool_blocks: int = None) -> "Workload":
        return replace(self, num_requests=num_requests or self.num_requests,
                       ctx_pool_blocks=ctx_pool_blocks or self.ctx_pool_blocks,
                       dec_pool_blocks=dec_pool_blocks or self.dec_pool_blocks)


@dataclass(frozen=True)
class TraceItem:
    request_id: int
    prompt_len: int
    src_blocks: Tuple[int, ...]
    dst_blocks: Tuple[int, ...]


# sigma of the lognormal length distributions is not fixed by the benchmark
# description; 0.7 is used throughout and recorded with every result.
LOGNORMAL_SIGMA = 0.7

WORKLOADS: Dict[str, Workload] = {
    # OPT-125M-shaped, CPU-runnable
    "c1": Workload("c1-opt125m-tp1-to-tp1", KVModelConfig(12, 12, 64), 16, 1, 1, 1, 1, 32,
                   ("uniform", 64, 512), 512, 512, 1001),
    # OPT-13B-shaped, one context GPU -> one decoding GPU
    "c2": Workload("c2-opt13b-tp1-to-tp1", KVModelConfig(40, 40, 128), 16, 1, 1, 1, 1, 64,
                   ("lognormal", 700, LOGNORMAL_SIGMA, 2048), 4096, 4096, 1002),
    # LLaMA-2-13B-shaped, context tp=2 -> decoding tp=1
    "c3": Workload("c3-llama13b-tp2-to-tp1", KVModelConfig(40, 40, 128), 16, 2, 1, 1, 1, 128,
                   ("uniform", 128, 2048), 4096, 4096, 1003, "pool size not fixed by the description; 4096 used"),
    # LLaMA-2-70B-shaped GQA, context tp=4,pp=1 -> decoding tp=2,pp=2
    "c4": Workload("c4-llama70b-tp4pp1-to-tp2pp2", KVModelConfig(80, 8, 128), 16, 4, 1, 2, 2, 256,
                   ("lognormal", 1024, LOGNORMAL_SIGMA, 4096), 8192, 8192, 1004, "pool size not fixed; 8192 used"),
    # LLaMA-2-7B-shaped, context tp=2 -> decoding tp=2 (the end-to-end loop's layout)
    "c5": Workload("c5-llama7b-tp2-to-tp2", KVModelConfig(32, 32, 128), 16, 2, 1, 2, 1, 64,
                   ("lognormal", 512, LOGNORMAL_SIGMA, 2048), 4096, 4096, 1005),
}


def _rng(seed: int, stream: int) -> np.random.Generator:
    return np.random.default_rng([seed, stream])


def prompt_lengths(w: Workload) -> List[int]:
    rng = _rng(w.seed, 0)
    kind = w.length_dist[0]
    if kind == "uniform":
        _, lo, hi = w.length_dist
        return [int(x) for x in rng.integers(lo, hi + 1, size=w.num_requests)]
    if kind == "lognormal":
        _, median, sigma, cap = w.length_dist
        raw = rng.lognormal(mean=np.log(median), sigma=sigma, size=w.num_requests)
        return [int(min(cap, max(1, round(x)))) for x in raw]
    raise ValueError(f"unknown length distribution {kind!r}")


def _noop(*_args, **_kwargs):
    return []


def make_trace(w: Workload) -> List[TraceItem]:
    """Block-id lists of every request of the workload, in arrival order."""
    cache = CacheConfig(w.block_size, max_num_blocks_per_req=1 << 30)
    ctx_bm = BlockManager("context", w.ctx_pool_blocks, 1, w.model, w.ctx_config(), cache, _noop)
    dec_bm = BlockManager("decoding", w.dec_pool_blocks, 1, w.model, w.dec_config(), cache, _noop)
    ctx_bm.free_gpu_blocks_list[:] = [int(x) for x in _rng(w.seed, 1).permutation(w.ctx_pool_blocks)]
    dec_bm.free_gpu_blocks_list[:] = [int(x) for x in _rng(w.seed, 2).permutation(w.dec_pool_blocks)]
    resident: List[int] = []
    trace: List[TraceItem] = []
    for rid, n_tokens in enumerate(prompt_lengths(w)):
        req = Request.of_length(rid, n_tokens)
        need = dec_bm.get_num_blocks_needed(req)
        if need > w.dec_pool_blocks or need > w.ctx_pool_blocks:
            raise ValueError(f"request {rid} needs {need} blocks, more than a pool holds")
        ctx_bm.allocate_blocks(req)
        src = tuple(ctx_bm.get_block_table(rid))
        while dec_bm.get_num_avail_gpu_blocks() < need:
            dec_bm.free_blocks(resident.pop(0))
        dec_bm.allocate_blocks(req)
        resident.append(rid)
        dst = tuple(dec_bm.get_block_table(rid))
        ctx_bm.free_blocks(rid)
        trace.append(TraceItem(rid, n_tokens, src, dst))
    return trace


def trace_blocks(trace: List[TraceItem]) -> int:
    return sum(len(t.src_blocks) for t in trace)

"""Read-back of sampled requests after a multi-process migration run, for a
bit-exact check by whoever holds a checker: the "per-request slab read-back"
that pools too large for host memory call for.

Every rank computes the same plan from the trace and the rank roles.  For each
sampled request, every contributing *context* rank copies the request's source
blocks out of its OWN pool to host memory and sends them to the decoding rank
over the process group (gloo: host tensors only); the *decoding* rank copies
its own target blocks to host memory.  No rank touches another GPU's memory
here — that is what the copy kernel under test did.  What the decoding rank
ends up with is, per sample, compact source pools (block i of the sample is
block i of the pool) and the blocks it actually holds, ready for a checker
that re-executes the migration on the host.

Sampled requests are those whose target blocks no later request of the same
decoding worker wrote again, so that the pools' final state still shows them.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np

from .config import plan_overlaps
from .launch import Role, num_replicas, shard_trace
from .workloads import TraceItem, Workload


@dataclass(frozen=True)
class Sample:
    dec_rank: int                      # rank of the decoding worker that is checked
    dec_pp_rank: int
    dec_tp_rank: int
    request_id: int
    src_blocks: Tuple[int, ...]        # the sampled blocks' ids in the context pools
    dst_blocks: Tuple[int, ...]        # ... and in the decoding worker's pools
    ctx_ranks: Tuple[Tuple[int, int, int], ...]   # (pp_rank, tp_rank, rank) of every contributing context worker


def surviving_requests(trace: Sequence[TraceItem]) -> List[TraceItem]:
    """Requests none of whose target blocks a later request of the trace wrote again."""
    last_writer: Dict[int, int] = {}
    for item in trace:
        for d in item.dst_blocks:
            last_writer[d] = item.request_id
    return [item for item in trace if item.dst_blocks and all(last_writer[d] == item.request_id for d in item.dst_blocks)]


def never_written_blocks(trace: Sequence[TraceItem], pool_blocks: int) -> List[int]:
    """Target-pool blocks that no request of the trace names."""
    used = {d for item in trace for d in item.dst_blocks}
    return [b for b in range(pool_blocks) if b not in used]


def _spread(items: Sequence, k: int) -> List:
    if len(items) <= k:
        return list(items)
    picks = sorted({round(i * (len(items) - 1) / (k - 1)) for i in range(k)}) if k > 1 else [len(items) - 1]
    return [items[i] for i in picks]


def plan_samples(workload: Workload, roles: Optional[Dict[int, Role]], trace: Sequence[TraceItem], requests_per_worker: int = 8,
                 blocks_per_request: int = 12, traces_by_rank: Optional[Dict[int, Sequence[TraceItem]]] = None) -> List[Sample]:
    """The same list on every rank, ordered by decoding rank and request.  With `roles` None (one process
    holding both stages) every worker is rank 0.  `traces_by_rank` replaces the share of `trace` that a
    decoding rank would be dealt by what that rank actually migrated (its own records, made known to every
    rank beforehand)."""
    if roles is None:
        roles = {0: Role("both")}
    ctx_rank_of = {}
    for rank, role in roles.items():
        if role.stage in ("ctx", "both"):
            for p in range(workload.ctx_pp):
                for t in range(workload.ctx_tp):
                    if role.stage == "both" or (role.pp_rank, role.tp_rank) == (p, t):
                        ctx_rank_of[(p, t)] = rank
    replicas = num_replicas(roles)
    out: List[Sample] = []
    for rank in sorted(roles):
        role = roles[rank]
        if role.stage not in ("dec", "both"):
            continue
        if traces_by_rank is not None:
            mine = list(traces_by_rank.get(rank) or [])
        else:
            mine = list(trace) if role.stage == "both" else shard_trace(trace, role, replicas)
        dec = workload.dec_config(role.pp_rank, role.tp_rank)
        overlaps = plan_overlaps(workload.model, workload.ctx_config(), dec)
        contributors = tuple((o.ctx_pp_rank, o.ctx_tp_rank, ctx_rank_of[(o.ctx_pp_rank, o.ctx_tp_rank)]) for o in overlaps)
        for item in _spread(surviving_requests(mine), requests_per_worker):
            positions = _spread(range(len(item.dst_blocks)), blocks_per_request)
            out.append(Sample(rank, role.pp_rank, role.tp_rank, item.request_id,
                              tuple(item.src_blocks[i] for i in positions), tuple(item.dst_blocks[i] for i in positions),
                              contributors))
    return out


ReadBlocks = Callable[[Sequence[int]], Tuple[np.ndarray, np.ndarray]]   # block ids -> (K slabs, V slabs) on the host


@dataclass
class ReadBack:
    sample: Sample
    ctx_pools: Dict[Tuple[int, int], Tuple[np.ndarray, np.ndarray]]   # compact: sample block i is pool block i
    target: Tuple[np.ndarray, np.ndarray]                             # the decoding worker's blocks, same order


def exchange_samples(samples: Sequence[Sample], rank: int, read_source: Optional[ReadBlocks], read_target: Optional[ReadBlocks],
                     dist=None) -> List[ReadBack]:
    """Run the plan: context ranks send, decoding ranks receive and read their own blocks.  Every rank walks the
    plan in the same order and each transfer involves exactly two ranks, so the pairwise sends cannot deadlock.
    Returns the read-backs of the samples this rank checks (empty on pure context ranks)."""
    import torch

    out: List[ReadBack] = []
    for s in samples:
        pools: Dict[Tuple[int, int], Tuple[np.ndarray, np.ndarray]] = {}
        for p, t, ctx_rank in s.ctx_ranks:
            if ctx_rank == rank:
                k, v = read_source_for(read_source, (p, t))(s.src_blocks)
                if s.dec_rank == rank:
                    pools[(p, t)] = (k, v)
                else:
                    for arr in (k, v):
                        header = torch.tensor(list(arr.shape) + [arr.dtype.itemsize], dtype=torch.int64)
                        dist.send(header, dst=s.dec_rank)
                        dist.send(torch.from_numpy(np.ascontiguousarray(arr)).view(torch.uint8).reshape(-1), dst=s.dec_rank)
            elif s.dec_rank == rank:
                got = []
                for _ in range(2):
                    header = torch.zeros(6, dtype=torch.int64)
                    dist.recv(header, src=ctx_rank)
                    *shape, itemsize = [int(x) for x in header]
                    flat = torch.empty(int(np.prod(shape)) * itemsize, dtype=torch.uint8)
                    dist.recv(flat, src=ctx_rank)
                    got.append(flat.numpy().view({1: np.int8, 2: np.int16, 4: np.int32, 8: np.int64}[itemsize]).reshape(shape))
                pools[(p, t)] = (got[0], got[1])
        if s.dec_rank == rank:
            out.append(ReadBack(s, pools, read_target(s.dst_blocks)))
    return out


def read_source_for(read_source, key):
    """`read_source` is either one reader (this rank holds one context worker) or a dict of readers keyed by
    (pp_rank, tp_rank) (one process holding several context workers)."""
    return read_source[key] if isinstance(read_source, dict) else read_source


def torch_pool_reader(k_pool, v_pool) -> ReadBlocks:
    """Reader over a worker's own device pools: gathers the blocks on that GPU and copies them to the host as
    integers of the element width (bit patterns, so that comparisons are exact for any float type)."""
    import torch

    width = {1: torch.int8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[k_pool.element_size()]

    def read(block_ids: Sequence[int]):
        idx = torch.as_tensor(list(block_ids), dtype=torch.int64, device=k_pool.device)
        return tuple(pool.view(width).index_select(0, idx).cpu().numpy() for pool in (k_pool, v_pool))

    return read

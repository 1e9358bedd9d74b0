"""Placing the two stages' workers on the ranks of a one-node job and handing
the context stage's pool handles to the decoding workers — what the reference
does with Ray placement groups and actor return values
(distserve/engine.py:168-216, distserve/single_stage_engine.py:194-223,469-483),
done here over a ``torch.distributed`` group (gloo: only small Python objects
travel; the KV payload never touches a collective).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

from .workloads import TraceItem, Workload


@dataclass(frozen=True)
class Role:
    stage: str        # "ctx" | "dec" | "idle"
    pp_rank: int = 0
    tp_rank: int = 0
    replica: int = 0


def plan_roles(workload: Workload, world_size: int) -> Dict[int, Role]:
    """rank -> role.  The context stage takes the first tp*pp ranks,
    pipeline-major like the reference's worker grid; every further group of
    dec_tp*dec_pp ranks is one decoding replica; leftovers idle."""
    n_ctx = workload.ctx_tp * workload.ctx_pp
    n_dec = workload.dec_tp * workload.dec_pp
    if world_size < n_ctx + n_dec:
        raise ValueError(f"workload {workload.name} needs {n_ctx + n_dec} ranks, got {world_size}")
    roles: Dict[int, Role] = {}
    rank = 0
    for p in range(workload.ctx_pp):
        for t in range(workload.ctx_tp):
            roles[rank] = Role("ctx", p, t)
            rank += 1
    replica = 0
    while rank + n_dec <= world_size:
        for p in range(workload.dec_pp):
            for t in range(workload.dec_tp):
                roles[rank] = Role("dec", p, t, replica)
                rank += 1
        replica += 1
    for r in range(rank, world_size):
        roles[r] = Role("idle")
    return roles


def num_replicas(roles: Dict[int, Role]) -> int:
    return max(1, len({r.replica for r in roles.values() if r.stage == "dec"}))


def handle_table(workload: Workload, roles: Dict[int, Role], per_rank_handles: Sequence) -> List[List[Tuple[List[int], List[int]]]]:
    """Arrange what each rank returned from ``init_kvcache_and_swap`` (None for
    non-context ranks) as [pp_rank][tp_rank] -> (k_handle, v_handle)."""
    table: List[List[Optional[tuple]]] = [[None] * workload.ctx_tp for _ in range(workload.ctx_pp)]
    for rank, role in roles.items():
        if role.stage == "ctx":
            if per_rank_handles[rank] is None:
                raise ValueError(f"context rank {rank} returned no handles")
            table[role.pp_rank][role.tp_rank] = tuple(per_rank_handles[rank])
    if any(cell is None for row in table for cell in row):
        raise ValueError("handle table has holes: a context rank is missing")
    return table


def exchange_handles(workload: Workload, roles: Dict[int, Role], my_handles, group=None):
    """all_gather_object of the per-rank handles, then :func:`handle_table`."""
    import torch.distributed as dist

    gathered = [None] * dist.get_world_size(group)
    dist.all_gather_object(gathered, my_handles, group=group)
    return handle_table(workload, roles, gathered)


def shard_trace(trace: Sequence[TraceItem], role: Role, replicas: int) -> List[TraceItem]:
    """Requests are dealt round-robin to the decoding replicas; every worker of
    a replica sees all of that replica's requests (each pulls its own slice)."""
    if role.stage != "dec":
        return []
    return [item for i, item in enumerate(trace) if i % replicas == role.replica]

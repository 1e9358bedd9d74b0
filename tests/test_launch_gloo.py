"""Host logic of the multi-rank path on CPU: role placement, trace sharding,
and the handle hand-off over a world_size-2 gloo group."""
import multiprocessing as mp
import os

import pytest

from distserve_b200.launch import Role, handle_table, num_replicas, plan_roles, shard_trace
from distserve_b200.workloads import WORKLOADS, make_trace, trace_blocks


def test_roles_for_the_benchmark_layouts():
    r2 = plan_roles(WORKLOADS["c2"], 2)
    assert r2 == {0: Role("ctx", 0, 0), 1: Role("dec", 0, 0, 0)}
    r4 = plan_roles(WORKLOADS["c3"], 4)
    assert [r4[i].stage for i in range(4)] == ["ctx", "ctx", "dec", "dec"]
    assert (r4[0].tp_rank, r4[1].tp_rank) == (0, 1) and (r4[2].replica, r4[3].replica) == (0, 1)
    assert num_replicas(r4) == 2
    r8 = plan_roles(WORKLOADS["c4"], 8)
    assert [(r8[i].stage, r8[i].pp_rank, r8[i].tp_rank) for i in range(8)] == [
        ("ctx", 0, 0), ("ctx", 0, 1), ("ctx", 0, 2), ("ctx", 0, 3),
        ("dec", 0, 0), ("dec", 0, 1), ("dec", 1, 0), ("dec", 1, 1)]
    assert plan_roles(WORKLOADS["c5"], 8)[7] == Role("dec", 0, 1, 2)       # ctx pair + three decoding pairs
    assert plan_roles(WORKLOADS["c2"], 3)[2] == Role("dec", 0, 0, 1)
    assert plan_roles(WORKLOADS["c3"], 5)[4].stage == "dec" and plan_roles(WORKLOADS["c4"], 8)[7].replica == 0
    with pytest.raises(ValueError):
        plan_roles(WORKLOADS["c4"], 4)


def test_trace_sharding_covers_every_request_once():
    w = WORKLOADS["c3"]
    trace = make_trace(w)
    roles = plan_roles(w, 4)
    parts = [shard_trace(trace, roles[r], num_replicas(roles)) for r in range(4)]
    assert parts[0] == [] and parts[1] == []
    assert sorted(t.request_id for t in parts[2] + parts[3]) == list(range(len(trace)))
    assert trace_blocks(parts[2]) + trace_blocks(parts[3]) == trace_blocks(trace)
    # both workers of one tp=2 decoding replica see the same requests
    w5 = WORKLOADS["c5"]
    r5 = plan_roles(w5, 4)
    t5 = make_trace(w5)
    assert shard_trace(t5, r5[2], 1) == shard_trace(t5, r5[3], 1) == list(t5)


def test_handle_table_shape_and_holes():
    w = WORKLOADS["c4"]
    roles = plan_roles(w, 8)
    per_rank = [([r], [100 + r]) if roles[r].stage == "ctx" else None for r in range(8)]
    table = handle_table(w, roles, per_rank)
    assert len(table) == 1 and [cell[0] for cell in table[0]] == [[0], [1], [2], [3]]
    per_rank[2] = None
    with pytest.raises(ValueError):
        handle_table(w, roles, per_rank)


def _rank_main(rank, world, port, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist

    from distserve_b200.launch import exchange_handles

    dist.init_process_group("gloo", rank=rank, world_size=world)
    w = WORKLOADS["c2"]
    roles = plan_roles(w, world)
    mine = ([11] * 24, [22] * 24) if roles[rank].stage == "ctx" else None     # stand-ins for exported handles
    table = exchange_handles(w, roles, mine)
    trace = make_trace(w)
    part = shard_trace(trace, roles[rank], num_replicas(roles))
    queue.put((rank, table, len(part)))
    dist.barrier()
    dist.destroy_process_group()


def test_handle_exchange_over_gloo_world_size_2():
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = 29600 + os.getpid() % 300
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, queue)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(queue.get(timeout=240) for _ in procs)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    (r0, t0, n0), (r1, t1, n1) = results
    assert t0 == t1 == [[([11] * 24, [22] * 24)]]
    assert (n0, n1) == (0, 64)

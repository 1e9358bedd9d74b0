"""The benchmark's multi-GPU result check, exercised on CPU: which requests are
sampled, the slab exchange between a context rank and a decoding rank over a
world-size-2 gloo group (numpy pools standing in for the device pools), and the
oracle comparison — which must fail when a single value is wrong."""
import multiprocessing as mp
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from distserve_b200 import spotcheck
from distserve_b200.launch import plan_roles
from distserve_b200.workloads import WORKLOADS, TraceItem, make_trace
from oracle import kv_oracle as O


def test_only_requests_whose_blocks_survive_are_sampled():
    trace = [TraceItem(0, 32, (5, 6), (1, 2)), TraceItem(1, 32, (7, 8), (2, 3)), TraceItem(2, 16, (9,), (4,)),
             TraceItem(3, 0, (), ())]
    assert [t.request_id for t in spotcheck.surviving_requests(trace)] == [1, 2]
    assert spotcheck.never_written_blocks(trace, 7) == [0, 5, 6]


@pytest.mark.parametrize("name,world", [("c2", 2), ("c3", 4), ("c4", 8), ("c5", 4)])
def test_sample_plans_name_the_contributing_context_ranks(name, world):
    w = WORKLOADS[name].scaled(num_requests=24)
    trace = make_trace(w)
    roles = plan_roles(w, world)
    samples = spotcheck.plan_samples(w, roles, trace)
    dec_ranks = [r for r, role in roles.items() if role.stage == "dec"]
    assert {s.dec_rank for s in samples} == set(dec_ranks)
    for s in samples:
        assert 1 <= len(s.src_blocks) == len(s.dst_blocks) <= 12
        want = O.contributing_workers(w.model.num_layers, w.model.num_kv_heads, w.ctx_tp, w.ctx_pp, w.dec_tp, s.dec_tp_rank,
                                      w.dec_pp, s.dec_pp_rank)
        assert [(p, t) for p, t, _ in s.ctx_ranks] == want
        for p, t, rank in s.ctx_ranks:
            assert roles[rank].stage == "ctx" and (roles[rank].pp_rank, roles[rank].tp_rank) == (p, t)
        item = trace[s.request_id]
        pairs = set(zip(item.src_blocks, item.dst_blocks))
        assert all(pair in pairs for pair in zip(s.src_blocks, s.dst_blocks))
    per_worker = {r: sum(1 for s in samples if s.dec_rank == r) for r in dec_ranks}
    assert all(1 <= n <= 8 for n in per_worker.values())


def _numpy_reader(k, v):
    return lambda ids: (k[list(ids)].copy(), v[list(ids)].copy())


def _apply_trace(w, trace, ctx_pools, dec_k, dec_v, t_rank=0, p_rank=0):
    for item in trace:
        O.migrate_blocks_numpy(ctx_pools, w.ctx_tp, w.ctx_pp, list(item.src_blocks), w.dec_tp, t_rank, w.dec_pp, p_rank,
                               list(item.dst_blocks), dec_k, dec_v, w.model.num_layers, w.model.num_kv_heads)


def _small_workload():
    from dataclasses import replace

    from distserve_b200.config import KVModelConfig

    return replace(WORKLOADS["c2"], model=KVModelConfig(4, 4, 8), block_size=4, num_requests=20, ctx_pool_blocks=96,
                   dec_pool_blocks=64, length_dist=("uniform", 4, 40))


def _pools(w, seed):
    rng = np.random.default_rng(seed)
    shape = lambda n, pc: (n, w.model.get_num_layers(pc), w.model.get_num_heads(pc), w.block_size, w.model.head_dim)
    ck = rng.integers(-30000, 30000, size=shape(w.ctx_pool_blocks, w.ctx_config()), dtype=np.int16)
    cv = rng.integers(-30000, 30000, size=shape(w.ctx_pool_blocks, w.ctx_config()), dtype=np.int16)
    dk = np.zeros(shape(w.dec_pool_blocks, w.dec_config()), dtype=np.int16)
    return ck, cv, dk, dk.copy()


def _rank_main(rank, world, port, queue, corrupt):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist

    import bench

    dist.init_process_group("gloo", rank=rank, world_size=world)
    w = _small_workload()
    trace = make_trace(w)
    roles = plan_roles(w, world)                          # rank 0 context, rank 1 decoding
    ck, cv, dk, dv = _pools(w, 5)                         # both ranks build the same arrays; each uses its own side
    read_source = read_target = None
    if roles[rank].stage == "ctx":
        read_source = _numpy_reader(ck, cv)
    else:
        _apply_trace(w, trace, {(0, 0): (ck, cv)}, dk, dv)     # what a correct migration leaves in the decoding pools
        if corrupt:
            victim = spotcheck.plan_samples(w, roles, trace)[0].dst_blocks[0]
            dv[victim, 1, 2, 3, 4] ^= 1                   # one wrong bit in one sampled block
        read_target = _numpy_reader(dk, dv)
    samples = spotcheck.plan_samples(w, roles, trace)
    readbacks = spotcheck.exchange_samples(samples, rank, read_source, read_target, dist)
    n, blocks, bad = bench.check_readbacks(w, readbacks)
    queue.put((rank, n, blocks, bad))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("corrupt", [False, True])
def test_exchange_and_oracle_check_over_gloo_world_size_2(corrupt):
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = 29900 + os.getpid() % 200 + (50 if corrupt else 0)
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, queue, corrupt)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(2):
        rank, n, blocks, bad = queue.get(timeout=300)
        got[rank] = (n, blocks, bad)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert got[0] == (0, 0, [])                           # the context rank only sends
    n, blocks, bad = got[1]
    assert n >= 1 and blocks >= n
    if corrupt:
        assert len(bad) == 1 and bad[0][0] == 1           # the decoding rank's first sampled request is reported
    else:
        assert bad == []


def test_single_process_check_and_a_wrong_expected_value():
    """One process holding both stages (the 1-GPU benchmark): the same plan and checker, no process group."""
    import bench

    w = _small_workload()
    trace = make_trace(w)
    ck, cv, dk, dv = _pools(w, 6)
    _apply_trace(w, trace, {(0, 0): (ck, cv)}, dk, dv)
    samples = spotcheck.plan_samples(w, None, trace)
    assert samples and all(s.dec_rank == 0 for s in samples)
    readbacks = spotcheck.exchange_samples(samples, 0, {(0, 0): _numpy_reader(ck, cv)}, _numpy_reader(dk, dv))
    assert bench.check_readbacks(w, readbacks)[2] == []
    # the checker itself must notice a wrong source slab (i.e. a wrong expected value)
    readbacks[-1].ctx_pools[(0, 0)][0][0, 0, 0, 0, 0] ^= 0x10
    n, blocks, bad = bench.check_readbacks(w, readbacks)
    assert bad == [(0, readbacks[-1].sample.request_id)]

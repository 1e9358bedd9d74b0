"""The one-process-per-worker harness: ordering, failures on the host side,
and (on a GPU) the stage engines driving workers that live in other processes."""
import numpy as np
import pytest

from distserve_b200.actors import ActorError, ActorPool
from tests import actor_fixtures as F


def test_calls_run_in_order_and_results_come_back():
    with ActorPool() as pool:
        a = pool.spawn(F.Echo, "a", env={"ACTOR_TEST_ENV": "x1"})
        b = pool.spawn(F.Echo, "b")
        futures = [a.add(i, 1, delay=0.01 if i == 0 else 0.0) for i in range(20)]
        assert [f.result(60) for f in futures] == [i + 1 for i in range(20)]
        assert a.history().result(60) == [(i, 1) for i in range(20)]       # submission order, one at a time
        tag, pid, env = a.whoami().result(60)
        assert (tag, env) == ("a", "x1") and pid == a.pid and pid != b.pid
        assert b.history().result(60) == []


def test_failures_surface_on_the_host():
    with ActorPool() as pool:
        with pytest.raises(ActorError, match="refusing to start"):
            pool.spawn(F.Echo, "c", fail_on_start=True)
        a = pool.spawn(F.Echo, "a")
        with pytest.raises(ActorError, match="RuntimeError: boom"):
            a.fail("boom").result(60)
        assert a.add(2, 3).result(60) == 5                                   # the actor survives a failed call
        with pytest.raises(ActorError, match="AttributeError"):
            a.no_such_method().result(60)
        # a worker that exits between steps: the pending and every later call fail, nothing hangs
        doomed = a.die()
        with pytest.raises(ActorError, match="ended before answering"):
            doomed.result(60)
        with pytest.raises(ActorError):
            a.add(1, 1).result(60)
        assert not a.is_alive()


@pytest.mark.gpu
def test_stage_engines_over_worker_processes():
    """Context tp=2 and decoding tp=1·pp=2 workers, each in its own process
    (spread over the available GPUs), driven by the engines in this process;
    handles travel pickled, data moves GPU to GPU."""
    import torch

    from distserve_b200.config import CacheConfig, KVModelConfig, ParallelConfig
    from distserve_b200.request import Request
    from distserve_b200.stage import ContextStageEngine, DecodingStageEngine
    from oracle import kv_oracle as O

    n_gpu = torch.cuda.device_count()
    model, cache = KVModelConfig(8, 8, 32), CacheConfig(16, 1 << 20)
    ctx_pc, dec_pc = ParallelConfig(2, 0, 1, 0), ParallelConfig(1, 0, 2, 0)
    with ActorPool() as pool:
        spec = (8, 8, 32, 16)
        ctx_workers = [[pool.spawn(F.make_kv_worker, t, "context", *spec, [2, t, 1, 0], t % n_gpu) for t in range(2)]]
        dec_workers = [[pool.spawn(F.make_kv_worker, 2 + p, "decoding", *spec, [1, 0, 2, p], (2 + p) % n_gpu)] for p in range(2)]
        ctx_engine = ContextStageEngine(model, ctx_pc, cache, ctx_workers)
        dec_engine = DecodingStageEngine(model, dec_pc, cache, dec_workers,
                                         clear_migrated_blocks_callback=ctx_engine.clear_migrated_blocks)
        handles = ctx_engine.init_kvcache(64, 1)
        dec_engine.init_kvcache(48, 1)
        for i, w in enumerate([w for row in ctx_workers + dec_workers for w in row]):
            w.fill(100 + i).result(120)
        dec_engine.register_kvcache_mem_handles(ctx_pc, handles)
        src_host = {(0, t): ctx_workers[0][t].snapshot().result(120) for t in range(2)}
        dst_host = {(p, 0): tuple(a.copy() for a in dec_workers[p][0].snapshot().result(120)) for p in range(2)}
        rng = np.random.default_rng(5)
        singles = [ctx_engine.finish_prefill(Request.of_length(r, int(rng.integers(1, 120)))) for r in range(3)]
        batch = [ctx_engine.finish_prefill(Request.of_length(3 + r, int(rng.integers(1, 120)))) for r in range(4)]
        done = [(m, dec_engine.migrate_blocks(m)) for m in singles]
        done += list(zip(batch, dec_engine.migrate_blocks_batched(batch)))
        for m, target in done:
            for (p, t), (k, v) in dst_host.items():
                O.migrate_blocks_numpy(src_host, 2, 1, m.block_indexes, 1, t, 2, p, target, k, v, 8, 8)
        for p in range(2):
            gk, gv = dec_workers[p][0].snapshot().result(120)
            assert np.array_equal(gk, dst_host[(p, 0)][0]) and np.array_equal(gv, dst_host[(p, 0)][1])
        assert ctx_engine.block_manager.get_num_avail_gpu_blocks() == 64
        # a refusal inside a worker process reaches the engine as an exception, as in the reference
        with pytest.raises(ActorError, match="outside the context pool"):
            dec_workers[0][0].migrate_blocks([999], ctx_pc, [0]).result(120)

"""The full call chain of the reference — stage engines, block managers,
workers, operator shim — on the OPT-125M-shaped workload and on resharded
layouts, replayed against the oracle; plus two worker processes exchanging
CUDA IPC handles."""
import multiprocessing as mp

import numpy as np
import pytest
import torch

from distserve_b200 import capi
from distserve_b200.config import CacheConfig, KVModelConfig, ParallelConfig
from distserve_b200.request import Request
from distserve_b200.stage import ContextStageEngine, DecodingStageEngine
from distserve_b200.worker import KVWorker
from distserve_b200.workloads import WORKLOADS, make_trace, prompt_lengths
from oracle import kv_oracle as O

pytestmark = pytest.mark.gpu


def build_stages(model, block_size, ctx, dec, ctx_blocks, dec_blocks, seed):
    cache = CacheConfig(block_size, 1 << 20)

    def grid(stage, pc):
        return [[KVWorker(p * pc.tensor_parallel_size + t, stage, model, cache, pc.with_rank(p, t))
                 for t in range(pc.tensor_parallel_size)] for p in range(pc.pipeline_parallel_size)]

    ctx_engine = ContextStageEngine(model, ctx, cache, grid("context", ctx))
    dec_engine = DecodingStageEngine(model, dec, cache, grid("decoding", dec),
                                     clear_migrated_blocks_callback=ctx_engine.clear_migrated_blocks)
    handles = ctx_engine.init_kvcache(ctx_blocks, 1)
    dec_engine.init_kvcache(dec_blocks, 1)
    g = torch.Generator(device="cuda").manual_seed(seed)
    for engine in (ctx_engine, dec_engine):
        for row in engine.workers:
            for w in row:
                for pool in (w.k_cache, w.v_cache):
                    pool.copy_(torch.randn(pool.shape, device="cuda", generator=g).to(pool.dtype))
    dec_engine.register_kvcache_mem_handles(ctx, handles)
    return ctx_engine, dec_engine


def host_copy(engine):
    return {(p, t): (w.k_cache.cpu().view(torch.int16).numpy().copy(), w.v_cache.cpu().view(torch.int16).numpy().copy())
            for p, row in enumerate(engine.workers) for t, w in enumerate(row)}


def run_and_check(model, block_size, ctx, dec, ctx_blocks, dec_blocks, lengths, seed):
    capi.reset_registry()
    ctx_engine, dec_engine = build_stages(model, block_size, ctx, dec, ctx_blocks, dec_blocks, seed)
    src_host, dst_host = host_copy(ctx_engine), host_copy(dec_engine)
    resident = []
    for rid, n in enumerate(lengths):
        req = Request.of_length(rid, n)
        need = -(-n // block_size)
        while dec_engine.block_manager.get_num_avail_gpu_blocks() < need:
            dec_engine.block_manager.free_blocks(resident.pop(0))
        migrating = ctx_engine.finish_prefill(req)
        req.append_token()                                   # the prefill step produced one token
        target = dec_engine.migrate_blocks(migrating)
        resident.append(rid)
        assert len(target) == need == len(migrating.block_indexes)
        assert dec_engine.migration_latency(rid) > 0
        for (p, t), (k, v) in dst_host.items():
            O.migrate_blocks_numpy(src_host, ctx.tensor_parallel_size, ctx.pipeline_parallel_size, migrating.block_indexes,
                                   dec.tensor_parallel_size, t, dec.pipeline_parallel_size, p, target, k, v,
                                   model.num_layers, model.num_kv_heads)
    assert ctx_engine.block_manager.get_num_avail_gpu_blocks() == ctx_blocks      # every source block was recycled
    got = host_copy(dec_engine)
    for key in dst_host:
        assert np.array_equal(got[key][0], dst_host[key][0]) and np.array_equal(got[key][1], dst_host[key][1]), key


def test_opt125m_workload_end_to_end():
    """32 requests, lengths U[64,512], 512-block pools on both sides: total
    demand exceeds a pool, so ids are recycled as the engines recycle them."""
    w = WORKLOADS["c1"]
    lengths = prompt_lengths(w)
    assert len(lengths) == 32 and sum(-(-n // 16) for n in lengths) > 512
    run_and_check(w.model, w.block_size, w.ctx_config(), w.dec_config(), 512, 512, lengths, seed=21)


@pytest.mark.parametrize("name,model", [("c3", KVModelConfig(4, 8, 32)), ("c4", KVModelConfig(8, 8, 32)),
                                        ("c5", KVModelConfig(4, 8, 32))])
def test_resharded_layouts_end_to_end(name, model):
    """The benchmark's tensor/pipeline reshard layouts with a scaled-down model."""
    w = WORKLOADS[name]
    rng = np.random.default_rng(22)
    lengths = [int(x) for x in rng.integers(1, 200, size=24)]
    run_and_check(model, 16, w.ctx_config(), w.dec_config(), 48, 40, lengths, seed=23)


def test_batched_acceptance_equals_one_by_one():
    """Several requests accepted with one launch per decoding worker leave the
    same pools as accepting them one awaited call at a time."""
    capi.reset_registry()
    model = KVModelConfig(8, 8, 32)
    ctx, dec = ParallelConfig(4, 0, 1, 0), ParallelConfig(2, 0, 2, 0)
    ctx_engine, dec_engine = build_stages(model, 16, ctx, dec, 96, 80, seed=25)
    src_host, dst_host = host_copy(ctx_engine), host_copy(dec_engine)
    rng = np.random.default_rng(26)
    batch = []
    for rid in range(7):
        req = Request.of_length(rid, int(rng.integers(1, 150)))
        batch.append(ctx_engine.finish_prefill(req))
        req.append_token()
    targets = dec_engine.migrate_blocks_batched(batch)
    assert [len(t) for t in targets] == [len(m.block_indexes) for m in batch]
    assert ctx_engine.block_manager.get_num_avail_gpu_blocks() == 96
    for m, target in zip(batch, targets):
        for (p, t), (k, v) in dst_host.items():
            O.migrate_blocks_numpy(src_host, 4, 1, m.block_indexes, 2, t, 2, p, target, k, v, 8, 8)
    got = host_copy(dec_engine)
    for key in dst_host:
        assert np.array_equal(got[key][0], dst_host[key][0]) and np.array_equal(got[key][1], dst_host[key][1]), key
    assert dec_engine.migrate_blocks_batched([]) == []


def test_trace_replay_matches_engine_flow():
    """make_trace() (used by the benchmark) yields the ids the engines yield."""
    w = WORKLOADS["c1"]
    trace = make_trace(w)
    assert [t.prompt_len for t in trace] == prompt_lengths(w)
    for item in trace:
        assert len(item.src_blocks) == len(item.dst_blocks) == -(-item.prompt_len // w.block_size)
        assert len(set(item.dst_blocks)) == len(item.dst_blocks)


def _context_process(conn, device, seed):
    """A context-stage worker in its own process: fills its pools from the
    seed, sends the handles, stays alive until told to stop."""
    torch.cuda.set_device(device)
    model, cache = KVModelConfig(4, 4, 32), CacheConfig(8, 64)
    worker = KVWorker(0, "context", model, cache, ParallelConfig(), device=device)
    handles = worker.init_kvcache_and_swap(20, 1)
    g = torch.Generator(device="cpu").manual_seed(seed)
    worker.k_cache.copy_(torch.randn(worker.k_cache.shape, generator=g).half())
    worker.v_cache.copy_(torch.randn(worker.v_cache.shape, generator=g).half())
    torch.cuda.synchronize()
    conn.send(handles)
    conn.recv()


def test_two_processes_share_pools_through_ipc_handles():
    """The decoding worker opens a handle exported by ANOTHER process (on the
    second GPU when there is one, else on the same GPU)."""
    ctxmp = mp.get_context("spawn")
    parent, child = ctxmp.Pipe()
    src_device = 1 if torch.cuda.device_count() > 1 else 0
    proc = ctxmp.Process(target=_context_process, args=(child, src_device, 31), daemon=True)
    proc.start()
    try:
        assert parent.poll(180), "context process did not report its handles"
        k_handle, v_handle = parent.recv()
        assert len(k_handle) == capi.HANDLE_WORDS and k_handle[11] == proc.pid
        capi.reset_registry()
        model, cache = KVModelConfig(4, 4, 32), CacheConfig(8, 64)
        mapped_before = capi.get_counter("mapped_peers")
        for t in range(2):                                  # decoding stage tp=2 pulling from a tp=1 context worker
            dec = KVWorker(t, "decoding", model, cache, ParallelConfig(2, t, 1, 0), device=0)
            dec.init_kvcache_and_swap(16, 1)
            dec.k_cache.zero_()
            dec.v_cache.zero_()
            dec.register_kvcache_mem_handles(ParallelConfig(), [[(k_handle, v_handle)]])
            src, dst = [19, 0, 7], [2, 15, 3]
            dec.migrate_blocks(src, ParallelConfig(), dst)
            g = torch.Generator(device="cpu").manual_seed(31)
            ref_k = torch.randn(20, 4, 4, 8, 32, generator=g).half()
            ref_v = torch.randn(20, 4, 4, 8, 32, generator=g).half()
            assert torch.equal(dec.k_cache[dst].cpu(), ref_k[src][:, :, 2 * t:2 * t + 2])
            assert torch.equal(dec.v_cache[dst].cpu(), ref_v[src][:, :, 2 * t:2 * t + 2])
            untouched = [i for i in range(16) if i not in dst]
            assert not dec.k_cache[untouched].any() and not dec.v_cache[untouched].any()
        assert capi.get_counter("mapped_peers") - mapped_before >= 1      # really went through cudaIpcOpenMemHandle
    finally:
        parent.send("stop")
        proc.join(30)
        if proc.is_alive():
            proc.kill()


def test_scheduler_driven_loop_keeps_every_request_intact():
    """The whole decoding-stage control path over real pools: the scheduler
    accepts requests (batched migration), swaps them out under block pressure
    and back in, requests finish and their blocks are recycled.  At every
    checkpoint each live request's prompt blocks — on the GPU or in the pinned
    host pool — must equal what the context stage held for it."""
    import random

    from distserve_b200.block_manager import BlockLocation
    from distserve_b200.scheduler import DecodingStageFCFSScheduler, DecodingStageSchedConfig

    capi.reset_registry()
    model, block_size = KVModelConfig(4, 4, 32), 16
    pc = ParallelConfig()
    cache = CacheConfig(block_size, 1 << 20)
    ctx_w = KVWorker(0, "context", model, cache, pc)
    dec_w = KVWorker(1, "decoding", model, cache, pc)
    ctx_engine = ContextStageEngine(model, pc, cache, [[ctx_w]])
    dec_engine = DecodingStageEngine(model, pc, cache, [[dec_w]], clear_migrated_blocks_callback=ctx_engine.clear_migrated_blocks)
    handles = ctx_engine.init_kvcache(256, 1)
    dec_engine.init_kvcache(48, 64)
    g = torch.Generator(device="cuda").manual_seed(77)
    for pool in (ctx_w.k_cache, ctx_w.v_cache):
        pool.copy_(torch.randn(pool.shape, device="cuda", generator=g).half())
    dec_w.k_cache.zero_()
    dec_w.v_cache.zero_()
    dec_engine.register_kvcache_mem_handles(pc, handles)
    bm = dec_engine.block_manager
    sched = DecodingStageFCFSScheduler(DecodingStageSchedConfig("fcfs", 8, 64, 0.25), pc, bm, dec_engine.migrate_blocks,
                                       dec_engine.migrate_blocks_batched)
    rng = random.Random(11)
    expected, live, next_id, swaps_seen = {}, {}, 0, 0

    def check_all():
        dec_w.wait_for_all_swap_out()
        dec_w.wait_for_all_swap_in()
        torch.cuda.synchronize()
        for rid, req in live.items():
            if rid not in bm.block_table:
                continue                                     # not accepted yet
            n = -(-req.get_input_len() // block_size)
            ids = bm.get_block_table(rid)[:n]
            want_k, want_v = expected[rid]
            if bm.get_location(rid) == BlockLocation.GPU:
                got_k, got_v = dec_w.k_cache[ids].cpu(), dec_w.v_cache[ids].cpu()
            else:
                got_k, got_v = dec_w.k_swap[ids], dec_w.v_swap[ids]
            assert torch.equal(got_k, want_k) and torch.equal(got_v, want_v), f"request {rid} lost its KV"

    for it in range(160):
        for _ in range(rng.choice([0, 0, 0, 1, 1, 2])):
            n, mt = rng.randint(4, 12 * block_size), rng.randint(2, 40)
            if ctx_engine.block_manager.get_num_avail_gpu_blocks() < -(-n // block_size):
                continue
            req = Request(next_id, [0] * n, max_tokens=mt)
            m = ctx_engine.finish_prefill(req)
            expected[next_id] = (ctx_w.k_cache[m.block_indexes].cpu(), ctx_w.v_cache[m.block_indexes].cpu())
            req.add_generated_token()
            sched.add_request(m)
            live[next_id] = req
            next_id += 1
        before = len(bm.swapping_gpu_blocks_list) + len(bm.swapping_cpu_blocks_list)
        batch = sched.get_next_batch()
        swaps_seen += (len(bm.swapping_gpu_blocks_list) + len(bm.swapping_cpu_blocks_list)) != before
        if len(batch):
            bm.allocate_blocks_batched(batch)
            dec_w.prepare_step(batch.get_request_ids())
            for r in batch.requests:
                r.add_generated_token()
            finished = sched.pop_finished_requests()
            bm.free_blocks_batched(finished)
            dec_w.clear_request_resource_batched(finished)
            for r in finished:
                live.pop(r.request_id)
        sched.post_process_batched()
        if it % 20 == 19:
            check_all()
    check_all()
    assert swaps_seen >= 3 and next_id >= 40
    assert len(sched.waiting_queue) + sched.get_processing_num_requests() + len(sched.swapped_queue) > 0

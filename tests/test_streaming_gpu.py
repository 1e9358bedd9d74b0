"""Layer-wise streaming: a stand-in prefill writes a request's KV group by group
and signals each group over the host channel; the decoding workers pull each
signalled window.  After window k only the layers of windows 0..k may have
changed in the decoding pools, and after the last window the pools must equal
what the oracle's whole-request migration of the finished context pools gives."""
import numpy as np
import pytest
import torch

from distserve_b200 import capi, load_ops, streaming
from distserve_b200.actors import ActorPool
from distserve_b200.config import CacheConfig, KVModelConfig, ParallelConfig
from oracle import kv_oracle as O

pytestmark = pytest.mark.gpu

L, H, D, B = 12, 4, 16, 4
MODEL, CACHE = KVModelConfig(L, H, D), CacheConfig(B, 1 << 20)


def test_layer_groups_cover_every_layer_once():
    for n, g in [(40, 8), (80, 7), (12, 5), (3, 8), (32, 1)]:
        w = streaming.layer_groups(n, g)
        assert w[0][0] == 0 and w[-1][1] == n and all(a[1] == b[0] for a, b in zip(w, w[1:]))
        assert len(w) == min(n, g) and max(b - a for a, b in w) - min(b - a for a, b in w) <= 1


def _expected(ctx_bits, src, dst, dec_before, dec_pc_list):
    tp, t, pp, p = dec_pc_list
    k, v = dec_before[0].copy(), dec_before[1].copy()
    O.migrate_blocks_numpy(ctx_bits, 2, 1, src, tp, t, pp, p, dst, k, v, L, H)
    return k, v


def test_streamed_windows_in_one_process():
    load_ops()
    capi.reset_registry()
    ctx_pc = ParallelConfig(2, 0, 1, 0)
    ctx = [streaming.StreamingWorker(t, "context", MODEL, CACHE, ParallelConfig(2, t, 1, 0), device=0) for t in range(2)]
    table = [[w.init_kvcache_and_swap(40, 1) for w in ctx]]
    dec = [streaming.StreamingWorker(10 + p, "decoding", MODEL, CACHE, ParallelConfig(1, 0, 2, p), device=0) for p in range(2)]
    for i, w in enumerate(ctx + dec):
        if w in dec:
            w.init_kvcache_and_swap(32, 1)
            w.register_kvcache_mem_handles(ctx_pc, table)
        w.fill_pools(50 + i)
    rng = np.random.default_rng(1)
    src = [int(x) for x in rng.permutation(40)[:9]]
    dst = [int(x) for x in rng.permutation(32)[:9]]
    for i, w in enumerate(ctx):
        w.stage_request_kv(src, 70 + i)
    ctx_before = [w.pool_bits() for w in ctx]
    dec_before = [w.pool_bits() for w in dec]
    windows = streaming.layer_groups(L, 5)                 # 12 layers in 5 windows; decoding worker p holds [6p, 6p+6)
    seen = []

    def observe(k):
        """After window k: layers below its end hold their final values, the others what they held before."""
        done = windows[k][1]
        for p, w in enumerate(dec):
            k_now, _ = w.pool_bits()
            lo = 6 * p
            moved = [l - lo for l in range(lo, lo + 6) if l < done]
            kept = [l - lo for l in range(lo, lo + 6) if l >= done]
            assert np.array_equal(k_now[:, kept], dec_before[p][0][:, kept]), f"window {k}: layers beyond it changed"
            untouched_blocks = [b for b in range(32) if b not in dst]
            assert np.array_equal(k_now[untouched_blocks], dec_before[p][0][untouched_blocks])
            seen.append((k, p, len(moved)))

    out = streaming.stream_request(ctx, dec, ctx_pc, src, dst, windows, compute_us_per_group=200.0, observe=observe)
    assert out["windows"] == 5 and out["tail_ms"] >= 0
    # the producer wrote exactly the staged K/V into the request's blocks and nothing else
    ctx_after = {(0, t): w.pool_bits() for t, w in enumerate(ctx)}
    for t, w in enumerate(ctx):
        staged_k, staged_v = w.read_request_kv()
        want_k, want_v = ctx_before[t][0].copy(), ctx_before[t][1].copy()
        want_k[src], want_v[src] = staged_k, staged_v
        assert np.array_equal(ctx_after[(0, t)][0], want_k) and np.array_equal(ctx_after[(0, t)][1], want_v)
    # and the decoding pools equal the oracle's whole-request migration of the finished context pools
    for p, w in enumerate(dec):
        want_k, want_v = _expected(ctx_after, src, dst, dec_before[p], [1, 0, 2, p])
        got_k, got_v = w.pool_bits()
        assert np.array_equal(got_k, want_k) and np.array_equal(got_v, want_v)
    assert [s[0] for s in seen] == [0, 0, 1, 1, 2, 2, 3, 3, 4, 4]
    # the reference's order on the same workers gives the same pools
    for i, w in enumerate(ctx):
        w.stage_request_kv(src, 90 + i)
    streaming.whole_request(ctx, dec, ctx_pc, src, dst, windows, compute_us_per_group=50.0)
    ctx_after = {(0, t): w.pool_bits() for t, w in enumerate(ctx)}
    for p, w in enumerate(dec):
        want_k, want_v = _expected(ctx_after, src, dst, dec_before[p], [1, 0, 2, p])
        got_k, got_v = w.pool_bits()
        assert np.array_equal(got_k, want_k) and np.array_equal(got_v, want_v)
    capi.reset_registry()


def test_streamed_windows_between_worker_processes():
    """Producer and consumer in different processes (on different GPUs when there are two): the per-group signal is
    the return of ``wait_layer_group`` over the actor pipe."""
    n_gpu = torch.cuda.device_count()
    ctx_pc = ParallelConfig(2, 0, 1, 0)
    with ActorPool() as pool:
        ctx = [pool.spawn(streaming.make_streaming_worker, t, "context", MODEL, CACHE, [2, t, 1, 0], 0) for t in range(2)]
        dec = [pool.spawn(streaming.make_streaming_worker, 10, "decoding", MODEL, CACHE, [1, 0, 1, 0], 1 % n_gpu)]
        table = [[w.init_kvcache_and_swap(40, 1).result(300) for w in ctx]]
        dec[0].init_kvcache_and_swap(32, 1).result(300)
        dec[0].register_kvcache_mem_handles(ctx_pc, table).result(300)
        for i, w in enumerate(ctx + dec):
            w.fill_pools(20 + i).result(300)
        rng = np.random.default_rng(2)
        src = [int(x) for x in rng.permutation(40)[:11]]
        dst = [int(x) for x in rng.permutation(32)[:11]]
        for i, w in enumerate(ctx):
            w.stage_request_kv(src, 30 + i).result(300)
        dec_before = dec[0].pool_bits().result(300)
        windows = streaming.layer_groups(L, 4)
        out = streaming.stream_request(ctx, dec, ctx_pc, src, dst, windows, compute_us_per_group=300.0)
        assert out["windows"] == 4
        ctx_after = {(0, t): w.pool_bits().result(300) for t, w in enumerate(ctx)}
        want_k, want_v = _expected(ctx_after, src, dst, dec_before, [1, 0, 1, 0])
        got_k, got_v = dec[0].pool_bits().result(300)
        assert np.array_equal(got_k, want_k) and np.array_equal(got_v, want_v)

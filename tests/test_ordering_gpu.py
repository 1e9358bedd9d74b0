"""Ordering of migrations that the library lets overlap on the GPU.

A migration may begin before earlier ones have finished only when it is
independent of them.  These cases are the dependent ones — a pool that is the
destination of one migration and the source of the next, layer windows that
return to layers an older launch is still writing, and conflicting launches on
two streams — each sized so that the earlier launch is still running when the
later one is enqueued, and each checked bit for bit against the oracle's result
for the same sequence executed in order.
"""
import numpy as np
import pytest
import torch

from distserve_b200 import capi
from oracle import kv_oracle as O
from tests.kvutil import Stage, assert_stage_equals_host, oracle_all, register_all

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def fresh_library_state():
    capi.reset_registry()
    yield
    capi.reset_registry()


def _register_single(stage: Stage, L, H):
    kh, vh = stage.handles()[0][0]
    capi.register_ipc_mem_handle(kh, vh, L, H, [1, 0, 1, 0], [1, 0, 1, 0])


def test_a_pool_that_is_written_and_then_read_is_read_after_the_write():
    """A -> B, then B -> C, both asynchronous on one stream: the second migration reads what the first
    writes, so it must not begin early.  C must end up holding A's blocks."""
    L, H, B, D, nb = 8, 8, 16, 64, 1000                       # 128 KiB per block per pool: 256 MB per hop
    rng = np.random.default_rng(3)
    a = Stage(L, H, 1, 1, nb, B, D, seed=60)
    b = Stage(L, H, 1, 1, nb, B, D, seed=61)
    c = Stage(L, H, 1, 1, nb, B, D, seed=62)
    stream = torch.cuda.Stream()
    for round_ in range(4):
        perm1 = [int(x) for x in rng.permutation(nb)]
        perm2 = [int(x) for x in rng.permutation(nb)]
        ids = list(range(nb))
        _register_single(a, L, H)
        t1 = capi.migrate_blocks_async(1, 1, ids, 1, 1, 0, 0, perm1, b.dev[(0, 0)][0].data_ptr(), b.dev[(0, 0)][1].data_ptr(),
                                       b.shape(), stream.cuda_stream)
        _register_single(b, L, H)                                # B's pools are now the context pools
        t2 = capi.migrate_blocks_async(1, 1, ids, 1, 1, 0, 0, perm2, c.dev[(0, 0)][0].data_ptr(), c.dev[(0, 0)][1].data_ptr(),
                                       c.shape(), stream.cuda_stream)
        capi.migrate_wait(t2)
        capi.migrate_wait(t1)
        # the same two hops, in order, on the host copies
        O.migrate_blocks_numpy(a.host, 1, 1, ids, 1, 0, 1, 0, perm1, *b.host[(0, 0)], L, H)
        O.migrate_blocks_numpy(b.host, 1, 1, ids, 1, 0, 1, 0, perm2, *c.host[(0, 0)], L, H)
        assert_stage_equals_host(b, f"round {round_}, first hop")
        assert_stage_equals_host(c, f"round {round_}, second hop")
        # new contents for the next round, so that a stale read cannot pass by coincidence
        for x in range(2):
            a.dev[(0, 0)][x].random_(-30000, 30000)
            a.host[(0, 0)][x][...] = a.dev[(0, 0)][x].cpu().numpy()


def test_a_pool_that_is_read_and_then_overwritten_is_overwritten_after_the_read():
    """A -> B, then C -> A: the second migration overwrites blocks the first is still reading."""
    L, H, B, D, nb = 8, 8, 16, 64, 1000
    rng = np.random.default_rng(4)
    a = Stage(L, H, 1, 1, nb, B, D, seed=63)
    b = Stage(L, H, 1, 1, nb, B, D, seed=64)
    c = Stage(L, H, 1, 1, nb, B, D, seed=65)
    stream = torch.cuda.Stream()
    ids = list(range(nb))
    perm = [int(x) for x in rng.permutation(nb)]
    _register_single(a, L, H)
    t1 = capi.migrate_blocks_async(1, 1, ids, 1, 1, 0, 0, perm, b.dev[(0, 0)][0].data_ptr(), b.dev[(0, 0)][1].data_ptr(),
                                   b.shape(), stream.cuda_stream)
    _register_single(c, L, H)
    t2 = capi.migrate_blocks_async(1, 1, ids, 1, 1, 0, 0, ids, a.dev[(0, 0)][0].data_ptr(), a.dev[(0, 0)][1].data_ptr(),
                                   a.shape(), stream.cuda_stream)
    capi.migrate_wait(t1)
    capi.migrate_wait(t2)
    O.migrate_blocks_numpy(a.host, 1, 1, ids, 1, 0, 1, 0, perm, *b.host[(0, 0)], L, H)
    O.migrate_blocks_numpy(c.host, 1, 1, ids, 1, 0, 1, 0, ids, *a.host[(0, 0)], L, H)
    assert_stage_equals_host(b, "the copy out of A")
    assert_stage_equals_host(a, "the copy into A")


def _pull_window(cs, ds, src, dst, window, stream):
    k, v = ds.dev[(0, 0)]
    return capi.migrate_layers_async(1, 1, src, 1, 1, 0, 0, dst, k.data_ptr(), v.data_ptr(), ds.shape(), window[0], window[1],
                                     stream.cuda_stream)


def _oracle_window(cs, ds, src, dst, window):
    """The oracle's full migration, restricted to the window's layers on the host copy."""
    k, v = ds.host[(0, 0)]
    fk, fv = k.copy(), v.copy()
    O.migrate_blocks_numpy(cs.host, 1, 1, src, 1, 0, 1, 0, dst, fk, fv, cs.L, cs.H)
    k[:, window[0]:window[1]] = fk[:, window[0]:window[1]]
    v[:, window[0]:window[1]] = fv[:, window[0]:window[1]]


def test_a_window_that_returns_to_layers_an_older_launch_still_writes_waits_for_it():
    """Layers [0,4) from one set of sources, then layers [4,8), then layers [0,4) of the SAME target blocks from
    other sources.  The third launch's blocks were last written by the second (other layers), but it must
    still come after the first."""
    L, H, B, D, nb = 8, 8, 16, 64, 900
    rng = np.random.default_rng(5)
    cs = Stage(L, H, 1, 1, 2 * nb, B, D, seed=66)
    ds = Stage(L, H, 1, 1, nb, B, D, seed=67)
    register_all(cs, ds)
    stream = torch.cuda.Stream()
    dst = [int(x) for x in rng.permutation(nb)]
    for round_ in range(3):
        src1 = [int(x) for x in rng.integers(0, 2 * nb, size=nb)]
        src2 = [int(x) for x in rng.integers(0, 2 * nb, size=nb)]
        tickets = [_pull_window(cs, ds, src1, dst, (0, 4), stream),
                   _pull_window(cs, ds, src1, dst, (4, 8), stream),
                   _pull_window(cs, ds, src2, dst, (0, 4), stream)]
        for t in tickets:
            capi.migrate_wait(t)
        _oracle_window(cs, ds, src1, dst, (0, 4))
        _oracle_window(cs, ds, src1, dst, (4, 8))
        _oracle_window(cs, ds, src2, dst, (0, 4))
        assert_stage_equals_host(ds, f"round {round_}")


def test_conflicting_launches_on_two_streams_run_in_the_order_they_were_enqueued():
    """The same target blocks written from two streams: the launch enqueued second must land second."""
    L, H, B, D, nb = 8, 8, 16, 64, 1000
    rng = np.random.default_rng(6)
    cs = Stage(L, H, 1, 1, 2 * nb, B, D, seed=68)
    ds = Stage(L, H, 1, 1, nb, B, D, seed=69)
    register_all(cs, ds)
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    k, v = ds.dev[(0, 0)]
    dst = [int(x) for x in rng.permutation(nb)]
    for round_ in range(3):
        src1 = [int(x) for x in rng.integers(0, 2 * nb, size=nb)]
        src2 = [int(x) for x in rng.integers(0, 2 * nb, size=nb)]
        t1 = capi.migrate_blocks_async(1, 1, src1, 1, 1, 0, 0, dst, k.data_ptr(), v.data_ptr(), ds.shape(), s1.cuda_stream)
        t2 = capi.migrate_blocks_async(1, 1, src2, 1, 1, 0, 0, dst, k.data_ptr(), v.data_ptr(), ds.shape(), s2.cuda_stream)
        capi.migrate_wait(t1)
        capi.migrate_wait(t2)
        oracle_all(cs, ds, src1, dst)
        oracle_all(cs, ds, src2, dst)
        assert_stage_equals_host(ds, f"round {round_}")


def test_independent_launches_still_overlap_and_planning_is_reused():
    """Requests with disjoint targets keep their early start, and consecutive calls with the same layouts reuse the
    planning of the first (visible in the library's counters)."""
    L, H, B, D, nb = 4, 4, 8, 32, 256
    rng = np.random.default_rng(7)
    cs = Stage(L, H, 1, 1, nb, B, D, seed=70)
    ds = Stage(L, H, 1, 1, nb, B, D, seed=71)
    register_all(cs, ds)
    k, v = ds.dev[(0, 0)]
    perm = [int(x) for x in rng.permutation(nb)]
    hits0, calls0 = capi.get_counter("plan_cache_hits"), capi.get_counter("migrate_calls")
    tickets = []
    for i in range(8):
        src = [int(x) for x in rng.integers(0, nb, size=32)]
        dst = perm[32 * i:32 * (i + 1)]
        tickets.append(capi.migrate_blocks_async(1, 1, src, 1, 1, 0, 0, dst, k.data_ptr(), v.data_ptr(), ds.shape()))
        oracle_all(cs, ds, src, dst)
    for t in tickets:
        capi.migrate_wait(t)
    assert_stage_equals_host(ds)
    assert capi.get_counter("migrate_calls") - calls0 == 8
    assert capi.get_counter("plan_cache_hits") - hits0 == 7
    # a changed option invalidates the planning
    saved = capi.get_option("chunk_bytes")
    try:
        capi.set_option("chunk_bytes", 8192)
        hits1 = capi.get_counter("plan_cache_hits")
        capi.migrate_blocks(1, 1, [0], 1, 1, 0, 0, [1], k.data_ptr(), v.data_ptr(), ds.shape())
        assert capi.get_counter("plan_cache_hits") == hits1
    finally:
        capi.set_option("chunk_bytes", saved)
    oracle_all(cs, ds, [0], [1])
    assert_stage_equals_host(ds)
    for name in ("ns_prepare", "ns_validate", "ns_order", "ns_launch", "ns_wait"):
        assert capi.get_counter(name) > 0, name

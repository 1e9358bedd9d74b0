"""Parity of the CUDA migration path with the oracle, bit for bit, through the
C ABI: every stage layout, both kernels, odd shapes, ragged and empty lists,
refusals, and size-independent properties at full block size."""
import numpy as np
import pytest
import torch

from distserve_b200 import capi
from tests.kvutil import Stage, assert_stage_equals_host, migrate_all, oracle_all, register_all

pytestmark = pytest.mark.gpu

LAYOUTS = [
    # L, H, (ctx_tp, ctx_pp), (dec_tp, dec_pp)
    (4, 4, (1, 1), (1, 1)),
    (4, 4, (2, 1), (1, 1)),      # gather heads from two sources
    (4, 4, (1, 1), (2, 1)),      # take a sub-range of one source's heads
    (8, 8, (4, 1), (2, 2)),      # the 8-GPU reshard layout, scaled down
    (6, 4, (1, 3), (2, 1)),      # gather layers from three sources
    (6, 4, (2, 2), (4, 3)),
    (8, 8, (8, 1), (1, 4)),
    (12, 6, (3, 3), (2, 4)),
]


@pytest.fixture(autouse=True)
def fresh_library_state():
    capi.reset_registry()
    saved = {k: capi.get_option(k) for k in ("kernel", "chunk_bytes", "stages", "ctas_per_sm", "inline_tables",
                                             "overlap_launches")}
    yield
    for k, v in saved.items():
        capi.set_option(k, v)
    capi.reset_registry()


def ragged_lists(rng, n_src, n_dst, n):
    src = [int(x) for x in rng.integers(0, n_src, size=n)]          # sources may repeat
    dst = [int(x) for x in rng.permutation(n_dst)[:n]]               # targets are distinct
    return src, dst


@pytest.mark.parametrize("kernel,inline", [(1, 0), (2, 1), (2, 0)], ids=["vec", "bulk-inline-tables", "bulk-device-tables"])
@pytest.mark.parametrize("L,H,ctx,dec", LAYOUTS)
def test_layouts_match_oracle(L, H, ctx, dec, kernel, inline):
    capi.set_option("kernel", kernel)
    capi.set_option("inline_tables", inline)
    rng = np.random.default_rng(L * 31 + H)
    B, D = 4, 16
    cs = Stage(L, H, ctx[0], ctx[1], 37, B, D, seed=1)
    ds = Stage(L, H, dec[0], dec[1], 29, B, D, seed=2)
    register_all(cs, ds)
    for n in (1, 5, 29):
        src, dst = ragged_lists(rng, 37, 29, n)
        migrate_all(cs, ds, src, dst)
        oracle_all(cs, ds, src, dst)
        assert_stage_equals_host(ds, f"n={n}")
    # the sources are never written
    for key, (hk, hv) in cs.host.items():
        assert np.array_equal(cs.dev[key][0].cpu().numpy(), hk) and np.array_equal(cs.dev[key][1].cpu().numpy(), hv)


@pytest.mark.parametrize("kernel,chunk,stages", [(1, 16, 4), (1, 4096, 4), (2, 16, 2), (2, 48, 3), (2, 1024, 16),
                                                (2, 32768, 4), (1, 1 << 20, 4), (2, 16384, 6)])
def test_chunking_does_not_change_the_result(kernel, chunk, stages):
    capi.set_option("kernel", kernel)
    capi.set_option("chunk_bytes", chunk)
    capi.set_option("stages", stages)
    rng = np.random.default_rng(chunk + stages)
    cs = Stage(4, 6, 2, 1, 40, 16, 40, seed=3)       # slab = 16*40*2 = 1280 B: runs are not chunk multiples
    ds = Stage(4, 6, 3, 2, 33, 16, 40, seed=4)
    register_all(cs, ds)
    src, dst = ragged_lists(rng, 40, 33, 33)
    migrate_all(cs, ds, src, dst)
    oracle_all(cs, ds, src, dst)
    assert_stage_equals_host(ds)


@pytest.mark.parametrize("B,D,elem", [(1, 4, 2), (3, 1, 2), (1, 1, 2), (16, 80, 2), (16, 64, 4), (5, 3, 4),
                                      (16, 128, 1), (7, 5, 1), (3, 1, 1), (4, 16, 8)])   # 1-byte (fp8-sized) and 8-byte values too
def test_odd_shapes_fall_back_to_narrower_vectors(B, D, elem):
    """Slabs that are not multiples of 16 bytes cannot use the bulk kernel;
    automatic selection must still be bit-exact."""
    rng = np.random.default_rng(B * 100 + D)
    cs = Stage(4, 4, 2, 2, 11, B, D, elem_size=elem, seed=5)
    src, dst = ragged_lists(rng, 11, 13, 9)
    for dec_tp, dec_pp in ((1, 1), (4, 1)):               # whole blocks, then single-head runs
        capi.reset_registry()
        ds = Stage(4, 4, dec_tp, dec_pp, 13, B, D, elem_size=elem, seed=6)
        register_all(cs, ds)
        migrate_all(cs, ds, src, dst)
        oracle_all(cs, ds, src, dst)
        assert_stage_equals_host(ds)
    if (B * D * elem) % 16:                               # ds now copies one head (= one slab) per run
        capi.set_option("kernel", 2)
        with pytest.raises(capi.KvmigError, match="16-byte"):
            migrate_all(cs, ds, src, dst)


def test_empty_lists_are_a_no_op():
    cs = Stage(2, 2, 1, 1, 4, 2, 8, seed=7)
    ds = Stage(2, 2, 1, 1, 4, 2, 8, seed=8)
    register_all(cs, ds)
    launches = capi.get_counter("kernel_launches")
    migrate_all(cs, ds, [], [])
    assert capi.get_counter("kernel_launches") == launches
    assert_stage_equals_host(ds)


def test_refusals_leave_the_pools_untouched():
    cs = Stage(4, 4, 2, 1, 6, 2, 8, seed=9)
    ds = Stage(4, 4, 1, 1, 5, 2, 8, seed=10)
    k, v = ds.dev[(0, 0)]
    args = lambda src, dst: (1, 2, src, 1, 1, 0, 0, dst, k.data_ptr(), v.data_ptr(), ds.shape())
    with pytest.raises(capi.KvmigError) as e:           # nothing registered yet
        capi.migrate_blocks(*args([0], [0]))
    assert e.value.code == capi.ENOTREG
    register_all(cs, ds)
    launches = capi.get_counter("kernel_launches")
    for src, dst, text in [([0, 1], [0], "entries"), ([6], [0], "outside the context pool"), ([-1], [0], "outside"),
                           ([0], [5], "outside the decoding pool"), ([0, 1], [2, 2], "twice")]:
        with pytest.raises(capi.KvmigError, match=text) as e:
            capi.migrate_blocks(*args(src, dst))
        assert e.value.code == capi.EINVAL
    with pytest.raises(capi.KvmigError, match="not divisible"):
        capi.migrate_blocks(1, 3, [0], 1, 1, 0, 0, [0], k.data_ptr(), v.data_ptr(), ds.shape())
    wrong = capi.PoolShape.of(5, 4, 4, 2, 16, 2)       # head_dim differs from the context pools'
    with pytest.raises(capi.KvmigError, match="geometry"):
        capi.migrate_blocks(1, 2, [0], 1, 1, 0, 0, [0], k.data_ptr(), v.data_ptr(), wrong)
    assert capi.get_counter("kernel_launches") == launches
    assert_stage_equals_host(ds, "after refusals")
    migrate_all(cs, ds, [5, 0], [1, 4])                  # and the library still works
    oracle_all(cs, ds, [5, 0], [1, 4])
    assert_stage_equals_host(ds, "after a valid call")


def test_corrupted_or_mismatched_handles_are_refused():
    cs = Stage(4, 4, 2, 1, 6, 2, 8, seed=11)
    handles = cs.handles()
    kh, vh = handles[0][0]
    broken = list(kh)
    broken[9] ^= 0x10                                     # flip a bit of the offset word
    with pytest.raises(capi.KvmigError, match="checksum"):
        capi.register_ipc_mem_handle(broken, vh, 4, 4, [2, 0, 1, 0], [1, 0, 1, 0])
    with pytest.raises(capi.KvmigError, match="holds"):  # a tp=2 shard registered as tp=1
        capi.register_ipc_mem_handle(kh, vh, 4, 4, [1, 0, 1, 0], [1, 0, 1, 0])
    with pytest.raises(capi.KvmigError, match="tp_size"):
        capi.register_ipc_mem_handle(kh, vh, 4, 4, [2, 2, 1, 0], [1, 0, 1, 0])
    sub = cs.dev[(0, 0)][0][1:]                           # a view that starts inside the allocation
    h = capi.get_ipc_mem_handle(sub.data_ptr(), capi.PoolShape.of(5, 4, 2, 2, 8, 2))
    assert h[9] >= sub.data_ptr() - cs.dev[(0, 0)][0].data_ptr()


def test_many_blocks_in_one_call_and_table_growth():
    rng = np.random.default_rng(12)
    cs = Stage(2, 2, 1, 1, 6000, 2, 8, seed=12)
    ds = Stage(2, 2, 2, 1, 5000, 2, 8, seed=13)
    register_all(cs, ds)
    for n in (3, 256, 257, 1024, 1025, 2500, 5000):     # both inline-table sizes, then device tables
        src, dst = ragged_lists(rng, 6000, 5000, n)
        migrate_all(cs, ds, src, dst)
        oracle_all(cs, ds, src, dst)
    assert_stage_equals_host(ds)


def test_async_tickets():
    rng = np.random.default_rng(14)
    cs = Stage(4, 4, 1, 1, 64, 4, 16, seed=14)
    ds = Stage(4, 4, 1, 1, 64, 4, 16, seed=15)
    register_all(cs, ds)
    k, v = ds.dev[(0, 0)]
    side = torch.cuda.Stream()
    perm = [int(x) for x in rng.permutation(64)]
    tickets = []
    for i in range(12):                                   # more than KVMIG_MAX_INFLIGHT: old ones retire implicitly
        src, dst = perm[i * 5:(i + 1) * 5], perm[i * 5:(i + 1) * 5][::-1]
        tickets.append(capi.migrate_blocks_async(1, 1, src, 1, 1, 0, 0, dst, k.data_ptr(), v.data_ptr(), ds.shape(),
                                                 side.cuda_stream))
        oracle_all(cs, ds, src, dst)
    for t in tickets:
        capi.migrate_wait(t)
    capi.migrate_wait(tickets[0])                         # waiting twice is harmless
    with pytest.raises(capi.KvmigError, match="unknown ticket"):
        capi.migrate_wait(tickets[-1] + 1000)
    assert_stage_equals_host(ds)


@pytest.mark.parametrize("overlap", [1, 0])
def test_launches_that_share_target_blocks_keep_stream_order(overlap):
    """Back-to-back launches may overlap on the GPU only when their target
    blocks are disjoint.  Here every launch rewrites the same targets from
    different sources (large enough that launches would still be running when
    the next one is enqueued); the pools must end up as if run one by one."""
    capi.set_option("overlap_launches", overlap)
    rng = np.random.default_rng(18)
    cs = Stage(8, 8, 1, 1, 256, 16, 64, seed=18)         # 256 KiB per block per pool
    ds = Stage(8, 8, 1, 1, 64, 16, 64, seed=19)
    register_all(cs, ds)
    k, v = ds.dev[(0, 0)]
    stream = torch.cuda.Stream()
    tickets = []
    targets = list(range(40))
    for i in range(7):
        src = [int(x) for x in rng.integers(0, 256, size=40)]
        dst = targets if i % 2 == 0 else targets[::-1]
        tickets.append(capi.migrate_blocks_async(1, 1, src, 1, 1, 0, 0, dst, k.data_ptr(), v.data_ptr(), ds.shape(),
                                                 stream.cuda_stream))
        oracle_all(cs, ds, src, dst)
    # independent launches in between and after: disjoint targets
    for i in range(3):
        src = [int(x) for x in rng.integers(0, 256, size=8)]
        dst = list(range(40 + 8 * i, 48 + 8 * i))
        tickets.append(capi.migrate_blocks_async(1, 1, src, 1, 1, 0, 0, dst, k.data_ptr(), v.data_ptr(), ds.shape(),
                                                 stream.cuda_stream))
        oracle_all(cs, ds, src, dst)
    for t in tickets:
        capi.migrate_wait(t)
    assert_stage_equals_host(ds)


def test_full_size_blocks_round_trip():
    """OPT-13B block geometry (6.25 MiB per block per pool): A -> B by one
    permutation, B -> C by its inverse; C must equal A block for block, and
    the byte counter must match the algorithmic bytes."""
    L, H, B, D, nb = 40, 40, 16, 128, 96
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(16)
    shape = (nb, L, H, B, D)
    pools = {name: [torch.randint(-2**15, 2**15, shape, dtype=torch.int16, device=dev, generator=g) for _ in range(2)]
             for name in "ABC"}
    ps = capi.PoolShape.of(*shape, 2)
    rng = np.random.default_rng(16)
    perm = [int(x) for x in rng.permutation(nb)]
    inv = [perm.index(i) for i in range(nb)]
    before = capi.get_counter("bytes_migrated")
    for kernel in (1, 2):
        capi.set_option("kernel", kernel)
        for src_name, dst_name, src_ids, dst_ids in (("A", "B", list(range(nb)), perm), ("B", "C", perm, list(range(nb)))):
            capi.reset_registry()
            kh, vh = (capi.get_ipc_mem_handle(t.data_ptr(), ps) for t in pools[src_name])
            capi.register_ipc_mem_handle(kh, vh, L, H, [1, 0, 1, 0], [1, 0, 1, 0])
            capi.migrate_blocks(1, 1, src_ids, 1, 1, 0, 0, dst_ids, pools[dst_name][0].data_ptr(),
                                pools[dst_name][1].data_ptr(), ps)
        for x in range(2):
            assert torch.equal(pools["C"][x], pools["A"][x])
            assert torch.equal(pools["B"][x][perm], pools["A"][x])
            pools["C"][x].zero_()
    assert inv is not None
    assert capi.get_counter("bytes_migrated") - before == 4 * nb * 2 * ps.block_bytes


def test_layer_windows_compose_to_the_full_migration():
    """Pulling a request layer group by layer group (out of order, on two
    streams) must leave exactly what one full migration leaves; after the
    first group only that group's layers may have changed."""
    rng = np.random.default_rng(20)
    L, H = 12, 4
    cs = Stage(L, H, 2, 3, 30, 4, 16, seed=20)            # context tp=2, pp=3
    ds = Stage(L, H, 1, 2, 26, 4, 16, seed=21)            # decoding tp=1, pp=2: worker p holds layers [6p, 6p+6)
    register_all(cs, ds)
    src, dst = ragged_lists(rng, 30, 26, 11)
    before = {key: (k.clone(), v.clone()) for key, (k, v) in ds.dev.items()}
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    windows = [(4, 9), (0, 4), (9, 12)]                    # the first one straddles both decoding workers
    tickets = []

    def pull(window, stream):
        for dp in range(2):
            k, v = ds.dev[(dp, 0)]
            tickets.append(capi.migrate_layers_async(3, 2, src, 2, 1, dp, 0, dst, k.data_ptr(), v.data_ptr(), ds.shape((dp, 0)),
                                                     window[0], window[1], stream.cuda_stream))

    pull(windows[0], streams[0])
    for t in tickets:
        capi.migrate_wait(t)
    oracle_all(cs, ds, src, dst)                           # host copies now hold the full result
    for dp in range(2):
        k, v = ds.dev[(dp, 0)]
        lo, hi = max(4, 6 * dp) - 6 * dp, min(9, 6 * dp + 6) - 6 * dp
        inside = list(range(lo, hi))
        outside = [l for l in range(6) if l not in inside]
        full_k = torch.from_numpy(ds.host[(dp, 0)][0]).cuda()
        assert torch.equal(k[:, inside], full_k[:, inside])
        assert torch.equal(k[:, outside], before[(dp, 0)][0][:, outside])
    pull(windows[1], streams[1])
    pull(windows[2], streams[0])
    for t in tickets:
        capi.migrate_wait(t)
    assert_stage_equals_host(ds)
    # a window that misses the worker launches nothing; a malformed one is refused
    k, v = ds.dev[(0, 0)]
    launches = capi.get_counter("kernel_launches")
    t = capi.migrate_layers_async(3, 2, src, 2, 1, 0, 0, dst, k.data_ptr(), v.data_ptr(), ds.shape((0, 0)), 6, 12, 0)
    capi.migrate_wait(t)
    assert capi.get_counter("kernel_launches") == launches
    with pytest.raises(capi.KvmigError, match="not a range"):
        capi.migrate_layers_async(3, 2, src, 2, 1, 0, 0, dst, k.data_ptr(), v.data_ptr(), ds.shape((0, 0)), 5, 2, 0)


def test_concurrent_host_threads():
    """Two host threads, each with its own decoding pools and stream, enqueue
    and await migrations at the same time (ctypes drops the GIL inside the
    library); both must end bit-exact."""
    import threading

    cs = Stage(4, 4, 1, 1, 128, 8, 32, seed=30)
    pools = [Stage(4, 4, 1, 1, 96, 8, 32, seed=31 + i) for i in range(2)]
    register_all(cs, pools[0])
    plans = []
    for i, ds in enumerate(pools):
        rng = np.random.default_rng(40 + i)
        plan = [ragged_lists(rng, 128, 96, int(rng.integers(1, 40))) for _ in range(60)]
        for src, dst in plan:
            oracle_all(cs, ds, src, dst)
        plans.append(plan)
    errors = []

    def worker(i):
        try:
            torch.cuda.set_device(0)
            ds, stream = pools[i], torch.cuda.Stream()
            k, v = ds.dev[(0, 0)]
            for j, (src, dst) in enumerate(plans[i]):
                if j % 3 == 0:
                    capi.migrate_blocks(1, 1, src, 1, 1, 0, 0, dst, k.data_ptr(), v.data_ptr(), ds.shape(), stream.cuda_stream)
                else:
                    t = capi.migrate_blocks_async(1, 1, src, 1, 1, 0, 0, dst, k.data_ptr(), v.data_ptr(), ds.shape(),
                                                  stream.cuda_stream)
                    capi.migrate_wait(t)
        except Exception as e:   # surfaced below
            errors.append(e)

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(120)
    assert not errors, errors
    torch.cuda.synchronize()
    for ds in pools:
        assert_stage_equals_host(ds)


def test_a_load_that_never_completes_is_reported_not_hung():
    """Failure-path exercise without any fault: one work unit arms its
    completion barrier but never issues its load.  The kernel's bounded wait
    must run out, the call must fail with KVMIG_EDEVICE, and the library and
    the CUDA context must stay usable."""
    cs = Stage(4, 4, 1, 1, 16, 16, 64, seed=50)
    ds = Stage(4, 4, 1, 1, 16, 16, 64, seed=51)
    register_all(cs, ds)
    src, dst = [3, 9, 1], [0, 5, 7]
    saved = {k: capi.get_option(k) for k in ("wait_limit_ms", "lose_unit_plus1")}
    try:
        capi.set_option("wait_limit_ms", 30)
        for entry in ("awaited", "ticket"):
            capi.set_option("lose_unit_plus1", 2)
            k, v = ds.dev[(0, 0)]
            with pytest.raises(capi.KvmigError, match="gave up") as e:
                if entry == "awaited":
                    capi.migrate_blocks(1, 1, src, 1, 1, 0, 0, dst, k.data_ptr(), v.data_ptr(), ds.shape())
                else:
                    capi.migrate_wait(capi.migrate_blocks_async(1, 1, src, 1, 1, 0, 0, dst, k.data_ptr(), v.data_ptr(),
                                                                ds.shape()))
            assert e.value.code == capi.EDEVICE
            assert "at work unit 1," in str(e.value)      # the launch-wide number of the unit that was lost
            capi.set_option("lose_unit_plus1", 0)
            torch.cuda.synchronize()                      # the context is alive
            migrate_all(cs, ds, src, dst)                 # and the same call now succeeds
    finally:
        for name, value in saved.items():
            capi.set_option(name, value)
    oracle_all(cs, ds, src, dst)
    assert_stage_equals_host(ds)


@pytest.mark.parametrize("L,ctx,dec", [(4, (2, 1), (1, 1)), (4, (1, 1), (2, 1)), (4, (2, 2), (2, 1)), (6, (4, 1), (2, 3)),
                                       (6, (2, 3), (4, 1))])
def test_single_kv_head_models_migrate_from_the_matching_replica(L, ctx, dec):
    """Multi-query attention: every tensor-parallel rank of both stages holds the model's one KV head
    (distserve/config.py:233-237).  The pools' replicas are given different contents, so the comparison with the
    oracle also pins WHICH replica a decoding rank reads."""
    rng = np.random.default_rng(L + 17)
    cs = Stage(L, 1, ctx[0], ctx[1], 23, 4, 16, seed=80)
    ds = Stage(L, 1, dec[0], dec[1], 19, 4, 16, seed=81)
    assert cs.dev[(0, 0)][0].shape[2] == 1 and ds.dev[(0, 0)][0].shape[2] == 1
    register_all(cs, ds)
    for n in (1, 7, 19):
        src, dst = ragged_lists(rng, 23, 19, n)
        migrate_all(cs, ds, src, dst)
        oracle_all(cs, ds, src, dst)
        assert_stage_equals_host(ds, f"n={n}")

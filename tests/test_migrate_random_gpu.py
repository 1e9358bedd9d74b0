"""Seeded random sweep of stage layouts, block shapes, list lengths, kernel
options, layer windows and call styles against the oracle; plus the layouts
with more contributing context workers than one launch can describe."""
import numpy as np
import pytest
import torch

from distserve_b200 import capi
from oracle import kv_oracle_c as OC
from tests.kvutil import Stage, assert_stage_equals_host, migrate_all, oracle_all, register_all

pytestmark = pytest.mark.gpu

OPTIONS = ("kernel", "chunk_bytes", "stages", "ctas_per_sm", "inline_tables", "overlap_launches", "dynamic_units", "max_ctas")


@pytest.fixture(autouse=True)
def restore_options():
    capi.reset_registry()
    saved = {k: capi.get_option(k) for k in OPTIONS}
    yield
    for k, v in saved.items():
        capi.set_option(k, v)
    capi.reset_registry()


def divisors(n):
    return [d for d in range(1, n + 1) if n % d == 0]


@pytest.mark.parametrize("ctx,dec,L,H", [((4, 4), (1, 1), 16, 16), ((16, 1), (1, 1), 4, 16), ((2, 8), (1, 2), 16, 4)])
def test_more_sources_than_one_launch_describes(ctx, dec, L, H):
    """16 or more contributing context workers give more than 16 segments:
    the call is split into several launches that share one ticket."""
    rng = np.random.default_rng(L + H)
    cs = Stage(L, H, ctx[0], ctx[1], 21, 4, 16, seed=60)
    ds = Stage(L, H, dec[0], dec[1], 19, 4, 16, seed=61)
    register_all(cs, ds)
    for inline in (1, 0):
        capi.set_option("inline_tables", inline)
        src = [int(x) for x in rng.integers(0, 21, size=13)]
        dst = [int(x) for x in rng.permutation(19)[:13]]
        before = capi.get_counter("kernel_launches")
        migrate_all(cs, ds, src, dst)
        launches = capi.get_counter("kernel_launches") - before
        oracle_all(cs, ds, src, dst, fn=OC.migrate_blocks_c)
        assert_stage_equals_host(ds)
        if dec == (1, 1):
            assert launches == 2          # 16 sources x (K, V) = 32 segments = 2 launches
    if dec == (1, 1):
        k, v = ds.dev[(0, 0)]
        with pytest.raises(capi.KvmigError, match="segments") as e:
            capi.migrate_blocks_static(ctx[1], ctx[0], [0], 1, 1, 0, 0, [0], k.data_ptr(), v.data_ptr(), ds.shape())
        assert e.value.code == capi.ELIMIT


@pytest.mark.parametrize("seed", [2024, 7, 99])
def test_random_cases_match_oracle(seed):
    rng = np.random.default_rng(seed)
    for case in range(60):
        L = int(rng.choice([2, 4, 6, 8, 12]))
        H = int(rng.choice([1, 2, 4, 6, 8]))
        ctx_pp, dec_pp = (int(rng.choice(divisors(L))) for _ in range(2))
        ctx_tp, dec_tp = (int(rng.choice(divisors(H))) for _ in range(2))
        B = int(rng.choice([1, 2, 4, 16]))
        D = int(rng.choice([1, 3, 8, 16, 40, 64]))
        elem = int(rng.choice([2, 4]))
        n_src, n_dst = int(rng.integers(1, 40)), int(rng.integers(1, 40))
        cs = Stage(L, H, ctx_tp, ctx_pp, n_src, B, D, elem_size=elem, seed=[seed, case, 1])
        ds = Stage(L, H, dec_tp, dec_pp, n_dst, B, D, elem_size=elem, seed=[seed, case, 2])
        capi.reset_registry()
        register_all(cs, ds)
        slab = B * D * elem
        capi.set_option("kernel", int(rng.choice([0, 0, 1])) if slab % 16 == 0 else 0)
        chunk = int(rng.choice([16, 64, 1024, 8192, 65536]))
        capi.set_option("chunk_bytes", chunk)
        capi.set_option("stages", max(2, min(int(rng.choice([2, 3, 5, 8])), (200 * 1024) // chunk)))   # ring must fit shared memory
        capi.set_option("ctas_per_sm", int(rng.choice([0, 1, 4])))
        capi.set_option("max_ctas", int(rng.choice([0, 0, 3, 40])))
        for name in ("inline_tables", "overlap_launches", "dynamic_units"):
            capi.set_option(name, int(rng.integers(0, 2)))
        stream = torch.cuda.Stream()
        tickets = []
        for call in range(int(rng.integers(1, 5))):
            n = int(rng.integers(0, n_dst + 1))
            src = [int(x) for x in rng.integers(0, n_src, size=n)]
            dst = [int(x) for x in rng.permutation(n_dst)[:n]]
            style = int(rng.integers(0, 3))
            if style == 0:
                migrate_all(cs, ds, src, dst, stream=stream.cuda_stream)
                oracle_all(cs, ds, src, dst)
            elif style == 1:
                for dp in range(dec_pp):
                    for dt in range(dec_tp):
                        k, v = ds.dev[(dp, dt)]
                        tickets.append(capi.migrate_blocks_async(ctx_pp, ctx_tp, src, dec_pp, dec_tp, dp, dt, dst, k.data_ptr(),
                                                                 v.data_ptr(), ds.shape((dp, dt)), stream.cuda_stream))
                oracle_all(cs, ds, src, dst, fn=OC.migrate_blocks_c)
            else:
                cut = int(rng.integers(0, L + 1))          # two layer windows that together cover every layer
                for lo, hi in ((cut, L), (0, cut)):
                    for dp in range(dec_pp):
                        for dt in range(dec_tp):
                            k, v = ds.dev[(dp, dt)]
                            tickets.append(capi.migrate_layers_async(ctx_pp, ctx_tp, src, dec_pp, dec_tp, dp, dt, dst,
                                                                     k.data_ptr(), v.data_ptr(), ds.shape((dp, dt)), lo, hi,
                                                                     stream.cuda_stream))
                oracle_all(cs, ds, src, dst)
        for t in tickets:
            capi.migrate_wait(t)
        torch.cuda.synchronize()
        assert_stage_equals_host(ds, f"seed {seed} case {case}: L={L} H={H} ctx=({ctx_tp},{ctx_pp}) dec=({dec_tp},{dec_pp}) "
                                     f"B={B} D={D} elem={elem}")

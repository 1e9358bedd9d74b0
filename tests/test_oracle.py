"""The oracle's three statements of migrate_blocks agree with each other, and
the decoding workers' rectangles tile the (layer, head) plane exactly once."""
import itertools

import numpy as np
import pytest
import torch

from oracle import kv_oracle as O
from oracle import kv_oracle_c as OC

LAYOUTS = [
    # L, H, (ctx_tp, ctx_pp), (dec_tp, dec_pp)
    (4, 4, (1, 1), (1, 1)),
    (4, 4, (2, 1), (1, 1)),
    (4, 4, (1, 1), (2, 1)),
    (4, 8, (4, 1), (2, 2)),
    (6, 4, (1, 3), (2, 1)),
    (6, 4, (2, 2), (4, 3)),
    (8, 8, (8, 1), (1, 4)),
    (12, 6, (3, 3), (2, 4)),
]


def make_pools(rng, n_blocks, L, H, tp, pp, B, D):
    pools = {}
    for p in range(pp):
        for t in range(tp):
            shape = (n_blocks, L // pp, H // tp, B, D)
            pools[(p, t)] = (rng.integers(-2**15, 2**15, size=shape, dtype=np.int16),
                             rng.integers(-2**15, 2**15, size=shape, dtype=np.int16))
    return pools


@pytest.mark.parametrize("L,H,ctx,dec", LAYOUTS)
def test_three_statements_agree(L, H, ctx, dec):
    rng = np.random.default_rng(L * 100 + H)
    B, D, nb_src, nb_dst = 2, 4, 7, 9
    (ctx_tp, ctx_pp), (dec_tp, dec_pp) = ctx, dec
    pools = make_pools(rng, nb_src, L, H, ctx_tp, ctx_pp, B, D)
    src = [5, 0, 3, 3]
    dst = [1, 8, 2, 4]
    for p in range(dec_pp):
        for t in range(dec_tp):
            shape = (nb_dst, L // dec_pp, H // dec_tp, B, D)
            init_k = rng.integers(-2**15, 2**15, size=shape, dtype=np.int16)
            init_v = rng.integers(-2**15, 2**15, size=shape, dtype=np.int16)
            outs = []
            for fn in (O.migrate_blocks_elementwise, O.migrate_blocks_numpy, OC.migrate_blocks_c):
                k, v = init_k.copy(), init_v.copy()
                fn(pools, ctx_tp, ctx_pp, src, dec_tp, t, dec_pp, p, dst, k, v, L, H)
                outs.append((k, v))
            tk, tv = torch.from_numpy(init_k.copy()), torch.from_numpy(init_v.copy())
            tpools = {key: (torch.from_numpy(a), torch.from_numpy(b)) for key, (a, b) in pools.items()}
            O.migrate_blocks_torch(tpools, ctx_tp, ctx_pp, src, dec_tp, t, dec_pp, p, dst, tk, tv, L, H)
            outs.append((tk.numpy(), tv.numpy()))
            for k, v in outs[1:]:
                assert np.array_equal(k, outs[0][0]) and np.array_equal(v, outs[0][1])
            # untouched target blocks keep their contents
            untouched = sorted(set(range(nb_dst)) - set(dst))
            assert np.array_equal(outs[0][0][untouched], init_k[untouched])
            assert np.array_equal(outs[0][1][untouched], init_v[untouched])


@pytest.mark.parametrize("L,H,ctx,dec", LAYOUTS)
def test_rectangles_tile_the_plane(L, H, ctx, dec):
    """Tag every source element with its global (layer, head); after all
    decoding workers pulled block 0, each holds exactly its own rectangle."""
    (ctx_tp, ctx_pp), (dec_tp, dec_pp) = ctx, dec
    pools = {}
    for p in range(ctx_pp):
        for t in range(ctx_tp):
            k = np.zeros((1, L // ctx_pp, H // ctx_tp, 1, 1), dtype=np.int32)
            for l, h in itertools.product(range(L // ctx_pp), range(H // ctx_tp)):
                k[0, l, h] = (p * (L // ctx_pp) + l) * 1000 + t * (H // ctx_tp) + h
            pools[(p, t)] = (k, -k)
    seen = set()
    for p in range(dec_pp):
        for t in range(dec_tp):
            k = np.full((1, L // dec_pp, H // dec_tp, 1, 1), -1, dtype=np.int32)
            v = k.copy()
            O.migrate_blocks_numpy(pools, ctx_tp, ctx_pp, [0], dec_tp, t, dec_pp, p, [0], k, v, L, H)
            for l, h in itertools.product(range(L // dec_pp), range(H // dec_tp)):
                tag = (p * (L // dec_pp) + l) * 1000 + t * (H // dec_tp) + h
                assert k[0, l, h, 0, 0] == tag and v[0, l, h, 0, 0] == -tag
                assert tag not in seen
                seen.add(tag)
    assert len(seen) == L * H


def test_equal_layouts_copy_whole_blocks():
    rng = np.random.default_rng(3)
    pools = make_pools(rng, 5, 4, 4, 2, 2, 2, 2)
    for (p, t), (sk, sv) in pools.items():
        k, v = np.zeros_like(sk), np.zeros_like(sv)
        O.migrate_blocks_numpy(pools, 2, 2, [4, 1], 2, t, 2, p, [0, 3], k, v, 4, 4)
        assert np.array_equal(k[[0, 3]], sk[[4, 1]]) and np.array_equal(v[[0, 3]], sv[[4, 1]])
        assert not k[[1, 2, 4]].any()
        assert O.contributing_workers(4, 4, 2, 2, 2, t, 2, p) == [(p, t)]


def test_length_mismatch_and_empty():
    pools = make_pools(np.random.default_rng(0), 2, 2, 2, 1, 1, 1, 1)
    k = np.zeros((2, 2, 2, 1, 1), dtype=np.int16)
    with pytest.raises(ValueError):
        O.migrate_blocks_numpy(pools, 1, 1, [0, 1], 1, 0, 1, 0, [0], k, k.copy(), 2, 2)
    before = k.copy()
    O.migrate_blocks_numpy(pools, 1, 1, [], 1, 0, 1, 0, [], k, k.copy(), 2, 2)
    assert np.array_equal(k, before)
    with pytest.raises(ValueError):
        O.migrate_blocks_numpy(pools, 1, 1, [0], 3, 0, 1, 0, [0], k, k.copy(), 2, 2)   # 2 heads over tp=3


def test_swap_oracle_directions_and_order():
    rng = np.random.default_rng(1)
    g_k, g_v = rng.integers(0, 99, (6, 1, 1, 2, 2)), rng.integers(0, 99, (6, 1, 1, 2, 2))
    h_k, h_v = rng.integers(0, 99, (4, 1, 1, 2, 2)), rng.integers(0, 99, (4, 1, 1, 2, 2))
    g_k0, h_k0, h_v0 = g_k.copy(), h_k.copy(), h_v.copy()
    O.swap_numpy([5, 2], [0, 3], False, g_k, g_v, h_k, h_v)            # out: GPU 5->host 0, GPU 2->host 3
    assert np.array_equal(h_k[0], g_k0[5]) and np.array_equal(h_k[3], g_k0[2])
    assert np.array_equal(h_k[[1, 2]], h_k0[[1, 2]]) and np.array_equal(g_k, g_k0)
    O.swap_numpy([0, 3], [1, 1], True, g_k, g_v, h_k, h_v)             # in, repeated target: last one wins
    assert np.array_equal(g_k[1], h_k[3]) and np.array_equal(g_v[1], h_v[3])
    assert not np.array_equal(h_v, h_v0)
    with pytest.raises(ValueError):
        O.swap_numpy([0], [], True, g_k, g_v, h_k, h_v)


def test_c_oracle_swap_and_refusals_agree_with_numpy():
    rng = np.random.default_rng(2)
    pools = [rng.integers(-2**15, 2**15, size=(n, 2, 3, 4, 8), dtype=np.int16) for n in (6, 6, 4, 4)]
    a = [p.copy() for p in pools]
    b = [p.copy() for p in pools]
    for src, dst, is_in in (([5, 2], [0, 3], False), ([0, 3], [1, 1], True), ([], [], True)):
        O.swap_numpy(src, dst, is_in, *a)
        OC.swap_c(src, dst, is_in, *b)
    for x, y in zip(a, b):
        assert np.array_equal(x, y)
    with pytest.raises(ValueError):
        OC.swap_c([0], [], True, *b)
    k = np.zeros((2, 2, 2, 1, 1), dtype=np.int16)
    ctx = make_pools(rng, 2, 2, 2, 1, 1, 1, 1)
    with pytest.raises(ValueError):
        OC.migrate_blocks_c(ctx, 1, 1, [0, 1], 1, 0, 1, 0, [0], k, k.copy(), 2, 2)
    with pytest.raises(ValueError):
        OC.migrate_blocks_c(ctx, 1, 1, [0], 3, 0, 1, 0, [0], k, k.copy(), 2, 2)


MQA_LAYOUTS = [
    # L, (ctx_tp, ctx_pp), (dec_tp, dec_pp) for a model with ONE KV head (multi-query attention)
    (4, (2, 1), (1, 1)),
    (4, (1, 1), (2, 1)),
    (4, (2, 2), (2, 1)),
    (6, (4, 1), (2, 3)),
    (6, (2, 3), (4, 1)),
]


@pytest.mark.parametrize("L,ctx,dec", MQA_LAYOUTS)
def test_single_kv_head_is_held_by_every_rank(L, ctx, dec):
    """Multi-query attention: ModelConfig.get_num_heads returns 1 whatever the tensor-parallel size
    (distserve/config.py:233-237), so every rank of both stages holds the one head.  All four statements read
    it from the context replica at the matching position, floor(dec_tp_rank * ctx_tp / dec_tp); the replicas
    are given different contents here so that the choice shows."""
    rng = np.random.default_rng(L)
    B, D, nb_src, nb_dst = 2, 4, 6, 8
    (ctx_tp, ctx_pp), (dec_tp, dec_pp) = ctx, dec
    pools = {(p, t): (rng.integers(-2**15, 2**15, size=(nb_src, L // ctx_pp, 1, B, D), dtype=np.int16),
                      rng.integers(-2**15, 2**15, size=(nb_src, L // ctx_pp, 1, B, D), dtype=np.int16))
             for p in range(ctx_pp) for t in range(ctx_tp)}
    src, dst = [4, 1, 1], [0, 7, 3]
    for p in range(dec_pp):
        for t in range(dec_tp):
            replica = t * ctx_tp // dec_tp
            assert O.contributing_workers(L, 1, ctx_tp, ctx_pp, dec_tp, t, dec_pp, p) == sorted(
                {(gl // (L // ctx_pp), replica) for gl in range(p * L // dec_pp, (p + 1) * L // dec_pp)})
            shape = (nb_dst, L // dec_pp, 1, B, D)
            want_k = rng.integers(-2**15, 2**15, size=shape, dtype=np.int16)
            init_k, init_v = want_k.copy(), want_k.copy()
            want_v = want_k.copy()
            for s_id, d_id in zip(src, dst):
                for dl in range(L // dec_pp):
                    gl = p * (L // dec_pp) + dl
                    cp, cl = gl // (L // ctx_pp), gl % (L // ctx_pp)
                    want_k[d_id, dl, 0] = pools[(cp, replica)][0][s_id, cl, 0]
                    want_v[d_id, dl, 0] = pools[(cp, replica)][1][s_id, cl, 0]
            for fn in (O.migrate_blocks_elementwise, O.migrate_blocks_numpy, OC.migrate_blocks_c):
                k, v = init_k.copy(), init_v.copy()
                fn(pools, ctx_tp, ctx_pp, src, dec_tp, t, dec_pp, p, dst, k, v, L, 1)
                assert np.array_equal(k, want_k) and np.array_equal(v, want_v), fn.__name__
            tk, tv = torch.from_numpy(init_k.copy()), torch.from_numpy(init_v.copy())
            tpools = {key: (torch.from_numpy(a), torch.from_numpy(b)) for key, (a, b) in pools.items()}
            O.migrate_blocks_torch(tpools, ctx_tp, ctx_pp, src, dec_tp, t, dec_pp, p, dst, tk, tv, L, 1)
            assert np.array_equal(tk.numpy(), want_k) and np.array_equal(tv.numpy(), want_v)

"""The allocation-free migration entry point (kvmig_migrate_blocks_static).

Some hosts may not allocate device memory once serving has started: a decoding
worker sizes its KV pools from the HBM that is free at start-up, so a later
cudaMalloc can fail or stall the device mid-loop, and some embedders forbid
allocation after start-up.  For them the library offers the same copy with its
scratch (block tables, status word) in a fixed array that is part of the loaded
module.  This file checks, through the C ABI, that the variant writes exactly
what the ordinary entry point writes and what the CPU oracle computes — on two
calls in a row, the second shorter than the first so that stale table contents
would show — that device
memory in use does not change across the calls, and that oversize requests
are refused.  It is collected last on purpose.
"""
import numpy as np
import pytest
import torch

from distserve_b200 import capi
from tests.kvutil import Stage, assert_stage_equals_host, oracle_all, register_all

pytestmark = pytest.mark.gpu


def pull(entry, ctx, dec, src, dst):
    for dp in range(dec.pp):
        for dt in range(dec.tp):
            k, v = dec.dev[(dp, dt)]
            entry(ctx.pp, ctx.tp, src, dec.pp, dec.tp, dp, dt, dst, k.data_ptr(), v.data_ptr(), dec.shape((dp, dt)))


def pools_equal(a: Stage, b: Stage):
    return all(torch.equal(a.dev[key][x], b.dev[key][x]) for key in a.dev for x in range(2))


@pytest.mark.parametrize("ctx_layout,dec_layout", [((1, 1), (1, 1)), ((4, 1), (2, 2))])
def test_static_entry_point_matches_the_ordinary_one_twice_in_a_row(ctx_layout, dec_layout):
    capi.reset_registry()
    rng = np.random.default_rng(77)
    L, H, B, D = 8, 8, 4, 16
    ctx = Stage(L, H, *ctx_layout, 300, B, D, seed=41)
    ordinary = Stage(L, H, *dec_layout, 280, B, D, seed=42)
    static = Stage(L, H, *dec_layout, 280, B, D, seed=42)           # same initial contents
    register_all(ctx, ordinary)                                    # one registry serves both: same device, same ranks
    assert pools_equal(ordinary, static)
    pull(capi.migrate_blocks, ctx, ordinary, [0], [0])              # loads the module's kernels before memory is sampled
    pull(capi.migrate_blocks_static, ctx, static, [0], [0])         # first call: looks up the array's address
    oracle_all(ctx, static, [0], [0])
    for n in (257, 9):                                              # two calls in a row; the second reuses the array
        src = [int(x) for x in rng.integers(0, 300, size=n)]
        dst = [int(x) for x in rng.permutation(280)[:n]]
        pull(capi.migrate_blocks, ctx, ordinary, src, dst)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        pull(capi.migrate_blocks_static, ctx, static, src, dst)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "device memory in use changed across the static call"
        assert pools_equal(ordinary, static), f"pools differ after the call with {n} blocks"   # bit-exact, no tolerance
        # and both equal what the CPU oracle computes for the same call (the host copies start out equal too)
        oracle_all(ctx, static, src, dst)
        assert_stage_equals_host(static, f"static entry point, {n} blocks")


def test_static_entry_point_limits_and_refusals():
    capi.reset_registry()
    ctx = Stage(2, 2, 1, 1, 8, 2, 8, seed=43)
    dec = Stage(2, 2, 1, 1, 8, 2, 8, seed=44)
    k, v = dec.dev[(0, 0)]
    args = lambda src, dst: (1, 1, src, 1, 1, 0, 0, dst, k.data_ptr(), v.data_ptr(), dec.shape())
    with pytest.raises(capi.KvmigError) as e:
        capi.migrate_blocks_static(*args([0], [0]))                 # nothing registered
    assert e.value.code == capi.ENOTREG
    register_all(ctx, dec)
    too_many = capi.STATIC_MAX_BLOCKS + 1
    with pytest.raises(capi.KvmigError, match="exceed the 4096") as e:
        capi.migrate_blocks_static(*args([0] * too_many, list(range(too_many))))
    assert e.value.code == capi.ELIMIT
    before = (k.clone(), v.clone())
    for src, dst, text in [([0, 1], [0], "entries"), ([8], [0], "outside the context pool"), ([0, 1], [3, 3], "twice")]:
        with pytest.raises(capi.KvmigError, match=text):
            capi.migrate_blocks_static(*args(src, dst))
    capi.migrate_blocks_static(*args([], []))
    assert torch.equal(k, before[0]) and torch.equal(v, before[1])
    capi.migrate_blocks_static(*args([7, 2], [1, 6]))
    sk, sv = ctx.dev[(0, 0)]
    assert torch.equal(k[[1, 6]], sk[[7, 2]]) and torch.equal(v[[1, 6]], sv[[7, 2]])

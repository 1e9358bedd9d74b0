"""ctypes face of oracle/kv_oracle.c (TEST INFRASTRUCTURE ONLY; parity
unpinned, see kv_oracle.py).  Same call shapes as the numpy oracle; pools may
be numpy arrays or CPU torch tensors (anything with a writable buffer address)."""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np

from .build_oracle import build

_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(build()))
        _lib.kv_oracle_migrate.restype = C.c_int
        _lib.kv_oracle_swap.restype = C.c_int
    return _lib


def _addr(pool) -> int:
    if isinstance(pool, np.ndarray):
        if not pool.flags["C_CONTIGUOUS"]:
            raise ValueError("pools must be contiguous")
        return pool.ctypes.data
    if not pool.is_contiguous():
        raise ValueError("pools must be contiguous")
    return pool.data_ptr()


def _i64(values: Sequence[int]):
    return (C.c_int64 * max(1, len(values)))(*values)


def _slab(pool) -> int:
    shape = tuple(pool.shape)
    item = pool.itemsize if isinstance(pool, np.ndarray) else pool.element_size()
    return shape[3] * shape[4] * item


def migrate_blocks_c(ctx_pools, ctx_tp, ctx_pp, ctx_blocks, dec_tp, dec_tp_rank, dec_pp, dec_pp_rank, dec_blocks,
                     k_cache, v_cache, num_layers, num_heads) -> None:
    n = ctx_tp * ctx_pp
    ks, vs = (C.c_void_p * n)(), (C.c_void_p * n)()
    for (p, t), (k, v) in ctx_pools.items():
        ks[p * ctx_tp + t], vs[p * ctx_tp + t] = _addr(k), _addr(v)
    rc = lib().kv_oracle_migrate(ks, vs, C.c_int64(ctx_tp), C.c_int64(ctx_pp), _i64(ctx_blocks), C.c_int64(len(ctx_blocks)),
                                 C.c_int64(dec_tp), C.c_int64(dec_tp_rank), C.c_int64(dec_pp), C.c_int64(dec_pp_rank),
                                 _i64(dec_blocks), C.c_int64(len(dec_blocks)), C.c_void_p(_addr(k_cache)),
                                 C.c_void_p(_addr(v_cache)), C.c_int64(num_layers), C.c_int64(num_heads),
                                 C.c_int64(_slab(k_cache)))
    if rc != 0:
        raise ValueError("kv_oracle_migrate refused its arguments (list lengths or divisibility)")


def swap_c(source_block_ids, target_block_ids, is_swap_in, k_cache, v_cache, k_swap, v_swap) -> None:
    shape = tuple(k_cache.shape)
    block_bytes = shape[1] * shape[2] * _slab(k_cache)
    rc = lib().kv_oracle_swap(_i64(source_block_ids), C.c_int64(len(source_block_ids)), _i64(target_block_ids),
                              C.c_int64(len(target_block_ids)), C.c_int(int(bool(is_swap_in))), C.c_void_p(_addr(k_cache)),
                              C.c_void_p(_addr(v_cache)), C.c_void_p(_addr(k_swap)), C.c_void_p(_addr(v_swap)),
                              C.c_int64(block_bytes))
    if rc != 0:
        raise ValueError("kv_oracle_swap refused its arguments (list lengths)")

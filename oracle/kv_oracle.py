"""CPU oracle for DistServe's paged-KV block migration and block swap.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module;
only the test-suite, the smoke check and the benchmark's CPU-baseline leg do,
and there only as the checker / the timed CPU arm.

PARITY UNPINNED.  The arithmetic of this path is implemented by the reference
in SwiftTransformer (``libst_pybinding.so``, loaded at
``distserve/__init__.py:4-16``), a separate un-vendored project for which the
reference pins no commit and ships no test vector.  What follows is therefore a
restatement of the semantics that the reference's *call sites* fix:

* pool layout ``[num_blocks, layers_local, kv_heads_local, block_size,
  head_dim]``, K and V separately (``distserve/worker.py:107-121``);
* a worker ``(tp, tp_rank, pp, pp_rank)`` owns ``L/pp`` consecutive layers and
  ``H/tp`` consecutive KV heads (``distserve/config.py:244-257,279-286``; head
  chunk ``i`` belongs to tensor-parallel rank ``i``,
  ``distserve/downloader/converter.py:339-350``; pipeline rank ``i`` holds the
  ``i``-th run of layers, ``distserve/single_stage_engine.py:152-161``);
* ``migrate_blocks`` receives only block indexes, so whole blocks move, for K
  and for V (``distserve/worker.py:250-267``);
* ``swap`` copies ``source_block_ids[i] -> target_block_ids[i]`` between the
  GPU pool and the pinned host pool, direction chosen by ``is_swap_in``
  (``distserve/worker.py:269-311``).

Three forms are given.  ``migrate_blocks_elementwise`` is the literal
per-(block, layer, head) statement and is only meant for small cases;
``migrate_blocks_numpy`` is the same thing with sliced assignments and is
checked against the literal form in the tests; ``migrate_blocks_torch`` is the
"block-indexed gather/scatter as torch CPU copies" that the benchmark times as
the CPU baseline.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import numpy as np

# (pp_rank, tp_rank) -> (k_pool, v_pool); the order pp-then-tp mirrors the
# nesting of the handle table in distserve/worker.py:234-235.
PoolMap = Dict[Tuple[int, int], Tuple[object, object]]


def _owner(index: int, total: int, parts: int) -> Tuple[int, int]:
    """Which of ``parts`` equal consecutive chunks of ``range(total)`` holds
    ``index``, and at which local offset (distserve/config.py:244-257,279-286)."""
    if total % parts != 0:
        raise ValueError(f"{total} is not divisible by {parts}")
    per = total // parts
    return index // per, index % per


def migrate_blocks_elementwise(
    ctx_pools: PoolMap,
    ctx_tp: int,
    ctx_pp: int,
    ctx_blocks: Sequence[int],
    dec_tp: int,
    dec_tp_rank: int,
    dec_pp: int,
    dec_pp_rank: int,
    dec_blocks: Sequence[int],
    k_cache,
    v_cache,
    num_layers: int,
    num_heads: int,
) -> None:
    """Literal statement: every (block, global layer, global head) of the
    decoding worker's rectangle is fetched from whichever context worker owns
    that layer and head.  Follows distserve/worker.py:250-267 for the argument
    meaning and distserve/single_stage_engine.py:516-517 for the equal-length
    requirement."""
    if len(ctx_blocks) != len(dec_blocks):
        raise ValueError("block index lists differ in length")
    l_per_dec = num_layers // dec_pp
    h_per_dec = 1 if num_heads == 1 else num_heads // dec_tp
    for src_id, dst_id in zip(ctx_blocks, dec_blocks):
        for dl in range(l_per_dec):
            gl = dec_pp_rank * l_per_dec + dl
            c_pp_rank, cl = _owner(gl, num_layers, ctx_pp)
            for dh in range(h_per_dec):
                if num_heads == 1:
                    # Multi-query attention: every tensor-parallel rank of either stage holds the one KV head
                    # (distserve/config.py:233-237); which replica is read does not change the result.
                    c_tp_rank, ch = dec_tp_rank * ctx_tp // dec_tp, 0
                else:
                    gh = dec_tp_rank * h_per_dec + dh
                    c_tp_rank, ch = _owner(gh, num_heads, ctx_tp)
                src_k, src_v = ctx_pools[(c_pp_rank, c_tp_rank)]
                k_cache[dst_id, dl, dh] = src_k[src_id, cl, ch]
                v_cache[dst_id, dl, dh] = src_v[src_id, cl, ch]


def _overlaps(num_layers, num_heads, ctx_tp, ctx_pp, dec_tp, dec_tp_rank, dec_pp, dec_pp_rank):
    """Yield, for each context worker that feeds this decoding worker, the
    slices to read and to write.  Derived by walking the global (layer, head)
    plane in the decoding worker's own order and cutting wherever the owning
    context worker changes."""
    checks = [(num_layers, dec_pp), (num_layers, ctx_pp)] + ([] if num_heads == 1 else [(num_heads, dec_tp), (num_heads, ctx_tp)])
    for total, parts in checks:
        if total % parts != 0:
            raise ValueError(f"{total} is not divisible by {parts}")
    l_per_dec, l_per_ctx = num_layers // dec_pp, num_layers // ctx_pp
    gl0 = dec_pp_rank * l_per_dec
    if num_heads == 1:
        # Multi-query attention (distserve/config.py:233-237): one KV head on every rank; read the replica at the
        # matching position of the context stage.
        t = dec_tp_rank * ctx_tp // dec_tp
        g = gl0
        while g < gl0 + l_per_dec:
            p = g // l_per_ctx
            end = min(gl0 + l_per_dec, (p + 1) * l_per_ctx)
            yield (p, t), (slice(g - p * l_per_ctx, end - p * l_per_ctx), slice(0, 1)), (slice(g - gl0, end - gl0), slice(0, 1))
            g = end
        return
    h_per_dec, h_per_ctx = num_heads // dec_tp, num_heads // ctx_tp
    gh0 = dec_tp_rank * h_per_dec

    def cuts(g0, n, per):
        out, g = [], g0
        while g < g0 + n:
            owner = g // per
            end = min(g0 + n, (owner + 1) * per)
            out.append((owner, g, end))
            g = end
        return out

    for p, la, lb in cuts(gl0, l_per_dec, l_per_ctx):
        for t, ha, hb in cuts(gh0, h_per_dec, h_per_ctx):
            yield (
                (p, t),
                (slice(la - p * l_per_ctx, lb - p * l_per_ctx), slice(ha - t * h_per_ctx, hb - t * h_per_ctx)),
                (slice(la - gl0, lb - gl0), slice(ha - gh0, hb - gh0)),
            )


def migrate_blocks_numpy(
    ctx_pools: PoolMap,
    ctx_tp: int,
    ctx_pp: int,
    ctx_blocks: Sequence[int],
    dec_tp: int,
    dec_tp_rank: int,
    dec_pp: int,
    dec_pp_rank: int,
    dec_blocks: Sequence[int],
    k_cache: np.ndarray,
    v_cache: np.ndarray,
    num_layers: int,
    num_heads: int,
) -> None:
    """Same result as :func:`migrate_blocks_elementwise`, with one gather and
    one scatter per contributing context worker and per K/V pool."""
    if len(ctx_blocks) != len(dec_blocks):
        raise ValueError("block index lists differ in length")
    if len(ctx_blocks) == 0:
        return
    src_ids = np.asarray(ctx_blocks, dtype=np.int64)
    dst_ids = np.asarray(dec_blocks, dtype=np.int64)
    for key, (sl, sh), (dl, dh) in _overlaps(
        num_layers, num_heads, ctx_tp, ctx_pp, dec_tp, dec_tp_rank, dec_pp, dec_pp_rank
    ):
        src_k, src_v = ctx_pools[key]
        k_cache[dst_ids, dl, dh] = src_k[src_ids, sl, sh]
        v_cache[dst_ids, dl, dh] = src_v[src_ids, sl, sh]


def migrate_blocks_torch(
    ctx_pools: PoolMap,
    ctx_tp: int,
    ctx_pp: int,
    ctx_blocks: Sequence[int],
    dec_tp: int,
    dec_tp_rank: int,
    dec_pp: int,
    dec_pp_rank: int,
    dec_blocks: Sequence[int],
    k_cache,
    v_cache,
    num_layers: int,
    num_heads: int,
) -> None:
    """The timed CPU baseline: block-indexed gather (``index_select``) and
    scatter (``index_copy_``) on host tensors, one call per request as in
    distserve/single_stage_engine.py:490-536.  torch runs these with its
    intra-op thread pool."""
    import torch

    if len(ctx_blocks) != len(dec_blocks):
        raise ValueError("block index lists differ in length")
    if len(ctx_blocks) == 0:
        return
    src_ids = torch.as_tensor(list(ctx_blocks), dtype=torch.int64)
    dst_ids = torch.as_tensor(list(dec_blocks), dtype=torch.int64)
    for key, (sl, sh), (dl, dh) in _overlaps(
        num_layers, num_heads, ctx_tp, ctx_pp, dec_tp, dec_tp_rank, dec_pp, dec_pp_rank
    ):
        src_k, src_v = ctx_pools[key]
        whole = (
            sl == slice(0, src_k.shape[1]) and sh == slice(0, src_k.shape[2])
            and dl == slice(0, k_cache.shape[1]) and dh == slice(0, k_cache.shape[2])
        )
        for src, dst in ((src_k, k_cache), (src_v, v_cache)):
            if whole:
                dst.index_copy_(0, dst_ids, src.index_select(0, src_ids))
            else:
                dst[:, dl, dh].index_copy_(0, dst_ids, src[:, sl, sh].index_select(0, src_ids))


def swap_numpy(
    source_block_ids: Sequence[int],
    target_block_ids: Sequence[int],
    is_swap_in: bool,
    k_cache,
    v_cache,
    k_swap,
    v_swap,
) -> None:
    """Block swap between the GPU pool and the host pool, in list order
    (distserve/worker.py:269-311; the lists come from
    distserve/block_manager.py:288-315).  Applied one block at a time so that a
    repeated target id ends up holding the last source, as a sequence of
    copies on one stream would leave it."""
    if len(source_block_ids) != len(target_block_ids):
        raise ValueError("block id lists differ in length")
    for s, t in zip(source_block_ids, target_block_ids):
        if is_swap_in:
            k_cache[t] = k_swap[s]
            v_cache[t] = v_swap[s]
        else:
            k_swap[t] = k_cache[s]
            v_swap[t] = v_cache[s]


def contributing_workers(num_layers, num_heads, ctx_tp, ctx_pp, dec_tp, dec_tp_rank, dec_pp, dec_pp_rank) -> List[Tuple[int, int]]:
    """(pp_rank, tp_rank) of every context worker a decoding worker reads."""
    return [k for k, _, _ in _overlaps(num_layers, num_heads, ctx_tp, ctx_pp, dec_tp, dec_tp_rank, dec_pp, dec_pp_rank)]

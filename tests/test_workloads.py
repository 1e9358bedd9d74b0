"""Seeded workloads: determinism, shapes, and block-id hygiene of the traces
that the benchmark and the end-to-end tests replay."""
import math

import pytest

from distserve_b200.config import KVModelConfig, ParallelConfig, plan_overlaps
from distserve_b200.workloads import WORKLOADS, make_trace, prompt_lengths, trace_blocks
from oracle import kv_oracle as O

EXPECTED_BYTES = {"c1": 589_824, "c2": 13_107_200, "c3": 13_107_200, "c4": 1_310_720, "c5": 4_194_304}


@pytest.mark.parametrize("name", sorted(WORKLOADS))
def test_trace_is_deterministic_and_well_formed(name):
    w = WORKLOADS[name]
    assert w.dec_block_bytes() == EXPECTED_BYTES[name]
    lengths = prompt_lengths(w)
    assert lengths == prompt_lengths(w) and len(lengths) == w.num_requests
    kind = w.length_dist[0]
    if kind == "uniform":
        assert min(lengths) >= w.length_dist[1] and max(lengths) <= w.length_dist[2]
    else:
        assert min(lengths) >= 1 and max(lengths) <= w.length_dist[3]
        median = sorted(lengths)[len(lengths) // 2]
        assert 0.6 * w.length_dist[1] < median < 1.6 * w.length_dist[1]
    trace = make_trace(w)
    assert trace == make_trace(w)
    for item in trace:
        n = math.ceil(item.prompt_len / w.block_size)
        assert len(item.src_blocks) == len(item.dst_blocks) == n
        assert len(set(item.src_blocks)) == n and len(set(item.dst_blocks)) == n
        assert all(0 <= b < w.ctx_pool_blocks for b in item.src_blocks)
        assert all(0 <= b < w.dec_pool_blocks for b in item.dst_blocks)
    assert trace_blocks(trace) == sum(math.ceil(n / w.block_size) for n in lengths)
    # ids are scattered, not consecutive runs (a permuted free list)
    first = trace[0].dst_blocks
    assert any(b - a != 1 for a, b in zip(first, first[1:]))


def test_c1_demand_exceeds_its_pool_so_ids_are_recycled():
    w = WORKLOADS["c1"]
    trace = make_trace(w)
    assert trace_blocks(trace) > w.dec_pool_blocks
    used = [b for item in trace for b in item.dst_blocks]
    assert len(set(used)) < len(used)


@pytest.mark.parametrize("name", sorted(WORKLOADS))
def test_host_overlap_plan_agrees_with_the_oracle(name):
    """The package's interval-intersection plan and the oracle's ownership walk
    name the same context workers for every decoding worker."""
    w = WORKLOADS[name]
    for p in range(w.dec_pp):
        for t in range(w.dec_tp):
            plan = plan_overlaps(w.model, w.ctx_config(), w.dec_config(p, t))
            ours = sorted((o.ctx_pp_rank, o.ctx_tp_rank) for o in plan)
            theirs = sorted(O.contributing_workers(w.model.num_layers, w.model.num_kv_heads, w.ctx_tp, w.ctx_pp,
                                                   w.dec_tp, t, w.dec_pp, p))
            assert ours == theirs
            layers = sum((o.dst_layers[1] - o.dst_layers[0]) * (o.dst_heads[1] - o.dst_heads[0]) for o in plan)
            assert layers == w.model.get_num_layers(w.dec_config()) * w.model.get_num_heads(w.dec_config())


def test_c4_decoding_workers_pull_from_the_expected_context_gpus():
    w = WORKLOADS["c4"]
    for p in range(2):
        for t in range(2):
            plan = plan_overlaps(w.model, w.ctx_config(), w.dec_config(p, t))
            assert [(o.ctx_pp_rank, o.ctx_tp_rank) for o in plan] == [(0, 2 * t), (0, 2 * t + 1)]
            assert all(o.src_layers == (40 * p, 40 * p + 40) and o.src_heads == (0, 2) for o in plan)
            assert [o.dst_heads for o in plan] == [(0, 2), (2, 4)]


def test_invalid_layouts_are_refused():
    with pytest.raises(ValueError):
        ParallelConfig(2, 2, 1, 0)
    with pytest.raises(ValueError):
        KVModelConfig(40, 40, 128).get_num_heads(ParallelConfig(3, 0, 1, 0))


def test_single_kv_head_geometry_mirrors_the_reference():
    """distserve/config.py:233-237: a multi-query model has one KV head on every tensor-parallel rank."""
    from distserve_b200.config import KVModelConfig, ParallelConfig, plan_overlaps

    m = KVModelConfig(8, 1, 64)
    for tp in (1, 2, 4):
        for t in range(tp):
            pc = ParallelConfig(tp, t, 2, 1)
            assert m.get_num_heads(pc) == 1 and m.head_range(pc) == (0, 1) and m.get_num_layers(pc) == 4
    ov = plan_overlaps(m, ParallelConfig(4, 0, 1, 0), ParallelConfig(2, 1, 2, 0))
    assert [(o.ctx_pp_rank, o.ctx_tp_rank, o.src_layers, o.src_heads, o.dst_layers, o.dst_heads) for o in ov] == \
        [(0, 2, (0, 4), (0, 1), (0, 4), (0, 1))]

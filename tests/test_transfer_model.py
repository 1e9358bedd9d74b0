"""The transfer-cost model against what the benchmark measured on B200
(median awaited-call latency and back-to-back throughput per workload)."""
import pytest

from distserve_b200 import transfer_model as T
from distserve_b200.workloads import WORKLOADS, make_trace

# workload -> (median awaited call in µs, per-destination GB/s with calls enqueued back to back)
MEASURED_NVLINK = {"c2": (671, 792), "c3": (1230, 782), "c5": (183, 789), "c4": (132, 787)}


@pytest.mark.parametrize("name", sorted(MEASURED_NVLINK))
def test_nvlink_model_matches_measured_latency_and_throughput(name):
    w = WORKLOADS[name]
    trace = make_trace(w)
    lengths = sorted(t.prompt_len for t in trace)
    median_len = lengths[len(lengths) // 2]
    p50_us, chained_gbps = MEASURED_NVLINK[name]
    predicted = T.migration_seconds(median_len, w.model, w.dec_config(), w.block_size, T.NVLINK5, awaited=True) * 1e6
    assert predicted == pytest.approx(p50_us, rel=0.06)
    total_payload = sum(T.blocks_for(t.prompt_len, w.block_size) for t in trace) * w.dec_block_bytes()
    total_time = sum(T.migration_seconds(t.prompt_len, w.model, w.dec_config(), w.block_size, T.NVLINK5, awaited=False)
                     for t in trace)
    assert total_payload / total_time / 1e9 == pytest.approx(chained_gbps, rel=0.04)


def test_same_gpu_model_and_limits():
    w = WORKLOADS["c2"]
    trace = make_trace(w)
    total_payload = sum(len(t.src_blocks) for t in trace) * w.dec_block_bytes()
    chained = sum(T.migration_seconds(t.prompt_len, w.model, w.dec_config(), 16, T.SAME_GPU_HBM3E, awaited=False) for t in trace)
    awaited = sum(T.migration_seconds(t.prompt_len, w.model, w.dec_config(), 16, T.SAME_GPU_HBM3E, awaited=True) for t in trace)
    assert 2 * total_payload / chained / 1e9 == pytest.approx(6897, rel=0.03)      # measured `value`, read + write
    assert 2 * total_payload / awaited / 1e9 == pytest.approx(6155, rel=0.04)      # measured `e2e`
    assert T.migration_seconds(0, w.model, w.dec_config()) == 0.0
    short = T.effective_GBps(16, w.model, w.dec_config())       # one block: dominated by the fixed cost
    long_ = T.effective_GBps(2048, w.model, w.dec_config())
    assert short < 0.5 * long_ < 0.5 * T.NVLINK5.payload_GBps + 1


def test_charging_the_transfer_changes_the_placement():
    """The reference's simulator hands a request from prefill to decode with no delay, so a search on it prefers
    whatever decodes most cheaply; once the hand-off is charged, a stage that pulls over a slow link needs more
    workers (each pulls a smaller share), and the choice flips.  Over NVLink the transfer is too short to matter."""
    w = WORKLOADS["c2"]
    lens = [t.prompt_len for t in make_trace(w)]
    slow = [T.DecodePlacement(1, 1, T.CROSS_NODE_400G, goodput_per_gpu=1.00),
            T.DecodePlacement(2, 1, T.CROSS_NODE_400G, goodput_per_gpu=0.93),
            T.DecodePlacement(4, 1, T.CROSS_NODE_400G, goodput_per_gpu=0.85)]
    free, delay = T.pick_decode_placement(slow, lens, w.model, max_handoff_ms=10.0, charge_transfer=False)
    assert (free.tp, free.pp, delay) == (1, 1, 0.0)
    charged, delay = T.pick_decode_placement(slow, lens, w.model, max_handoff_ms=10.0, charge_transfer=True)
    assert (charged.tp, charged.pp) == (4, 1) and 5.0 < delay <= 10.0
    # streaming the KV during prefill leaves only the last group after prefill ends: the cheapest layout fits again
    streamed, delay = T.pick_decode_placement(slow, lens, w.model, max_handoff_ms=10.0, streamed_groups=8)
    assert (streamed.tp, streamed.pp) == (1, 1) and delay < 10.0
    fast = [T.DecodePlacement(c.tp, c.pp, T.NVLINK5, c.goodput_per_gpu) for c in slow]
    nv, delay = T.pick_decode_placement(fast, lens, w.model, max_handoff_ms=10.0)
    assert (nv.tp, nv.pp) == (1, 1) and delay < 2.5
    with pytest.raises(ValueError):
        T.pick_decode_placement(slow, lens, w.model, max_handoff_ms=1.0)


def test_exit_prefill_delay_is_the_awaited_migration_in_milliseconds():
    w = WORKLOADS["c4"]
    dec = w.dec_config()
    assert T.exit_prefill_delay_ms(1024, w.model, dec) == pytest.approx(T.migration_seconds(1024, w.model, dec) * 1e3)
    assert T.exit_prefill_delay_ms(0, w.model, dec) == 0.0
    whole = T.exit_prefill_delay_ms(4096, w.model, dec)
    assert T.exit_prefill_delay_ms(4096, w.model, dec, streamed_groups=8) < whole / 4

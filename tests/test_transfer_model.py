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

"""The serving loop around the migration path: migrations enqueued beside
decode steps must leave the same KV in the decoding pool as awaited ones, and
must not cost the loop more than the awaited cadence does."""
import pytest
import torch

from distserve_b200 import capi, e2e_loop

pytestmark = pytest.mark.gpu


def test_overlapped_loop_is_correct_and_no_slower_than_serial():
    capi.reset_registry()
    gpus = 2 if torch.cuda.device_count() >= 2 else 1
    out = e2e_loop.run(gpus=gpus, steps=80, rate=4.0, weight_gb=1.0, pool_blocks=512, time_scale=400.0)
    assert out["verified"] is True
    assert out["migrations"] >= 5 and out["blocks_migrated"] > 0
    loop = out["loop_ms"]
    assert loop["serial"] >= loop["decode_only"] * 0.98
    assert loop["overlapped"] <= loop["serial"] * 1.05
    capi.reset_registry()


def test_swaps_beside_decode_steps_keep_the_data_and_cost_less_than_waiting():
    out = e2e_loop.run_swap(steps=60, weight_gb=1.0, pool_blocks=256, request_blocks=16, every=5)
    assert out["data_intact_after_round_trips"] is True
    assert out["loop_ms"]["overlapped"] <= out["loop_ms"]["awaited"] * 1.05


def test_loop_with_one_worker_process_per_gpu():
    """The loop at the layout of the end-to-end configuration — context tp=2 and decoding tp=2 workers, each in
    its own process, on four GPUs when there are four (sharing the GPUs that exist otherwise): every mode moves
    the same requests, the overlapped copies end up bit-identical to their sources, and the loop that enqueues
    them beside the steps is not slower than the one that awaits them between steps."""
    out = e2e_loop.run_actors(n_gpus=min(4, torch.cuda.device_count()), steps=60, weight_gb=0.5, pool_blocks=256,
                              time_scale=400.0, passes=1)
    assert out["replicas"] == 1 and out["verified"] is True
    rep = out["per_replica"][0]
    assert rep["migrations"] >= 5 and rep["blocks_migrated"] > 0
    loop = rep["loop_ms"]
    assert loop["serial"] >= loop["decode_only"] * 0.95
    assert loop["overlapped"] <= loop["serial"] * 1.10
    assert out["layout"].startswith("context tp2pp1 -> decoding tp2pp1")


def test_arrivals_follow_the_reference_generator():
    """Gamma(shape 1) inter-arrival times at the requested rate (evaluation/2-benchmark-serving/
    2-benchmark-serving.py:49-53): the mean gap over a long horizon is 1/rate."""
    steps = e2e_loop.poisson_arrival_steps(rate_per_s=200.0, step_ms=1.0, steps=20000, seed=3)
    assert steps == sorted(steps) and 3600 < len(steps) < 4400       # 20 s at 200 requests per second

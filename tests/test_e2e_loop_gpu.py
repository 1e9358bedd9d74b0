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

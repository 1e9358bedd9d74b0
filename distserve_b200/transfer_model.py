"""Cost model of one KV migration, fitted to the measurements of this library
on B200: what a placement search or a simulator needs in order to
charge for the transfer.  The reference's simulator charges nothing for it
(simdistserve/base/worker.py:264-279 moves a request from prefill to decode
with no delay; the only KV-related helper is a size estimate,
simdistserve/profilers/profile_memory.py:90).

time = fixed cost per call + bytes into the slowest decoding worker / bandwidth

* Each decoding worker pulls its own rectangle concurrently, so the request's
  transfer time is that of ONE worker's share: ``2·(L/dec_pp)·(H/dec_tp)·
  block_size·head_dim·elem`` bytes per block.
* Across NVLink a call moves 790 GB/s into a GPU once it is running, plus about
  14 µs of ramp-up and tail; an awaited call adds the platform's
  launch-and-wait round trip, about 15 µs more.  Calls enqueued back to back
  with disjoint targets overlap their ramp-up and tail, and pay about 2 µs.
* Inside one GPU the same copy runs at 6.8 TB/s counted read + write, i.e.
  3.4 TB/s of payload.
"""
from __future__ import annotations

from dataclasses import dataclass

from .config import KVModelConfig, ParallelConfig


@dataclass(frozen=True)
class LinkModel:
    payload_GBps: float            # bytes written into the destination per second, steady state
    awaited_call_us: float         # fixed cost of one awaited call (launch, ramp-up, tail, wake-up)
    chained_call_us: float         # fixed cost of a call enqueued behind another, independent one


NVLINK5 = LinkModel(payload_GBps=790.0, awaited_call_us=29.0, chained_call_us=2.0)
SAME_GPU_HBM3E = LinkModel(payload_GBps=3400.0, awaited_call_us=22.0, chained_call_us=1.0)


def blocks_for(prompt_len: int, block_size: int) -> int:
    return -(-prompt_len // block_size)


def bytes_per_block_per_worker(model: KVModelConfig, dec: ParallelConfig, block_size: int) -> int:
    return 2 * model.block_bytes(dec, block_size)


def migration_seconds(prompt_len: int, model: KVModelConfig, dec: ParallelConfig, block_size: int = 16,
                      link: LinkModel = NVLINK5, awaited: bool = True) -> float:
    """Time until the request's KV is in place on every decoding worker."""
    if prompt_len <= 0:
        return 0.0
    payload = blocks_for(prompt_len, block_size) * bytes_per_block_per_worker(model, dec, block_size)
    fixed_us = link.awaited_call_us if awaited else link.chained_call_us
    return fixed_us * 1e-6 + payload / (link.payload_GBps * 1e9)


def effective_GBps(prompt_len: int, model: KVModelConfig, dec: ParallelConfig, block_size: int = 16,
                   link: LinkModel = NVLINK5, awaited: bool = True) -> float:
    """Payload bytes per second into one decoding worker for requests of this length."""
    payload = blocks_for(prompt_len, block_size) * bytes_per_block_per_worker(model, dec, block_size)
    return payload / migration_seconds(prompt_len, model, dec, block_size, link, awaited) / 1e9


# ---------------------------------------------------------------------------------------------------------
# The term as a simulator / placement search would consume it
# ---------------------------------------------------------------------------------------------------------

# A 400 Gb/s network port between nodes, for placements that put the two stages on different nodes.  Not
# measured here (this library moves blocks inside one node); the figure only has to be an order of magnitude
# below NVLink for the search to see the difference.
CROSS_NODE_400G = LinkModel(payload_GBps=45.0, awaited_call_us=60.0, chained_call_us=10.0)


def exit_prefill_delay_ms(prompt_len: int, model: KVModelConfig, dec: ParallelConfig, block_size: int = 16,
                          link: LinkModel = NVLINK5, streamed_groups: int = 0) -> float:
    """Delay to charge between the end of a request's prefill and its entry into the decoding stage, in the
    simulator's time unit (milliseconds): what a hook in ``Worker._exit_prefill`` would wait before it calls
    ``forward_decode`` (simdistserve/base/worker.py:264-279 hands the request over with no delay at all).

    With ``streamed_groups`` > 0 the KV is pulled layer group by layer group while prefill is still running, and
    only the last group's share of the payload is left after prefill ends."""
    if prompt_len <= 0:
        return 0.0
    payload = blocks_for(prompt_len, block_size) * bytes_per_block_per_worker(model, dec, block_size)
    if streamed_groups > 0:
        payload = payload / streamed_groups
    return (link.awaited_call_us * 1e-6 + payload / (link.payload_GBps * 1e9)) * 1e3


@dataclass(frozen=True)
class DecodePlacement:
    """One candidate of a placement search: the decoding stage's layout, the link its workers pull the KV over,
    and the decoding goodput per GPU the simulator predicts for it (any unit; only the order matters)."""

    tp: int
    pp: int
    link: LinkModel
    goodput_per_gpu: float

    def worker(self) -> ParallelConfig:
        return ParallelConfig(self.tp, 0, self.pp, 0)


def pick_decode_placement(candidates, prompt_lens, model: KVModelConfig, max_handoff_ms: float, block_size: int = 16,
                          charge_transfer: bool = True, streamed_groups: int = 0, percentile: float = 0.9):
    """The candidate with the highest goodput per GPU among those whose hand-off delay (at the given percentile of
    the prompt lengths) fits `max_handoff_ms`.  With ``charge_transfer`` off every candidate fits — the reference
    simulator's view, in which the transfer is free.  Returns (candidate, its hand-off delay in ms); raises if
    nothing fits."""
    lens = sorted(prompt_lens)
    at = lens[min(len(lens) - 1, int(percentile * len(lens)))]
    best = None
    for c in candidates:
        delay = exit_prefill_delay_ms(at, model, c.worker(), block_size, c.link, streamed_groups) if charge_transfer else 0.0
        if delay <= max_handoff_ms and (best is None or c.goodput_per_gpu > best[0].goodput_per_gpu):
            best = (c, delay)
    if best is None:
        raise ValueError("no placement hands a request over within the budget")
    return best

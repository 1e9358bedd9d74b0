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

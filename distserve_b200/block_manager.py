"""Block-id bookkeeping for one stage: the mirror of
``distserve/block_manager.py`` (BlockManager 20-330).  It produces the source
and target index lists that the migration and swap operators consume, so its
observable behaviour — which ids come out, in which order — is kept identical
to the reference (the golden traces under ``tests/golden`` were recorded from
the reference class).

Ids are handed out from the head of a free list that starts as ``range(n)``
and grows at the tail as requests are freed.  A block that is the *source* of
a swap still in flight is parked on a second list and only recycled after the
workers confirmed that every swap in that direction has finished
(distserve/block_manager.py:66-98, design note 211-286).
"""
from __future__ import annotations

from enum import Enum
from typing import Callable, Dict, List

from .config import CacheConfig, KVModelConfig, ParallelConfig


class BlockLocation(Enum):
    GPU = "gpu"
    CPU = "cpu"


class _IdPool:
    """Free ids plus ids whose outbound copy may still be running."""

    def __init__(self, capacity: int, flush_method: str, where: str) -> None:
        self.capacity = capacity
        self.free: List[int] = list(range(capacity))
        self.parked: List[int] = []
        self.flush_method = flush_method   # worker method that drains the copies reading `parked`
        self.where = where

    def available(self) -> int:
        return len(self.free) + len(self.parked)

    def take(self, count: int, call_all_workers: Callable) -> List[int]:
        have = self.available()
        assert have >= count, f"not enough free blocks on {self.where}, requested {count}, available {have}"
        if len(self.free) < count:
            call_all_workers(self.flush_method)
            self.free.extend(self.parked)
            self.parked = []
        taken = self.free[:count]
        del self.free[:count]      # in place: the list can be as long as the pool
        return taken

    def used(self) -> int:
        return self.capacity - self.available()


class BlockManager:
    def __init__(self, stage, max_num_gpu_blocks: int, max_num_cpu_blocks: int, model_config: KVModelConfig,
                 parallel_config: ParallelConfig, cache_config: CacheConfig,
                 engine_remote_call_all_workers_async: Callable) -> None:
        self.stage = stage
        self.max_num_gpu_blocks = max_num_gpu_blocks
        self.max_num_cpu_blocks = max_num_cpu_blocks
        self.model_config = model_config
        self.parallel_config = parallel_config
        self.cache_config = cache_config
        self.engine_remote_call_all_workers_async = engine_remote_call_all_workers_async
        # A GPU block is parked while it is being swapped *out*; a host block while swapped *in*.
        self._pools = {
            BlockLocation.GPU: _IdPool(max_num_gpu_blocks, "wait_for_all_swap_out", "GPU"),
            BlockLocation.CPU: _IdPool(max_num_cpu_blocks, "wait_for_all_swap_in", "CPU"),
        }
        self.block_table: Dict[int, List[int]] = {}
        self.request_location: Dict[int, BlockLocation] = {}

    # --- views with the reference's attribute names -------------------------------------
    @property
    def free_gpu_blocks_list(self) -> List[int]:
        return self._pools[BlockLocation.GPU].free

    @property
    def free_cpu_blocks_list(self) -> List[int]:
        return self._pools[BlockLocation.CPU].free

    @property
    def swapping_gpu_blocks_list(self) -> List[int]:
        return self._pools[BlockLocation.GPU].parked

    @property
    def swapping_cpu_blocks_list(self) -> List[int]:
        return self._pools[BlockLocation.CPU].parked

    def get_num_avail_gpu_blocks(self) -> int:
        return self._pools[BlockLocation.GPU].available()

    def get_num_avail_cpu_blocks(self) -> int:
        return self._pools[BlockLocation.CPU].available()

    def _get_free_blocks(self, num_blocks: int, location: BlockLocation) -> List[int]:
        return self._pools[location].take(num_blocks, self.engine_remote_call_all_workers_async)

    # --- allocation ---------------------------------------------------------------------
    def get_allocated_num_blocks(self, request_id: int) -> int:
        return len(self.block_table.get(request_id, []))

    def get_location(self, request_id: int):
        return self.request_location.get(request_id, None)

    def get_num_blocks_needed(self, request) -> int:
        tokens = request.get_input_len() + request.get_output_len()
        return -(-tokens // self.cache_config.block_size)

    def get_num_append_blocks_needed(self, request) -> int:
        rid = request.request_id
        assert self.request_location[rid] == BlockLocation.GPU, \
            f"request {rid} is not on GPU when calling get_num_append_blocks_needed"
        return self.get_num_blocks_needed(request) - len(self.block_table[rid])

    def allocate_blocks(self, request) -> None:
        rid = request.request_id
        assert rid not in self.block_table or self.request_location.get(rid) == BlockLocation.GPU, \
            f"request {rid} is currently on CPU. Please migrate it to GPU before allocating more blocks"
        want = self.get_num_blocks_needed(request)
        held = self.block_table.get(rid)
        if held is None:
            self.block_table[rid] = self._get_free_blocks(want, BlockLocation.GPU)
            self.request_location[rid] = BlockLocation.GPU
        elif len(held) < want:
            held += self._get_free_blocks(want - len(held), BlockLocation.GPU)

    def allocate_blocks_batched(self, batch_requests) -> None:
        for request in batch_requests.requests:
            self.allocate_blocks(request)

    def free_blocks(self, request_id: int) -> None:
        assert request_id in self.block_table, f"request {request_id} not allocated"
        self._pools[self.request_location.pop(request_id)].free.extend(self.block_table.pop(request_id))

    def free_blocks_batched(self, requests) -> None:
        for request in requests:
            self.free_blocks(request.request_id)

    def get_block_table(self, request_id: int) -> List[int]:
        assert request_id in self.block_table, f"request {request_id} not allocated"
        return self.block_table[request_id]

    def get_partial_block_table(self, request_ids: List[int]) -> List[List[int]]:
        return [self.get_block_table(rid) for rid in request_ids]

    # --- swapping -----------------------------------------------------------------------
    def swap_requests(self, requests, is_swap_in: bool) -> None:
        """Move the requests' blocks to the other location.  New ids are taken
        there, the old ids are parked, and one ``swap_blocks`` call carrying
        the concatenated lists goes to every worker without being awaited
        (distserve/block_manager.py:288-315)."""
        here = BlockLocation.CPU if is_swap_in else BlockLocation.GPU
        there = BlockLocation.GPU if is_swap_in else BlockLocation.CPU
        source_block_ids: List[int] = []
        target_block_ids: List[int] = []
        for request in requests:
            rid = request.request_id
            assert rid in self.block_table, f"request {rid} not allocated"
            assert self.request_location[rid] == here, f"request {rid} is on {there} now"
            old = self.block_table[rid]
            new = self._get_free_blocks(len(old), there)
            source_block_ids += old
            target_block_ids += new
            self.block_table[rid] = new
            self.request_location[rid] = there
            self._pools[here].parked.extend(old)
        self.engine_remote_call_all_workers_async("swap_blocks", requests, source_block_ids, target_block_ids, is_swap_in)

    def swap_in_requests(self, requests) -> None:
        self.swap_requests(requests, is_swap_in=True)

    def swap_out_requests(self, requests) -> None:
        self.swap_requests(requests, is_swap_in=False)

    def is_all_requests_on_gpu(self, requests) -> bool:
        return all(self.request_location[r.request_id] != BlockLocation.CPU for r in requests.requests)

    def usage(self) -> Dict[str, int]:
        g, c = self._pools[BlockLocation.GPU], self._pools[BlockLocation.CPU]
        return {"gpu_used": g.used(), "gpu_swapping_out": len(g.parked), "cpu_used": c.used(), "cpu_swapping_in": len(c.parked)}

    def __repr__(self) -> str:
        return (f"BlockManager(max_num_gpu_blocks={self.max_num_gpu_blocks}, "
                f"max_num_cpu_blocks={self.max_num_cpu_blocks}, blocksize={self.cache_config.block_size})")

"""The KV-cache half of a stage worker: the mirror of the methods of
``distserve/worker.py``'s ParaWorker that own the K/V pools, export and
register their handles, migrate blocks and swap them (101-134, 229-334).
Method names, argument order and meaning follow the reference, so that code
written against ParaWorker's KV methods runs against this class.  The model
forward, Ray and weight loading are not part of this path.

Calls go through ``torch.ops.block_migration_ops.*`` / ``torch.ops.swapping_ops.swap``
— the operator names the reference resolves from its native library — which
this package's shim registers.  Without the built libraries or without a CUDA
device construction fails; there is no CPU fallback.

Deliberate differences from the reference worker, all in the swap event
protocol (design note at distserve/block_manager.py:211-286):
* swap events are numbered per direction and the highest finished number is
  remembered, so waits on swaps already known to be over are skipped — the
  optimisation the note leaves for later (277-285);
* the per-request event is recorded *after* the copies are enqueued, so that
  waiting on it really waits for them (the reference records it before,
  distserve/worker.py:286-287 vs 302-311);
* request ids are normalised, so the Request objects that BlockManager passes
  (distserve/block_manager.py:313-315) and the integer ids that ``step`` looks
  up (distserve/worker.py:205-211) meet in the same table.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from . import capi, load_ops
from .config import CacheConfig, KVModelConfig, ParallelConfig

cudaMemoryIpcHandle = List[int]


def _request_id(item) -> int:
    return item if isinstance(item, int) else item.request_id


class _SwapMark:
    """The event recorded after a swap, numbered within its direction.  Swaps of one direction run in
    order on one stream, so once mark n is known to have completed, every mark <= n has too — the
    shortcut the reference's design note proposes (distserve/block_manager.py:277-285)."""

    __slots__ = ("event", "seq", "is_swap_in")

    def __init__(self, event, seq: int, is_swap_in: bool) -> None:
        self.event, self.seq, self.is_swap_in = event, seq, is_swap_in


class KVWorker:
    def __init__(self, worker_id: int, stage, model_config: KVModelConfig, cache_config: CacheConfig,
                 parallel_config: ParallelConfig = ParallelConfig(), device: Optional[int] = None) -> None:
        if not torch.cuda.is_available():
            raise RuntimeError("KVWorker needs a CUDA device; there is no CPU implementation of this path")
        load_ops()
        self.worker_id = worker_id
        self.stage = stage
        self.model_config = model_config
        self.cache_config = cache_config
        self.parallel_config = parallel_config
        # The reference worker always sees its GPU as cuda:0 (distserve/worker.py:53-56);
        # a test process that hosts several workers passes the ordinal instead.
        self.device = torch.device("cuda", torch.cuda.current_device() if device is None else device)
        self.k_cache = self.v_cache = None
        self.k_swap = self.v_swap = None
        with torch.cuda.device(self.device):
            self.swap_in_stream = torch.cuda.Stream()
            self.swap_out_stream = torch.cuda.Stream()
        self.swap_event_table: Dict[int, _SwapMark] = {}
        self.latest_swap_in_event: Optional[torch.cuda.Event] = None
        self.latest_swap_out_event: Optional[torch.cuda.Event] = None
        self._swaps_issued = {True: 0, False: 0}        # per direction (is_swap_in)
        self._swaps_known_done = {True: 0, False: 0}    # highest mark known to have completed
        self.blocked_swapping_time = 0.0
        self._bind_migrate_op()

    # --- pools and handles ---------------------------------------------------------------
    def kv_cache_shape(self, num_blocks: int) -> Tuple[int, int, int, int, int]:
        return (num_blocks, self.model_config.get_num_layers(self.parallel_config),
                self.model_config.get_num_heads(self.parallel_config), self.cache_config.block_size,
                self.model_config.get_head_size())

    def init_kvcache_and_swap(self, num_gpu_blocks: int, num_cpu_blocks: int) -> Tuple[cudaMemoryIpcHandle, cudaMemoryIpcHandle]:
        """Allocate the GPU pools and the pinned host pools, return the K and V
        pool handles (distserve/worker.py:101-134)."""
        dtype = self.model_config.get_torch_dtype()
        with torch.cuda.device(self.device):
            self.k_cache = torch.empty(self.kv_cache_shape(num_gpu_blocks), dtype=dtype, device=self.device)
            self.v_cache = torch.empty(self.kv_cache_shape(num_gpu_blocks), dtype=dtype, device=self.device)
            self.k_swap = torch.empty(self.kv_cache_shape(num_cpu_blocks), dtype=dtype, device="cpu", pin_memory=True)
            self.v_swap = torch.empty(self.kv_cache_shape(num_cpu_blocks), dtype=dtype, device="cpu", pin_memory=True)
            torch.cuda.synchronize(self.device)
            return (torch.ops.block_migration_ops.get_ipc_mem_handle(self.k_cache),
                    torch.ops.block_migration_ops.get_ipc_mem_handle(self.v_cache))

    def register_kvcache_mem_handles(self, context_parallel_config: ParallelConfig,
                                     kvcache_ipc_mem_handles: Sequence[Sequence[Tuple[cudaMemoryIpcHandle, cudaMemoryIpcHandle]]]) -> None:
        """Register every context worker's pools; the table is indexed
        [pp_rank][tp_rank] -> (k_handle, v_handle) (distserve/worker.py:229-248)."""
        with torch.cuda.device(self.device):
            for pp_rank, stage_workers in enumerate(kvcache_ipc_mem_handles):
                for tp_rank, (k_handle, v_handle) in enumerate(stage_workers):
                    owner = context_parallel_config.with_rank(pp_rank, tp_rank)
                    torch.ops.block_migration_ops.register_ipc_mem_handle(
                        list(k_handle), list(v_handle),
                        self.model_config.get_num_layers(), self.model_config.get_num_heads(),
                        owner.to_list(), self.parallel_config.to_list())
            torch.cuda.synchronize(self.device)

    # --- migration -----------------------------------------------------------------------
    def _bind_migrate_op(self):
        """Resolve, once, the operator object and this worker's own layout in the operator's argument order
        (the lookup through ``torch.ops`` and the overload choice are host time on every request otherwise)."""
        packet = torch.ops.block_migration_ops.migrate_blocks
        self._migrate_op = getattr(packet, "default", packet)
        pc = self.parallel_config
        self._own_layout = (pc.pipeline_parallel_size, pc.tensor_parallel_size, pc.pipeline_parallel_rank,
                            pc.tensor_parallel_rank)
        return self._migrate_op

    def migrate_blocks(self, context_block_indexes: List[int], context_parallel_config: ParallelConfig,
                       decoding_block_indexes: List[int]) -> None:
        """Pull the listed context-stage blocks into this worker's pools
        (distserve/worker.py:250-267).  Returns when the sources have been read.  The operator itself
        makes the pools' device current for the call and launches on that device's current stream."""
        op = getattr(self, "_migrate_op", None) or self._bind_migrate_op()
        pp, tp, pp_rank, tp_rank = self._own_layout
        op(context_parallel_config.pipeline_parallel_size, context_parallel_config.tensor_parallel_size,
           context_block_indexes, pp, tp, pp_rank, tp_rank, decoding_block_indexes, self.k_cache, self.v_cache)

    def _pool_shape(self) -> capi.PoolShape:
        """The pools' shape as the C ABI takes it; built once per pool (the pools live as long as the worker)."""
        cached = getattr(self, "_shape_of_pool", None)
        if cached is None or cached[0] is not self.k_cache:
            cached = (self.k_cache, capi.PoolShape.of(*self.k_cache.shape, self.k_cache.element_size()))
            self._shape_of_pool = cached
        return cached[1]

    def migrate_blocks_async(self, context_block_indexes: List[int], context_parallel_config: ParallelConfig,
                             decoding_block_indexes: List[int], stream: Optional[torch.cuda.Stream] = None) -> int:
        """Enqueue the same copy on `stream` (default: the current stream)
        and return a ticket for :meth:`migrate_wait`.  The lists may hold the
        concatenated block tables of several requests."""
        with torch.cuda.device(self.device):
            s = stream if stream is not None else torch.cuda.current_stream()
            pc = self.parallel_config
            return capi.migrate_blocks_async(
                context_parallel_config.pipeline_parallel_size, context_parallel_config.tensor_parallel_size,
                context_block_indexes, pc.pipeline_parallel_size, pc.tensor_parallel_size,
                pc.pipeline_parallel_rank, pc.tensor_parallel_rank, decoding_block_indexes,
                self.k_cache.data_ptr(), self.v_cache.data_ptr(), self._pool_shape(), s.cuda_stream)

    def migrate_layers_async(self, context_block_indexes: List[int], context_parallel_config: ParallelConfig,
                             decoding_block_indexes: List[int], layer_begin: int, layer_end: int,
                             stream: Optional[torch.cuda.Stream] = None) -> int:
        """Enqueue the copy of the global layers [layer_begin, layer_end) only (the part this worker
        holds), for a context stage that releases a request's KV layer by layer while prefill runs."""
        with torch.cuda.device(self.device):
            s = stream if stream is not None else torch.cuda.current_stream()
            pc = self.parallel_config
            return capi.migrate_layers_async(
                context_parallel_config.pipeline_parallel_size, context_parallel_config.tensor_parallel_size,
                context_block_indexes, pc.pipeline_parallel_size, pc.tensor_parallel_size,
                pc.pipeline_parallel_rank, pc.tensor_parallel_rank, decoding_block_indexes,
                self.k_cache.data_ptr(), self.v_cache.data_ptr(), self._pool_shape(), layer_begin, layer_end, s.cuda_stream)

    def migrate_wait(self, ticket: int) -> None:
        capi.migrate_wait(ticket)

    # --- swapping ------------------------------------------------------------------------
    def swap_blocks(self, request_ids: Iterable, source_block_ids: List[int], target_block_ids: List[int],
                    is_swap_in: bool) -> None:
        """Copy host block source[i] -> GPU block target[i] (swap in) or the
        other way round (swap out) on the direction's own stream
        (distserve/worker.py:269-311)."""
        ids = [_request_id(r) for r in request_ids]
        with torch.cuda.device(self.device):
            stream = self.swap_in_stream if is_swap_in else self.swap_out_stream
            # The blocks may have been written by work still queued on the caller's stream.
            stream.wait_stream(torch.cuda.current_stream())
            for rid in ids:
                earlier = self.swap_event_table.get(rid)
                if earlier is not None and not self._swap_done(earlier):
                    earlier.event.wait(stream)
            with torch.cuda.stream(stream):
                torch.ops.swapping_ops.swap(source_block_ids, target_block_ids, is_swap_in,
                                            self.k_cache, self.v_cache, self.k_swap, self.v_swap)
            event = torch.cuda.Event()
            event.record(stream)
            self._swaps_issued[is_swap_in] += 1
            mark = _SwapMark(event, self._swaps_issued[is_swap_in], is_swap_in)
            for rid in ids:
                self.swap_event_table[rid] = mark
            if is_swap_in:
                self.latest_swap_in_event = event
            else:
                self.latest_swap_out_event = event

    def _swap_done(self, mark: _SwapMark) -> bool:
        """True if the swap behind `mark` has finished; remembers the highest finished mark per direction so
        that later questions about older swaps need no CUDA call at all."""
        if mark.seq <= self._swaps_known_done[mark.is_swap_in]:
            return True
        if mark.event.query():
            self._swaps_known_done[mark.is_swap_in] = mark.seq
            return True
        return False

    def swap_finished(self, request_id) -> bool:
        """Has the last swap of this request completed (or was there none)?  Lets a scheduler put a
        swapped-in request back into the batch only when that costs the step nothing."""
        mark = self.swap_event_table.get(_request_id(request_id))
        return mark is None or self._swap_done(mark)

    def prepare_step(self, request_ids: Iterable[int]) -> None:
        """What ``step`` does before the forward (distserve/worker.py:205-211):
        the compute stream waits for the last swap of each request in the batch."""
        with torch.cuda.device(self.device):
            current = torch.cuda.current_stream()
            for rid in request_ids:
                mark = self.swap_event_table.pop(_request_id(rid), None)
                if mark is not None and not self._swap_done(mark):
                    mark.event.wait(current)

    def clear_request_resource(self, request_id: int) -> None:
        self.swap_event_table.pop(request_id, None)

    def clear_request_resource_batched(self, requests) -> None:
        for request in requests:
            self.clear_request_resource(_request_id(request))

    def wait_for_all_swap_in(self) -> None:
        if self.latest_swap_in_event is not None:
            self.latest_swap_in_event.synchronize()
            self.latest_swap_in_event = None
            self._swaps_known_done[True] = self._swaps_issued[True]

    def wait_for_all_swap_out(self) -> None:
        if self.latest_swap_out_event is not None:
            self.latest_swap_out_event.synchronize()
            self.latest_swap_out_event = None
            self._swaps_known_done[False] = self._swaps_issued[False]


# Same name as the reference class for code written against it.
ParaWorker = KVWorker

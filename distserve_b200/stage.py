"""The callers of the migration path, reduced to what drives it: the parts of
``distserve/single_stage_engine.py`` that create the pools, hand the context
stage's handles to the decoding stage and migrate one request
(_init_kvcache 194-223, register_kvcache_mem_handles 469-483, _migrate_blocks
490-536, clear_migrated_blocks_callback 405-410).

Workers are any objects with KVWorker's method names: local ``KVWorker``
instances, or ``actors.ActorHandle`` proxies of workers living in their own
processes, whose calls return futures (the stand-in for the reference's Ray
actor handles).
"""
from __future__ import annotations

import time
from typing import Callable, Dict, List, Optional, Sequence, Tuple

from .block_manager import BlockManager
from .config import CacheConfig, KVModelConfig, ParallelConfig
from .request import MigratingRequest, Request

Handles = List[List[Tuple[List[int], List[int]]]]


def _resolve(results: Sequence):
    return [r.result() if hasattr(r, "result") else r for r in results]


class StageEngine:
    """One stage: a [pp][tp] grid of workers plus the stage's block manager."""

    def __init__(self, stage: str, model_config: KVModelConfig, parallel_config: ParallelConfig,
                 cache_config: CacheConfig, workers: Sequence[Sequence[object]]) -> None:
        assert len(workers) == parallel_config.pipeline_parallel_size
        assert all(len(row) == parallel_config.tensor_parallel_size for row in workers)
        self.stage = stage
        self.model_config = model_config
        self.parallel_config = parallel_config
        self.cache_config = cache_config
        self.workers = [list(row) for row in workers]
        self.block_manager: Optional[BlockManager] = None
        self.kv_cache_mem_handles: Handles = []

    def _remote_call_all_workers_async(self, func_name: str, *args) -> List:
        """Issue `func_name` on every worker, pipeline-major, and return what
        the calls returned (futures for remote workers) without waiting."""
        return [getattr(worker, func_name)(*args) for row in self.workers for worker in row]

    def init_kvcache(self, num_gpu_blocks: int, num_cpu_blocks: int) -> Handles:
        """Allocate every worker's pools and arrange the returned handles as
        [pp_rank][tp_rank] -> (k_handle, v_handle)."""
        flat = _resolve(self._remote_call_all_workers_async("init_kvcache_and_swap", num_gpu_blocks, num_cpu_blocks))
        tp = self.parallel_config.tensor_parallel_size
        self.kv_cache_mem_handles = [flat[i * tp:(i + 1) * tp] for i in range(self.parallel_config.pipeline_parallel_size)]
        self.block_manager = BlockManager(self.stage, num_gpu_blocks, num_cpu_blocks, self.model_config,
                                          self.parallel_config, self.cache_config, self._remote_call_all_workers_async)
        return self.kv_cache_mem_handles


class ContextStageEngine(StageEngine):
    def __init__(self, *args, **kwargs) -> None:
        super().__init__("context", *args, **kwargs)

    def finish_prefill(self, request: Request) -> MigratingRequest:
        """Allocate the prompt's blocks (the prefill forward itself is outside
        this path) and describe them for the bridge queue.  The blocks stay
        allocated until the decoding stage has pulled them."""
        self.block_manager.allocate_blocks(request)
        return MigratingRequest(request, list(self.block_manager.get_block_table(request.request_id)), self.parallel_config)

    def clear_migrated_blocks(self, migrating_req: MigratingRequest) -> None:
        self.block_manager.free_blocks(migrating_req.req.request_id)


class PendingMigration:
    """A group of requests whose copy has been enqueued on every decoding worker but not awaited yet."""

    __slots__ = ("requests", "workers", "tickets", "targets")

    def __init__(self, requests, workers, tickets, targets) -> None:
        self.requests, self.workers, self.tickets, self.targets = requests, workers, tickets, targets

    def num_blocks(self) -> int:
        return sum(len(t) for t in self.targets)


class DecodingStageEngine(StageEngine):
    def __init__(self, *args, clear_migrated_blocks_callback: Optional[Callable[[MigratingRequest], None]] = None,
                 **kwargs) -> None:
        super().__init__("decoding", *args, **kwargs)
        self.clear_migrated_blocks_callback = clear_migrated_blocks_callback
        self.lifetime_events: Dict[int, List[Tuple[str, float]]] = {}

    def register_kvcache_mem_handles(self, context_parallel_config: ParallelConfig, kv_cache_mem_handles: Handles) -> None:
        _resolve(self._remote_call_all_workers_async("register_kvcache_mem_handles", context_parallel_config,
                                                     kv_cache_mem_handles))

    def _stamp(self, request_id: int, name: str) -> None:
        self.lifetime_events.setdefault(request_id, []).append((name, time.time()))

    def migrate_blocks(self, migrating_req: MigratingRequest) -> List[int]:
        """Accept one request: reserve blocks for its prompt only, have every
        decoding worker pull its share, then let the context stage recycle the
        source blocks.  Returns the target block ids."""
        req = migrating_req.req
        # Tokens generated by the prefill step must not count towards the reservation.
        kept_ids, kept_tokens = req.generated_token_ids, req.generated_tokens
        req.generated_token_ids, req.generated_tokens = [], []
        try:
            self.block_manager.allocate_blocks(req)
        finally:
            req.generated_token_ids, req.generated_tokens = kept_ids, kept_tokens
        target = self.block_manager.get_block_table(req.request_id)
        assert len(target) == len(migrating_req.block_indexes)
        self._stamp(req.request_id, "migration_begin")
        _resolve(self._remote_call_all_workers_async("migrate_blocks", migrating_req.block_indexes,
                                                     migrating_req.context_parallel_config, target))
        self._stamp(req.request_id, "migration_end")
        if self.clear_migrated_blocks_callback is not None:
            self.clear_migrated_blocks_callback(migrating_req)
        return target

    def migrate_blocks_batched(self, migrating_reqs: Sequence[MigratingRequest]) -> List[List[int]]:
        """Accept several requests with ONE launch per decoding worker: their block tables are concatenated
        and handed to ``migrate_blocks_async``.  The reference accepts requests one awaited call at a time
        (distserve/decoding_stage_scheduler.py:247-260); for short prompts that cadence is bound by the
        launch-and-await round trip, which this removes.  Returns each request's target block ids."""
        if not migrating_reqs:
            return []
        return self.finish_migrate_blocks_batched(self.begin_migrate_blocks_batched(migrating_reqs))

    def begin_migrate_blocks_batched(self, migrating_reqs: Sequence[MigratingRequest]) -> "PendingMigration":
        """First half of :meth:`migrate_blocks_batched`: reserve the target blocks and enqueue the copy on every
        decoding worker, without waiting for it.  The caller may go on with host work (or enqueue the next
        group) and must call :meth:`finish_migrate_blocks_batched` before the requests join a batch; the
        context stage's blocks are released only there."""
        ctx_pc = migrating_reqs[0].context_parallel_config
        assert all(m.context_parallel_config.to_list()[::2] == ctx_pc.to_list()[::2] for m in migrating_reqs), \
            "requests of one batch must come from the same context stage layout"
        sources: List[int] = []
        targets: List[int] = []
        per_request: List[List[int]] = []
        for m in migrating_reqs:
            req = m.req
            kept_ids, kept_tokens = req.generated_token_ids, req.generated_tokens
            req.generated_token_ids, req.generated_tokens = [], []
            try:
                self.block_manager.allocate_blocks(req)
            finally:
                req.generated_token_ids, req.generated_tokens = kept_ids, kept_tokens
            target = list(self.block_manager.get_block_table(req.request_id))
            assert len(target) == len(m.block_indexes)
            per_request.append(target)
            sources += m.block_indexes
            targets += target
            self._stamp(req.request_id, "migration_begin")
        workers = [worker for row in self.workers for worker in row]
        tickets = [worker.migrate_blocks_async(sources, ctx_pc, targets) for worker in workers]
        return PendingMigration(list(migrating_reqs), workers, tickets, per_request)

    def finish_migrate_blocks_batched(self, pending: "PendingMigration") -> List[List[int]]:
        """Second half: wait until every worker has read the sources, then let the context stage recycle them."""
        tickets = _resolve(pending.tickets)
        _resolve([worker.migrate_wait(ticket) for worker, ticket in zip(pending.workers, tickets)])
        for m in pending.requests:
            self._stamp(m.req.request_id, "migration_end")
            if self.clear_migrated_blocks_callback is not None:
                self.clear_migrated_blocks_callback(m)
        return pending.targets

    def migration_latency(self, request_id: int) -> float:
        """Seconds between the two stamps, the reference's definition of the
        transfer time of a request."""
        events = dict(self.lifetime_events[request_id])
        return events["migration_end"] - events["migration_begin"]

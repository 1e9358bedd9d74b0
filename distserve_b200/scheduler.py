"""The decoding stage's first-come-first-served scheduler: the mirror of
``distserve/decoding_stage_scheduler.py`` (DecodingStageFCFSScheduler 92-260),
the component that decides *when* blocks migrate (``post_process``) and when
requests are swapped out and in (``get_next_batch``).  Its decisions are kept
identical to the reference's (replayed against a trace recorded from the
reference class, tests/golden/scheduler.json); what is added is
``post_process_batched``, which accepts the same requests as ``post_process``
but moves them with one launch per decoding worker.

Three queues, as in the reference: requests still sitting in the context
stage's pools (``unaccepted_queue``), requests whose blocks have arrived but
which are not in a batch yet (``waiting_queue``), and requests swapped out to
host memory (``swapped_queue``); plus one running batch per pipeline stage.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

from .block_manager import BlockManager
from .config import ParallelConfig
from .request import BatchedRequests, MigratingRequest, Request


@dataclass
class DecodingStageSchedConfig:
    """distserve/config.py DecodingStageSchedConfig."""

    policy: str = "fcfs"
    max_batch_size: int = 256
    max_tokens_per_batch: int = 8192
    waiting_block_prop_threshold: float = 0.05


class DecodingStageFCFSScheduler:
    def __init__(self, sched_config: DecodingStageSchedConfig, parallel_config: ParallelConfig, block_manager: BlockManager,
                 engine_migrate_block_callback: Callable[[MigratingRequest], object],
                 engine_migrate_blocks_batched_callback: Optional[Callable[[Sequence[MigratingRequest]], object]] = None,
                 engine_begin_migration_callback: Optional[Callable[[Sequence[MigratingRequest]], object]] = None,
                 engine_finish_migration_callback: Optional[Callable[[object], object]] = None) -> None:
        assert sched_config.policy == "fcfs", f"can not initialize a FCFS scheduler with policy {sched_config.policy}"
        self.sched_config = sched_config
        self.parallel_config = parallel_config
        self.block_manager = block_manager
        self.engine_migrate_block_callback = engine_migrate_block_callback
        self.engine_migrate_blocks_batched_callback = engine_migrate_blocks_batched_callback
        self.engine_begin_migration_callback = engine_begin_migration_callback
        self.engine_finish_migration_callback = engine_finish_migration_callback
        self._in_flight = None        # (pending migration, its requests) enqueued by post_process_pipelined
        self.unaccepted_queue: List[MigratingRequest] = []
        self.waiting_queue: List[Request] = []
        self.swapped_queue: List[Request] = []
        self.cur_index = -1
        self.batch_queues = [BatchedRequests() for _ in range(parallel_config.pipeline_parallel_size)]

    # --- block arithmetic ---------------------------------------------------------------
    def _blocks(self, num_tokens: int) -> int:
        return -(-num_tokens // self.block_manager.cache_config.block_size)

    def _running_blocks(self) -> int:
        """Blocks the running batches need for everything they have produced so far."""
        return sum(self._blocks(r.get_input_len() + r.get_output_len()) for batch in self.batch_queues for r in batch.requests)

    def _waiting_blocks(self) -> int:
        """Blocks the accepted-but-not-running requests hold (their prompts)."""
        return sum(self._blocks(r.get_input_len()) for r in self.waiting_queue)

    def _fits_current_batch(self, request: Request, running: Optional[int] = None, waiting: Optional[int] = None,
                            batch_tokens: Optional[int] = None) -> bool:
        """The reference's admission rule (distserve/decoding_stage_scheduler.py:155-181).  The three totals may be
        handed in by a caller that keeps them up to date while it moves requests; otherwise they are recomputed."""
        batch = self.batch_queues[self.cur_index]
        running = self._running_blocks() if running is None else running
        waiting = self._waiting_blocks() if waiting is None else waiting
        batch_tokens = batch.get_num_input_tokens() if batch_tokens is None else batch_tokens
        return (len(batch) < self.sched_config.max_batch_size
                and batch_tokens + request.get_num_input_tokens() <= self.sched_config.max_tokens_per_batch
                and running + waiting + self._blocks(request.get_input_len() + request.get_output_len())
                <= self.block_manager.max_num_gpu_blocks)

    # --- requests -----------------------------------------------------------------------
    def add_request(self, migrating_req: MigratingRequest) -> None:
        self.unaccepted_queue.append(migrating_req)

    def abort_request(self, request_id: int) -> None:
        for batch in self.batch_queues:
            for request in batch.requests:
                if request.request_id == request_id:
                    request.is_finished = True      # may be executing: let the normal path release it
                    return
        self.waiting_queue = [r for r in self.waiting_queue if r.request_id != request_id]

    def pop_finished_requests(self) -> List[Request]:
        last_stage = (self.cur_index + 1) % self.parallel_config.pipeline_parallel_size
        return self.batch_queues[last_stage].pop_finished_requests()

    # --- one iteration ------------------------------------------------------------------
    def get_next_batch(self) -> BatchedRequests:
        self.cur_index = (self.cur_index + 1) % self.parallel_config.pipeline_parallel_size
        batch = self.batch_queues[self.cur_index]
        # The block and token totals the rules below look at are summed once and then kept up to date as requests
        # move between the queues (the sums run over every running request; recomputing them per candidate is what
        # makes an iteration's host time grow with the batch).
        running, waiting, tokens = self._running_blocks(), self._waiting_blocks(), batch.get_num_input_tokens()
        # Not enough GPU blocks for what is running and waiting: swap out the newest member of this batch.
        while running + waiting > self.block_manager.max_num_gpu_blocks:
            victim = batch.requests.pop(-1)
            running -= self._blocks(victim.get_input_len() + victim.get_output_len())
            tokens -= victim.get_num_input_tokens()
            self.swapped_queue.append(victim)
            self.block_manager.swap_out_requests([victim])
        # Refill: swapped-out requests first, then waiting ones, each only while it fits.
        while self.swapped_queue or self.waiting_queue:
            from_swapped = bool(self.swapped_queue)
            request = self.swapped_queue[0] if from_swapped else self.waiting_queue[0]
            if not self._fits_current_batch(request, running, waiting, tokens):
                break
            if from_swapped:
                self.block_manager.swap_in_requests([request])
                self.swapped_queue.pop(0)
            else:
                self.waiting_queue.pop(0)
                waiting -= self._blocks(request.get_input_len())
            batch.add_request(request)
            running += self._blocks(request.get_input_len() + request.get_output_len())
            tokens += request.get_num_input_tokens()
        return batch

    def _should_accept(self, prompt_len: int, waiting_blocks: int, avail_blocks: int) -> bool:
        return (waiting_blocks < self.block_manager.max_num_gpu_blocks * self.sched_config.waiting_block_prop_threshold
                and self._blocks(prompt_len) <= avail_blocks)

    def post_process(self) -> List[int]:
        """After an iteration: accept requests from the head of the unaccepted queue while the waiting queue is
        short and blocks are free, migrating each with its own awaited call (the reference's cadence).  Returns
        the accepted request ids."""
        accepted = []
        while self.unaccepted_queue:
            m = self.unaccepted_queue[0]
            if not self._should_accept(m.req.get_input_len(), self._waiting_blocks(), self.block_manager.get_num_avail_gpu_blocks()):
                break
            self.unaccepted_queue.pop(0)
            self.engine_migrate_block_callback(m)
            self.waiting_queue.append(m.req)
            accepted.append(m.req.request_id)
        return accepted

    def post_process_batched(self) -> List[int]:
        """Same acceptance rule, evaluated on the state each earlier acceptance would have left, but all
        accepted requests migrate together (one launch per decoding worker)."""
        if self.engine_migrate_blocks_batched_callback is None:
            return self.post_process()
        chosen = self._choose_acceptable(self._waiting_blocks(), self.block_manager.get_num_avail_gpu_blocks())
        if chosen:
            del self.unaccepted_queue[:len(chosen)]
            self.engine_migrate_blocks_batched_callback(chosen)
            self.waiting_queue.extend(m.req for m in chosen)
        return [m.req.request_id for m in chosen]

    def _choose_acceptable(self, waiting: int, avail: int) -> List[MigratingRequest]:
        chosen: List[MigratingRequest] = []
        for m in self.unaccepted_queue:
            n = m.req.get_input_len()
            if not self._should_accept(n, waiting, avail):
                break
            chosen.append(m)
            waiting += self._blocks(n)
            avail -= self._blocks(n)
        return chosen

    def post_process_pipelined(self) -> List[int]:
        """``post_process_batched`` with one group of requests in flight: the group accepted now is enqueued on
        the workers first, and only then is the group enqueued by the previous call awaited, so the host work of
        an iteration (this acceptance included) runs while the previous group's copy is on the wire.  Requests
        join the waiting queue when their own copy has finished, i.e. one call later than with
        ``post_process_batched``.  The group in flight already holds its target blocks, so it counts against the
        free blocks of the acceptance rule; it does not count against the waiting-queue threshold, because in the
        unpipelined flow it would have moved from the waiting queue into a batch by now.  Returns the ids of the
        requests that became ready in this call."""
        if self.engine_begin_migration_callback is None or self.engine_finish_migration_callback is None:
            return self.post_process_batched()
        chosen = self._choose_acceptable(self._waiting_blocks(), self.block_manager.get_num_avail_gpu_blocks())
        started = None
        if chosen:
            del self.unaccepted_queue[:len(chosen)]
            started = (self.engine_begin_migration_callback(chosen), chosen)
        ready = self.flush_pipeline()
        self._in_flight = started
        return ready

    def flush_pipeline(self) -> List[int]:
        """Await the group in flight, if any, and hand its requests to the waiting queue."""
        if self._in_flight is None:
            return []
        pending, group = self._in_flight
        self._in_flight = None
        self.engine_finish_migration_callback(pending)
        self.waiting_queue.extend(m.req for m in group)
        return [m.req.request_id for m in group]

    # --- counters -----------------------------------------------------------------------
    def get_processing_num_requests(self) -> int:
        return sum(len(b) for b in self.batch_queues)

    def get_waiting_num_requests(self) -> int:
        return len(self.waiting_queue)

    def get_total_num_requests(self) -> int:
        return self.get_processing_num_requests() + self.get_waiting_num_requests()

    def __repr__(self) -> str:
        return (f"FCFS(max_batch_size={self.sched_config.max_batch_size}, "
                f"max_tokens_per_batch={self.sched_config.max_tokens_per_batch})")


@dataclass
class ContextStageSchedConfig:
    """distserve/config.py ContextStageSchedConfig."""

    policy: str = "fcfs"
    max_batch_size: int = 256
    max_tokens_per_batch: int = 8192


class ContextStageFCFSScheduler:
    """The context stage's scheduler, mirror of ``distserve/context_stage_scheduler.py``
    (ContextStageFCFSScheduler 82-188).  Its tie to the migration path: a request that finished prefill keeps
    its blocks — and keeps counting against the block budget of new prefill batches — until the decoding
    stage has pulled them (``on_request_migrated``), so slow migration throttles prefill."""

    def __init__(self, sched_config: ContextStageSchedConfig, parallel_config: ParallelConfig, block_manager: BlockManager) -> None:
        assert sched_config.policy == "fcfs", f"can not initialize a FCFS scheduler with policy {sched_config.policy}"
        self.sched_config = sched_config
        self.parallel_config = parallel_config
        self.block_manager = block_manager
        self.waiting_queue: List[Request] = []
        self.unaccepted_queue: List[Request] = []      # prefill done, blocks not yet pulled by the decoding stage
        self.num_on_fly_request_block = 0              # blocks of the batches being prefilled right now

    def _blocks(self, num_tokens: int) -> int:
        return -(-num_tokens // self.block_manager.cache_config.block_size)

    def add_request(self, request: Request) -> None:
        self.waiting_queue.append(request)

    def abort_request(self, request_id: int) -> None:
        for i, request in enumerate(self.waiting_queue):
            if request.request_id == request_id:
                del self.waiting_queue[i]
                return

    def get_next_batch_and_pop(self) -> BatchedRequests:
        batch = BatchedRequests()
        held = sum(self._blocks(r.get_input_len()) for r in self.unaccepted_queue) + self.num_on_fly_request_block
        batch_blocks = 0
        while self.waiting_queue:
            request = self.waiting_queue[0]
            need = self._blocks(request.get_input_len())
            if not (len(batch) < self.sched_config.max_batch_size
                    and batch.get_num_input_tokens() + request.get_num_input_tokens() <= self.sched_config.max_tokens_per_batch
                    and batch_blocks + need + held <= self.block_manager.max_num_gpu_blocks):
                break
            batch.add_request(request)
            batch_blocks += need
            self.waiting_queue.pop(0)
        self.num_on_fly_request_block += batch_blocks
        return batch

    def on_finish_requests(self, batch: BatchedRequests) -> None:
        for request in batch.requests:
            if not request.is_finished:
                self.unaccepted_queue.append(request)
        self.num_on_fly_request_block -= sum(self._blocks(r.get_input_len()) for r in batch.requests)

    def on_request_migrated(self, migrated_request: MigratingRequest) -> None:
        for i, request in enumerate(self.unaccepted_queue):
            if request.request_id == migrated_request.req.request_id:
                del self.unaccepted_queue[i]
                return

    def get_num_waiting_requests(self) -> int:
        return len(self.waiting_queue)

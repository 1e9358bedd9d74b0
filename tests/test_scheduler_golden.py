"""The decoding-stage scheduler mirror replays, decision for decision, a trace
recorded from the reference scheduler (tests/golden/make_golden.py): which
requests run in each iteration, which are accepted (= migrated) afterwards,
and every swap-out / swap-in with its block ids.  The batched acceptance must
choose exactly the requests the one-by-one acceptance chooses."""
import json
import random

import pytest

from distserve_b200.block_manager import BlockManager
from distserve_b200.config import CacheConfig, KVModelConfig, ParallelConfig
from distserve_b200.request import MigratingRequest, Request
from distserve_b200.scheduler import DecodingStageFCFSScheduler, DecodingStageSchedConfig
from tests.test_golden_host import state_digest


def load(golden_dir):
    with open(golden_dir / "scheduler.json") as f:
        return json.load(f)


def simulate(sc, batched: bool):
    """The loop of DecodingStageLLMEngine._step around the scheduler, as the fixture's recorder runs it."""
    rng = random.Random(sc["seed"])
    block_size = sc["block_size"]
    swaps, migrated = [], []

    def record(name, *args):
        if name == "swap_blocks":
            reqs, src, dst, is_in = args
            swaps.append([[r.request_id for r in reqs], list(src), list(dst), bool(is_in)])

    pc = ParallelConfig()
    bm = BlockManager("decoding", sc["gpu_blocks"], sc["cpu_blocks"], KVModelConfig(12, 12, 64), pc, CacheConfig(block_size, 256), record)

    def migrate(m):
        req = m.req
        kept = (req.generated_tokens, req.generated_token_ids)
        req.generated_tokens, req.generated_token_ids = [], []
        bm.allocate_blocks(req)
        req.generated_tokens, req.generated_token_ids = kept
        migrated.append(req.request_id)

    def migrate_many(ms):
        for m in ms:
            migrate(m)

    sched = DecodingStageFCFSScheduler(
        DecodingStageSchedConfig("fcfs", sc["max_batch_size"], sc["max_tokens_per_batch"], sc["threshold"]), pc, bm, migrate,
        migrate_many if batched else None)
    out, next_id = [], 0
    for _ in range(len(sc["steps"])):
        swaps.clear()
        migrated.clear()
        arrivals = []
        for _ in range(rng.choice([0, 0, 0, 1, 1, 2])):
            n, mt = rng.randint(4, 12 * block_size), rng.randint(2, 40)
            req = Request(next_id, [0] * n, max_tokens=mt)
            req.add_generated_token()
            sched.add_request(MigratingRequest(req, list(range(-(-n // block_size))), pc))
            arrivals.append([next_id, n, mt])
            next_id += 1
        batch = sched.get_next_batch()
        batch_ids = batch.get_request_ids()
        finished = []
        if len(batch):
            bm.allocate_blocks_batched(batch)
            for r in batch.requests:
                r.add_generated_token()
            finished = sched.pop_finished_requests()
            bm.free_blocks_batched(finished)
        swaps_in_batching = [list(x) for x in swaps]
        accepted = sched.post_process_batched() if batched else sched.post_process()
        assert accepted == migrated
        out.append(dict(arrivals=arrivals, batch=batch_ids, finished=[r.request_id for r in finished], swaps=swaps_in_batching,
                        accepted=list(accepted),
                        unaccepted=[len(sched.unaccepted_queue)] + [m.req.request_id for m in sched.unaccepted_queue[:2]],
                        waiting=[r.request_id for r in sched.waiting_queue], swapped=[r.request_id for r in sched.swapped_queue],
                        avail=[bm.get_num_avail_gpu_blocks(), bm.get_num_avail_cpu_blocks()], digest=state_digest(bm)))
    return out


@pytest.mark.parametrize("batched", [False, True], ids=["one-by-one", "batched"])
def test_scheduler_replays_reference_decisions(golden_dir, batched):
    scenarios = load(golden_dir)
    assert sum(len(s["swaps"]) for sc in scenarios for s in sc["steps"]) >= 20       # the trace does exercise swapping
    assert sum(len(s["accepted"]) for sc in scenarios for s in sc["steps"]) >= 200
    for sc in scenarios:
        got = simulate(sc, batched)
        for i, (mine, ref) in enumerate(zip(got, sc["steps"])):
            assert mine == ref, f"scenario seed {sc['seed']}, iteration {i}: {mine} != {ref}"


def test_abort_and_counters():
    bm = BlockManager("decoding", 16, 4, KVModelConfig(2, 2, 8), ParallelConfig(), CacheConfig(4, 64), lambda *a: None)
    sched = DecodingStageFCFSScheduler(DecodingStageSchedConfig("fcfs", 2, 64, 1.0), ParallelConfig(), bm,
                                       lambda m: bm.allocate_blocks(m.req))
    for rid in range(3):
        req = Request(rid, [0] * 4, max_tokens=8)
        sched.add_request(MigratingRequest(req, [rid], ParallelConfig()))
    assert sched.post_process() == [0, 1, 2]
    assert sched.get_waiting_num_requests() == 3
    batch = sched.get_next_batch()
    assert batch.get_request_ids() == [0, 1] and sched.get_processing_num_requests() == 2
    sched.abort_request(2)                                   # still waiting: dropped
    sched.abort_request(0)                                   # running: marked finished, released by the normal path
    assert sched.get_waiting_num_requests() == 0
    assert [r.request_id for r in sched.pop_finished_requests()] == [0]
    assert sched.get_total_num_requests() == 1
    with pytest.raises(AssertionError):
        DecodingStageFCFSScheduler(DecodingStageSchedConfig("srpt"), ParallelConfig(), bm, lambda m: None)


def test_context_scheduler_replays_reference_decisions(golden_dir):
    """Prefill batches while finished requests still hold their blocks, waiting to be migrated."""
    from distserve_b200.request import BatchedRequests  # noqa: F401  (the scheduler returns these)
    from distserve_b200.scheduler import ContextStageFCFSScheduler, ContextStageSchedConfig

    with open(golden_dir / "context_scheduler.json") as f:
        scenarios = json.load(f)
    assert sum(1 for sc in scenarios for s in sc["steps"] if s["waiting"][0]) >= 30      # back-pressure does occur
    for sc in scenarios:
        rng = random.Random(sc["seed"])
        block_size = sc["block_size"]
        pc = ParallelConfig()
        bm = BlockManager("context", sc["gpu_blocks"], 1, KVModelConfig(12, 12, 64), pc, CacheConfig(block_size, 256), lambda *a: None)
        sched = ContextStageFCFSScheduler(ContextStageSchedConfig("fcfs", sc["max_batch_size"], sc["max_tokens_per_batch"]), pc, bm)
        pending, next_id = [], 0
        for it, ref in enumerate(sc["steps"]):
            arrivals = []
            for _ in range(rng.choice([0, 1, 1, 2])):
                n = rng.randint(4, 10 * block_size)
                sched.add_request(Request(next_id, [0] * n, max_tokens=rng.choice([1, 8])))
                arrivals.append([next_id, n])
                next_id += 1
            batch = sched.get_next_batch_and_pop()
            ids = batch.get_request_ids()
            for r in batch.requests:
                r.add_generated_token()
            sched.on_finish_requests(batch)
            for r in batch.requests:
                if not r.is_finished:
                    pending.append((it + rng.randint(0, 14), r))
            done = [r for due, r in pending if due <= it]
            pending = [(due, r) for due, r in pending if due > it]
            for r in done:
                sched.on_request_migrated(MigratingRequest(r, [], pc))
            mine = dict(arrivals=arrivals, batch=ids, migrated=[r.request_id for r in done],
                        waiting=[len(sched.waiting_queue)] + [r.request_id for r in sched.waiting_queue[:2]],
                        unaccepted=[r.request_id for r in sched.unaccepted_queue], on_fly=sched.num_on_fly_request_block)
            assert mine == ref, f"seed {sc['seed']} iteration {it}: {mine} != {ref}"


def test_pipelined_acceptance_accepts_the_same_requests_one_call_later():
    """post_process_pipelined enqueues the group accepted now before it awaits the group enqueued by the
    previous call; over a whole run it accepts the requests post_process_batched accepts, in the same order,
    and every group is begun before the previous one is finished."""
    from distserve_b200.block_manager import BlockManager
    from distserve_b200.config import CacheConfig, KVModelConfig, ParallelConfig
    from distserve_b200.request import MigratingRequest, Request
    from distserve_b200.scheduler import DecodingStageFCFSScheduler, DecodingStageSchedConfig

    def run(pipelined):
        pc, cache, model = ParallelConfig(), CacheConfig(16, 1 << 20), KVModelConfig(2, 2, 8)
        bm = BlockManager("decoding", 256, 1, model, pc, cache, lambda *a: [])
        log = []

        def begin(group):
            for m in group:
                bm.allocate_blocks(Request.of_length(m.req.request_id, m.req.get_input_len()))
            log.append(("begin", [m.req.request_id for m in group]))
            return list(group)

        def finish(pending):
            log.append(("finish", [m.req.request_id for m in pending]))

        def batched(group):
            finish(begin(group))

        s = DecodingStageFCFSScheduler(DecodingStageSchedConfig(), pc, bm, lambda m: batched([m]), batched,
                                       begin if pipelined else None, finish if pipelined else None)
        for rid in range(30):
            req = Request.of_length(rid, 40 + 7 * rid)
            req.append_token()
            s.add_request(MigratingRequest(req, list(range(-(-req.get_input_len() // 16))), pc))
        ready_order = []
        for _ in range(200):
            ready_order += s.post_process_pipelined() if pipelined else s.post_process_batched()
            batch = s.get_next_batch()
            for r in list(batch.requests)[:2]:               # two requests finish per iteration
                r.is_finished = True
            for q in s.batch_queues:
                for r in q.pop_finished_requests():
                    bm.free_blocks(r.request_id)
            if not s.unaccepted_queue and s._in_flight is None:
                break
        return ready_order, log

    plain, _ = run(False)
    piped, log = run(True)
    assert plain == piped == list(range(30))
    # a group is begun before the group ahead of it is finished
    begins = [i for i, (kind, _) in enumerate(log) if kind == "begin"]
    finishes = [i for i, (kind, _) in enumerate(log) if kind == "finish"]
    assert len(begins) == len(finishes) >= 2
    assert all(log[b][1] == log[f][1] for b, f in zip(begins, finishes))
    assert any(begins[i + 1] < finishes[i] for i in range(len(begins) - 1))

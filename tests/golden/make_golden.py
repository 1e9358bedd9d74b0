"""Regenerates the fixtures in this directory from the UNMODIFIED reference
Python package.  Run once, where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

The reference's native library is absent, so nothing here executes the copy
itself; what the fixtures pin is everything the reference's own code decides
on this path:

* geometry.json       — ModelConfig.get_num_layers / get_num_heads /
                        get_head_size and ParallelConfig.to_list() for the
                        benchmark model shapes and stage layouts;
* block_manager.json  — every block table and every worker call produced by
                        the reference BlockManager over a seeded sequence of
                        allocate / extend / free / swap-out / swap-in steps;
* scheduler.json      — every decision of the reference decoding-stage scheduler
                        (batches, acceptances = migrations, swap-outs and
                        swap-ins) over seeded arrival traces;
* context_scheduler.json — prefill batches of the reference context-stage
                        scheduler while finished requests wait to be migrated;
* worker_calls.json   — the exact positional arguments the reference
                        ParaWorker passes to the four native operators.

``ray`` is not installed; a stub whose ``remote`` returns the class unchanged
is injected so that the reference modules import.
"""
from __future__ import annotations

import json
import os
import random
import sys
import tempfile
import types
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent

MODEL_SHAPES = {
    # name: HuggingFace config fields that the geometry methods read
    "opt-125m": dict(model_type="opt", hidden_size=768, num_attention_heads=12, num_hidden_layers=12,
                     max_position_embeddings=2048, vocab_size=50272, ffn_dim=3072),
    "opt-13b": dict(model_type="opt", hidden_size=5120, num_attention_heads=40, num_hidden_layers=40,
                    max_position_embeddings=2048, vocab_size=50272, ffn_dim=20480),
    "llama-2-13b": dict(model_type="llama", hidden_size=5120, num_attention_heads=40, num_key_value_heads=40,
                        num_hidden_layers=40, max_position_embeddings=4096, vocab_size=32000, intermediate_size=13824),
    "llama-2-70b": dict(model_type="llama", hidden_size=8192, num_attention_heads=64, num_key_value_heads=8,
                        num_hidden_layers=80, max_position_embeddings=4096, vocab_size=32000, intermediate_size=28672),
    "llama-2-7b": dict(model_type="llama", hidden_size=4096, num_attention_heads=32, num_key_value_heads=32,
                       num_hidden_layers=32, max_position_embeddings=4096, vocab_size=32000, intermediate_size=11008),
}
LAYOUTS = [(1, 1), (2, 1), (1, 2), (2, 2), (4, 1), (4, 2), (8, 1)]   # (tp, pp)


def import_reference(ref_root: str):
    ray = types.ModuleType("ray")
    ray.remote = lambda *a, **k: (a[0] if a and callable(a[0]) and not k else (lambda cls: cls))
    ray.get_gpu_ids = lambda: [0]
    for name in ("ray.util", "ray.util.placement_group", "ray.util.scheduling_strategies"):
        sys.modules[name] = types.ModuleType(name)
    sys.modules["ray.util.placement_group"].PlacementGroup = object
    sys.modules["ray.util.scheduling_strategies"].PlacementGroupSchedulingStrategy = object
    ray.util = sys.modules["ray.util"]
    sys.modules["ray"] = ray
    # distserve/__init__.py insists on loading a shared library; any loadable one will do.
    sys.path.insert(0, str(ROOT))
    from distserve_b200 import kvmig_library_path

    os.environ["SWIFT_TRANSFORMER_LIB_PATH"] = str(kvmig_library_path())
    sys.path.insert(0, ref_root)
    import distserve  # noqa: F401
    return distserve


def write_hf_dir(tmp: str, name: str) -> str:
    d = os.path.join(tmp, name)
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(MODEL_SHAPES[name], f)
    return d


def golden_geometry(tmp: str):
    from distserve.config import ModelConfig, ParallelConfig

    out = []
    for name in MODEL_SHAPES:
        mc = ModelConfig(write_hf_dir(tmp, name), None)
        for tp, pp in LAYOUTS:
            try:
                pc = ParallelConfig(tp, tp - 1, pp, pp - 1)
                out.append(dict(model=name, tp=tp, pp=pp, layers_total=mc.get_num_layers(), heads_total=mc.get_num_heads(),
                                layers_local=mc.get_num_layers(pc), heads_local=mc.get_num_heads(pc),
                                head_size=mc.get_head_size(), dtype_size=mc.get_dtype_size(), to_list=pc.to_list()))
            except AssertionError:
                out.append(dict(model=name, tp=tp, pp=pp, error="not divisible"))
    return out


def state_digest(bm) -> str:
    """Digest of every block table, location and free/parked list of a block manager."""
    import hashlib

    state = [sorted((k, list(v)) for k, v in bm.block_table.items()),
             sorted((k, v.value) for k, v in bm.request_location.items()),
             list(bm.free_gpu_blocks_list), list(bm.free_cpu_blocks_list),
             list(bm.swapping_gpu_blocks_list), list(bm.swapping_cpu_blocks_list)]
    return hashlib.sha1(json.dumps(state, separators=(",", ":")).encode()).hexdigest()[:16]


def golden_block_manager(tmp: str):
    from distserve.block_manager import BlockManager
    from distserve.config import CacheConfig, ModelConfig, ParallelConfig
    from distserve.request import Request
    from distserve.utils import Stage

    mc = ModelConfig(write_hf_dir(tmp, "opt-125m"), None)
    calls = []

    def record(name, *args):
        if name == "swap_blocks":
            reqs, src, dst, is_in = args
            calls.append([name, [r.request_id for r in reqs], list(src), list(dst), bool(is_in)])
        else:
            calls.append([name])

    scenarios = []
    for seed, (gpu_blocks, cpu_blocks, block_size) in enumerate([(64, 48, 16), (40, 40, 8), (128, 64, 16)]):
        rng = random.Random(7000 + seed)
        bm = BlockManager(Stage.DECODING, gpu_blocks, cpu_blocks, mc, ParallelConfig(), CacheConfig(block_size, 256), record)
        live, on_cpu, steps, next_id = {}, set(), [], 0
        for _ in range(300):
            calls.clear()
            choices = ["alloc"]
            if live:
                choices += ["extend", "free", "swap_out", "swap_in"]
            op = rng.choice(choices)
            entry = {"op": op}
            try:
                if op == "alloc":
                    n = rng.randint(1, 5 * block_size)
                    req = Request(0.0, next_id, "", [0] * n)
                    need = bm.get_num_blocks_needed(req)
                    if need > bm.get_num_avail_gpu_blocks():
                        continue
                    bm.allocate_blocks(req)
                    live[next_id] = req
                    entry.update(request_id=next_id, prompt_len=n)
                    next_id += 1
                elif op == "extend":
                    rid = rng.choice(sorted(set(live) - on_cpu) or [None])
                    if rid is None:
                        continue
                    req = live[rid]
                    k = rng.randint(1, 2 * block_size)
                    for _ in range(k):
                        req.generated_tokens.append("")
                        req.generated_token_ids.append(0)
                    if bm.get_num_append_blocks_needed(req) > bm.get_num_avail_gpu_blocks():
                        for _ in range(k):
                            req.generated_tokens.pop()
                            req.generated_token_ids.pop()
                        continue
                    bm.allocate_blocks(req)
                    entry.update(request_id=rid, new_tokens=k)
                elif op == "free":
                    rid = rng.choice(sorted(live))
                    bm.free_blocks(rid)
                    live.pop(rid)
                    on_cpu.discard(rid)
                    entry.update(request_id=rid)
                elif op == "swap_out":
                    cands = sorted(set(live) - on_cpu)
                    if not cands:
                        continue
                    picked = rng.sample(cands, min(len(cands), rng.randint(1, 2)))
                    if sum(len(bm.block_table[r]) for r in picked) > bm.get_num_avail_cpu_blocks():
                        continue
                    bm.swap_out_requests([live[r] for r in picked])
                    on_cpu.update(picked)
                    entry.update(request_ids=picked)
                elif op == "swap_in":
                    cands = sorted(on_cpu)
                    if not cands:
                        continue
                    picked = rng.sample(cands, min(len(cands), rng.randint(1, 2)))
                    if sum(len(bm.block_table[r]) for r in picked) > bm.get_num_avail_gpu_blocks():
                        continue
                    bm.swap_in_requests([live[r] for r in picked])
                    on_cpu.difference_update(picked)
                    entry.update(request_ids=picked)
            except AssertionError as e:   # recorded: the mirror must refuse the same step
                entry["assertion"] = str(e)[:40]
            entry["calls"] = [list(c) for c in calls]
            touched = entry.get("request_ids", [entry["request_id"]] if "request_id" in entry else [])
            entry["touched"] = {str(r): list(bm.block_table[r]) for r in touched if r in bm.block_table}
            entry["digest"] = state_digest(bm)
            entry["avail"] = [bm.get_num_avail_gpu_blocks(), bm.get_num_avail_cpu_blocks()]
            steps.append(entry)
        scenarios.append(dict(gpu_blocks=gpu_blocks, cpu_blocks=cpu_blocks, block_size=block_size, steps=steps))
    return scenarios


def golden_worker_calls(tmp: str):
    """Drive the reference ParaWorker's KV methods with recording stand-ins for
    the native operators and a meta-device torch.empty, and keep the arguments."""
    import torch
    from distserve.config import CacheConfig, ModelConfig, ParallelConfig
    from distserve.utils import Stage
    from distserve.worker import ParaWorker

    recorded = []

    class Recorder:
        def __init__(self, ns):
            self.ns = ns

        def __getattr__(self, op):
            def call(*args):
                norm = []
                for a in args:
                    if isinstance(a, torch.Tensor):
                        norm.append({"tensor": list(a.shape), "dtype": str(a.dtype)})
                    else:
                        norm.append(a)
                recorded.append({"op": f"{self.ns}.{op}", "args": norm})
                return [len(recorded)] * 3 if op == "get_ipc_mem_handle" else None
            return call

    torch.ops.block_migration_ops = Recorder("block_migration_ops")
    torch.ops.swapping_ops = Recorder("swapping_ops")
    real_empty, real_sync = torch.empty, torch.cuda.synchronize
    torch.empty = lambda shape, dtype=None, device=None, pin_memory=False: real_empty(shape, dtype=dtype, device="meta")
    torch.cuda.synchronize = lambda *a, **k: None

    class FakeStream:
        def __enter__(self):
            return self

        def __exit__(self, *a):
            return False

    real_stream_ctx, real_event = torch.cuda.stream, torch.cuda.Event
    torch.cuda.stream = lambda s: FakeStream()

    class FakeEvent:
        def record(self, stream=None):
            pass

        def wait(self, stream=None):
            pass

    torch.cuda.Event = FakeEvent
    cases = []
    try:
        for model, (ctx_tp, ctx_pp), (dec_tp, dec_pp) in [("opt-125m", (1, 1), (1, 1)), ("llama-2-13b", (2, 1), (1, 1)),
                                                          ("llama-2-70b", (4, 1), (2, 2))]:
            mc = ModelConfig(write_hf_dir(tmp, model), None)
            for dp in range(dec_pp):
                for dt in range(dec_tp):
                    recorded.clear()
                    w = object.__new__(ParaWorker)
                    w.model_config, w.cache_config = mc, CacheConfig(16, 256)
                    w.parallel_config = ParallelConfig(dec_tp, dt, dec_pp, dp)
                    w.stage = Stage.DECODING
                    w.swap_in_stream = w.swap_out_stream = object()
                    w.swap_event_table = {}
                    w.latest_swap_in_event = w.latest_swap_out_event = None
                    handles_back = w.init_kvcache_and_swap(32, 8)
                    table = [[([1000 + p * 10 + t], [2000 + p * 10 + t]) for t in range(ctx_tp)] for p in range(ctx_pp)]
                    ctx_pc = ParallelConfig(ctx_tp, 0, ctx_pp, 0)
                    w.register_kvcache_mem_handles(ctx_pc, table)
                    w.migrate_blocks([3, 1, 4], ctx_pc, [9, 2, 6])
                    w.swap_blocks([11], [5, 6], [0, 1], False)
                    w.swap_blocks([11], [0, 1], [7, 8], True)
                    cases.append(dict(model=model, ctx=[ctx_tp, ctx_pp], dec=[dec_tp, dt, dec_pp, dp],
                                      init_returned=[list(h) for h in handles_back], calls=[dict(c) for c in recorded]))
    finally:
        torch.empty, torch.cuda.synchronize = real_empty, real_sync
        torch.cuda.stream, torch.cuda.Event = real_stream_ctx, real_event
    return cases


SCHEDULER_SCENARIOS = [
    # seed, gpu_blocks, cpu_blocks, block_size, max_batch_size, max_tokens_per_batch, threshold, iterations
    (11, 48, 64, 16, 8, 64, 0.25, 260),
    (12, 96, 96, 8, 16, 32, 0.10, 260),
    (13, 400, 64, 16, 4, 8, 0.05, 200),
]


def golden_scheduler(tmp: str):
    """Drive the reference decoding-stage scheduler the way DecodingStageLLMEngine._step does
    (get_next_batch, allocate, one token per request, pop finished, free, post_process) over a seeded
    arrival trace, and record every decision."""
    import asyncio

    from distserve.block_manager import BlockManager
    from distserve.config import CacheConfig, DecodingStageSchedConfig, ModelConfig, ParallelConfig
    from distserve.decoding_stage_scheduler import DecodingStageFCFSScheduler
    from distserve.request import MigratingRequest, Request, SamplingParams
    from distserve.utils import Stage

    mc = ModelConfig(write_hf_dir(tmp, "opt-125m"), None)

    async def run(seed, gpu_blocks, cpu_blocks, block_size, max_bs, max_tok, thr, iters):
        rng = random.Random(seed)
        swaps, migrated = [], []

        def record(name, *args):
            if name == "swap_blocks":
                reqs, src, dst, is_in = args
                swaps.append([[r.request_id for r in reqs], list(src), list(dst), bool(is_in)])

        pc = ParallelConfig()
        bm = BlockManager(Stage.DECODING, gpu_blocks, cpu_blocks, mc, pc, CacheConfig(block_size, 256), record)

        async def migrate(m):
            req = m.req
            kept = (req.generated_tokens, req.generated_token_ids)
            req.generated_tokens, req.generated_token_ids = [], []
            bm.allocate_blocks(req)
            req.generated_tokens, req.generated_token_ids = kept
            migrated.append(req.request_id)

        sched = DecodingStageFCFSScheduler(DecodingStageSchedConfig("fcfs", max_bs, max_tok, waiting_block_prop_threshold=thr),
                                           pc, bm, migrate)
        steps, next_id = [], 0
        for _ in range(iters):
            swaps.clear()
            migrated.clear()
            arrivals = []
            for _ in range(rng.choice([0, 0, 0, 1, 1, 2])):
                n, mt = rng.randint(4, 12 * block_size), rng.randint(2, 40)
                req = Request(0.0, next_id, "", [0] * n, SamplingParams(max_tokens=mt))
                req.add_generated_token("", 0)        # the token prefill produced
                await sched.add_request(MigratingRequest(req, list(range(-(-n // block_size))), pc))
                arrivals.append([next_id, n, mt])
                next_id += 1
            batch = sched.get_next_batch()
            batch_ids = batch.get_request_ids()
            finished = []
            if len(batch):
                bm.allocate_blocks_batched(batch)
                for r in batch.requests:
                    r.add_generated_token("", 0)
                finished = sched.pop_finished_requests()
                bm.free_blocks_batched(finished)
            swaps_in_batching = [list(x) for x in swaps]
            await sched.post_process()
            steps.append(dict(arrivals=arrivals, batch=batch_ids, finished=[r.request_id for r in finished],
                              swaps=swaps_in_batching, accepted=list(migrated),
                              unaccepted=[len(sched.unaccepted_queue)] + [m.req.request_id for m in sched.unaccepted_queue[:2]],
                              waiting=[r.request_id for r in sched.waiting_queue],
                              swapped=[r.request_id for r in sched.swapped_queue],
                              avail=[bm.get_num_avail_gpu_blocks(), bm.get_num_avail_cpu_blocks()],
                              digest=state_digest(bm)))
        return dict(seed=seed, gpu_blocks=gpu_blocks, cpu_blocks=cpu_blocks, block_size=block_size, max_batch_size=max_bs,
                    max_tokens_per_batch=max_tok, threshold=thr, steps=steps)

    return [asyncio.run(run(*sc)) for sc in SCHEDULER_SCENARIOS]


def golden_context_scheduler(tmp: str):
    """The reference context-stage scheduler over a seeded trace: arrivals, prefill batches, and
    migrations completing a random number of iterations later."""
    from distserve.block_manager import BlockManager
    from distserve.config import CacheConfig, ContextStageSchedConfig, ModelConfig, ParallelConfig
    from distserve.context_stage_scheduler import ContextStageFCFSScheduler
    from distserve.request import MigratingRequest, Request, SamplingParams
    from distserve.utils import Stage

    mc = ModelConfig(write_hf_dir(tmp, "opt-125m"), None)
    out = []
    for seed, gpu_blocks, block_size, max_bs, max_tok in [(21, 30, 16, 4, 256), (22, 64, 8, 8, 100)]:
        rng = random.Random(seed)
        pc = ParallelConfig()
        bm = BlockManager(Stage.CONTEXT, gpu_blocks, 1, mc, pc, CacheConfig(block_size, 256), lambda *a: None)
        sched = ContextStageFCFSScheduler(ContextStageSchedConfig("fcfs", max_bs, max_tok), pc, bm)
        pending, steps, next_id = [], [], 0
        for it in range(200):
            arrivals = []
            for _ in range(rng.choice([0, 1, 1, 2])):
                n = rng.randint(4, 10 * block_size)
                sched.add_request(Request(0.0, next_id, "", [0] * n, SamplingParams(max_tokens=rng.choice([1, 8]))))
                arrivals.append([next_id, n])
                next_id += 1
            batch = sched.get_next_batch_and_pop()
            ids = batch.get_request_ids()
            for r in batch.requests:
                r.add_generated_token("", 0)             # a request with max_tokens 1 is finished after prefill
            sched.on_finish_requests(batch)
            for r in batch.requests:
                if not r.is_finished:
                    pending.append((it + rng.randint(0, 14), r))
            done = [r for due, r in pending if due <= it]
            pending = [(due, r) for due, r in pending if due > it]
            for r in done:
                sched.on_request_migrated(MigratingRequest(r, [], pc))
            steps.append(dict(arrivals=arrivals, batch=ids, migrated=[r.request_id for r in done],
                              waiting=[len(sched.waiting_queue)] + [r.request_id for r in sched.waiting_queue[:2]],
                              unaccepted=[r.request_id for r in sched.unaccepted_queue], on_fly=sched.num_on_fly_request_block))
        out.append(dict(seed=seed, gpu_blocks=gpu_blocks, block_size=block_size, max_batch_size=max_bs,
                        max_tokens_per_batch=max_tok, steps=steps))
    return out


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else str(ROOT.parent / "reference")   # a checkout beside this repo
    import_reference(ref_root)
    with tempfile.TemporaryDirectory() as tmp:
        for name, fn in (("geometry", golden_geometry), ("block_manager", golden_block_manager),
                         ("scheduler", golden_scheduler), ("context_scheduler", golden_context_scheduler),
                         ("worker_calls", golden_worker_calls)):
            data = fn(tmp)
            with open(HERE / f"{name}.json", "w") as f:
                json.dump(data, f, separators=(",", ":"))
            print(name, len(data), "entries,", (HERE / f"{name}.json").stat().st_size, "bytes")


if __name__ == "__main__":
    main()

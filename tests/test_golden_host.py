"""Host-side mirrors against fixtures recorded from the unmodified reference
package (tests/golden/make_golden.py): shard geometry, the block manager's id
sequences, and the positional arguments that reach the native operators."""
import hashlib
import json

import pytest
import torch

from distserve_b200.block_manager import BlockManager
from distserve_b200.config import CacheConfig, KVModelConfig, ParallelConfig
from distserve_b200.request import Request

MODEL_KV = {
    # name -> (layers, KV heads, head_dim) as the reference derives them from the HF config
    "opt-125m": (12, 12, 64), "opt-13b": (40, 40, 128), "llama-2-13b": (40, 40, 128),
    "llama-2-70b": (80, 8, 128), "llama-2-7b": (32, 32, 128),
}


def load(golden_dir, name):
    with open(golden_dir / f"{name}.json") as f:
        return json.load(f)


def test_geometry_matches_reference(golden_dir):
    rows = load(golden_dir, "geometry")
    assert len(rows) >= 30
    for row in rows:
        L, H, D = MODEL_KV[row["model"]]
        mc = KVModelConfig(L, H, D)
        if "error" in row:
            pc = ParallelConfig(row["tp"], 0, row["pp"], 0)
            with pytest.raises(ValueError):
                mc.get_num_layers(pc), mc.get_num_heads(pc)
            continue
        pc = ParallelConfig(row["tp"], row["tp"] - 1, row["pp"], row["pp"] - 1)
        assert (mc.get_num_layers(), mc.get_num_heads()) == (row["layers_total"], row["heads_total"])
        assert (mc.get_num_layers(pc), mc.get_num_heads(pc)) == (row["layers_local"], row["heads_local"])
        assert mc.get_head_size() == row["head_size"] and mc.get_dtype_size() == row["dtype_size"]
        assert pc.to_list() == row["to_list"]


def state_digest(bm) -> str:
    state = [sorted((k, list(v)) for k, v in bm.block_table.items()),
             sorted((k, v.value) for k, v in bm.request_location.items()),
             list(bm.free_gpu_blocks_list), list(bm.free_cpu_blocks_list),
             list(bm.swapping_gpu_blocks_list), list(bm.swapping_cpu_blocks_list)]
    return hashlib.sha1(json.dumps(state, separators=(",", ":")).encode()).hexdigest()[:16]


def test_block_manager_replays_reference_trace(golden_dir):
    for scenario in load(golden_dir, "block_manager"):
        calls = []

        def record(name, *args):
            if name == "swap_blocks":
                reqs, src, dst, is_in = args
                calls.append([name, [r.request_id for r in reqs], list(src), list(dst), bool(is_in)])
            else:
                calls.append([name])

        bm = BlockManager("decoding", scenario["gpu_blocks"], scenario["cpu_blocks"], KVModelConfig(12, 12, 64),
                          ParallelConfig(), CacheConfig(scenario["block_size"], 256), record)
        live = {}
        for i, step in enumerate(scenario["steps"]):
            calls.clear()
            op = step["op"]
            if op == "alloc":
                req = Request.of_length(step["request_id"], step["prompt_len"])
                live[req.request_id] = req
                bm.allocate_blocks(req)
            elif op == "extend":
                req = live[step["request_id"]]
                for _ in range(step["new_tokens"]):
                    req.append_token()
                bm.allocate_blocks(req)
            elif op == "free":
                bm.free_blocks(step["request_id"])
                live.pop(step["request_id"])
            elif op == "swap_out":
                bm.swap_out_requests([live[r] for r in step["request_ids"]])
            elif op == "swap_in":
                bm.swap_in_requests([live[r] for r in step["request_ids"]])
            assert calls == step["calls"], f"step {i} ({op}): worker calls differ"
            for rid, blocks in step["touched"].items():
                assert bm.get_block_table(int(rid)) == blocks, f"step {i} ({op}): block table of request {rid}"
            assert [bm.get_num_avail_gpu_blocks(), bm.get_num_avail_cpu_blocks()] == step["avail"]
            assert state_digest(bm) == step["digest"], f"step {i} ({op}): state digest"


def test_block_manager_refuses_what_the_reference_refuses():
    bm = BlockManager("decoding", 4, 2, KVModelConfig(2, 2, 8), ParallelConfig(), CacheConfig(4, 8), lambda *a: None)
    big = Request.of_length(0, 17)          # 5 blocks > 4
    with pytest.raises(AssertionError, match="not enough free blocks on GPU"):
        bm.allocate_blocks(big)
    with pytest.raises(AssertionError, match="not allocated"):
        bm.free_blocks(3)
    req = Request.of_length(1, 8)
    bm.allocate_blocks(req)
    bm.swap_out_requests([req])
    with pytest.raises(AssertionError, match="currently on CPU"):
        bm.allocate_blocks(req)
    with pytest.raises(AssertionError):
        bm.swap_out_requests([req])         # already on the host
    assert bm.is_all_requests_on_gpu(type("B", (), {"requests": [req]})()) is False


def test_worker_passes_the_reference_arguments(golden_dir, monkeypatch):
    """KVWorker must hand the operators exactly what ParaWorker hands them."""
    import distserve_b200.worker as W

    recorded = []

    class Recorder:
        def __init__(self, ns):
            self.ns = ns

        def __getattr__(self, op):
            def call(*args):
                norm = [{"tensor": list(a.shape), "dtype": str(a.dtype)} if isinstance(a, torch.Tensor) else a for a in args]
                recorded.append({"op": f"{self.ns}.{op}", "args": norm})
                return [len(recorded)] * 3 if op == "get_ipc_mem_handle" else None
            return call

    class Ctx:
        def __enter__(self):
            return self

        def __exit__(self, *a):
            return False

    class FakeStream(Ctx):
        cuda_stream = 0

        def wait_stream(self, other):
            pass

    class FakeEvent:
        def record(self, stream=None):
            pass

        def wait(self, stream=None):
            pass

        def query(self):
            return False

    real_empty = torch.empty
    monkeypatch.setattr(torch.ops, "block_migration_ops", Recorder("block_migration_ops"), raising=False)
    monkeypatch.setattr(torch.ops, "swapping_ops", Recorder("swapping_ops"), raising=False)
    monkeypatch.setattr(W.torch, "empty", lambda shape, dtype=None, device=None, pin_memory=False: real_empty(shape, dtype=dtype, device="meta"))
    monkeypatch.setattr(W.torch.cuda, "synchronize", lambda *a, **k: None)
    monkeypatch.setattr(W.torch.cuda, "device", lambda d: Ctx())
    monkeypatch.setattr(W.torch.cuda, "stream", lambda s: Ctx())
    monkeypatch.setattr(W.torch.cuda, "current_stream", lambda *a: FakeStream())
    monkeypatch.setattr(W.torch.cuda, "Event", FakeEvent)

    for case in load(golden_dir, "worker_calls"):
        L, H, D = MODEL_KV[case["model"]]
        recorded.clear()
        w = object.__new__(W.KVWorker)
        w.model_config, w.cache_config = KVModelConfig(L, H, D), CacheConfig(16, 256)
        dec_tp, dt, dec_pp, dp = case["dec"]
        w.parallel_config = ParallelConfig(dec_tp, dt, dec_pp, dp)
        w.device = "meta"
        w.swap_in_stream, w.swap_out_stream = FakeStream(), FakeStream()
        w.swap_event_table, w.latest_swap_in_event, w.latest_swap_out_event = {}, None, None
        w._swaps_issued, w._swaps_known_done = {True: 0, False: 0}, {True: 0, False: 0}
        ctx_tp, ctx_pp = case["ctx"]
        returned = w.init_kvcache_and_swap(32, 8)
        table = [[([1000 + p * 10 + t], [2000 + p * 10 + t]) for t in range(ctx_tp)] for p in range(ctx_pp)]
        ctx_pc = ParallelConfig(ctx_tp, 0, ctx_pp, 0)
        w.register_kvcache_mem_handles(ctx_pc, table)
        w.migrate_blocks([3, 1, 4], ctx_pc, [9, 2, 6])
        w.swap_blocks([11], [5, 6], [0, 1], False)
        w.swap_blocks([11], [0, 1], [7, 8], True)
        assert [list(h) for h in returned] == case["init_returned"]
        assert recorded == case["calls"], case["model"]


def test_swap_waits_are_skipped_once_a_later_swap_is_known_to_be_done(monkeypatch):
    """Swaps of one direction run in order on one stream: when mark n is known to have finished, questions
    about marks <= n must not touch CUDA any more (the shortcut of distserve/block_manager.py:277-285)."""
    import distserve_b200.worker as W

    log = []

    class Ctx:
        def __enter__(self):
            return self

        def __exit__(self, *a):
            return False

    class FakeStream(Ctx):
        def wait_stream(self, other):
            pass

    class FakeEvent:
        finished = set()

        def __init__(self):
            self.id = len(log)

        def record(self, stream=None):
            log.append(("record", id(self)))

        def wait(self, stream=None):
            log.append(("wait", id(self)))

        def query(self):
            log.append(("query", id(self)))
            return id(self) in FakeEvent.finished

        def synchronize(self):
            log.append(("synchronize", id(self)))

    class Ops:
        def swap(self, *args):
            pass

    monkeypatch.setattr(torch.ops, "swapping_ops", Ops(), raising=False)
    monkeypatch.setattr(W.torch.cuda, "device", lambda d: Ctx())
    monkeypatch.setattr(W.torch.cuda, "stream", lambda s: Ctx())
    monkeypatch.setattr(W.torch.cuda, "current_stream", lambda *a: FakeStream())
    monkeypatch.setattr(W.torch.cuda, "Event", FakeEvent)
    w = object.__new__(W.KVWorker)
    w.device = "meta"
    w.k_cache = w.v_cache = w.k_swap = w.v_swap = None
    w.swap_in_stream, w.swap_out_stream = FakeStream(), FakeStream()
    w.swap_event_table, w.latest_swap_in_event, w.latest_swap_out_event = {}, None, None
    w._swaps_issued, w._swaps_known_done = {True: 0, False: 0}, {True: 0, False: 0}

    for rid in (1, 2, 3):
        w.swap_blocks([rid], [rid], [rid], False)                  # three swap-outs, marks 1..3
    marks = {rid: w.swap_event_table[rid] for rid in (1, 2, 3)}
    assert [m.seq for m in marks.values()] == [1, 2, 3]
    assert w.swap_finished(2) is False                              # queried, not finished
    FakeEvent.finished.add(id(marks[3].event))
    assert w.swap_finished(3) is True                               # one query: mark 3 is over ...
    log.clear()
    assert w.swap_finished(1) is True and w.swap_finished(2) is True   # ... so 1 and 2 are, without any CUDA call
    w.prepare_step([1, 2])
    assert log == []
    w.swap_blocks([9], [0], [0], True)                              # the other direction keeps its own numbering
    assert w.swap_event_table[9].seq == 1 and w.swap_finished(9) is False
    w.prepare_step([9])
    assert ("wait", id(w.latest_swap_in_event)) in log
    w.swap_blocks([7], [1], [1], True)
    w.wait_for_all_swap_in()
    log.clear()
    assert w.swap_finished(7) is True and log == []                 # the flush marked everything issued as done

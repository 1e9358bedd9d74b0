"""Drives the UNMODIFIED reference classes — ``distserve.worker.ParaWorker`` and
``distserve.block_manager.BlockManager`` — against this repository's operator
library, on a GPU, and checks what they leave in the pools against the oracle.

Run by tests/test_reference_dropin_gpu.py in child processes (the reference's
``distserve/__init__.py`` loads whatever ``SWIFT_TRANSFORMER_LIB_PATH`` names at
import time, and its worker pins itself to ``cuda:0``, so each role gets a
process of its own):

    python reference_dropin_driver.py <reference root> single <out.json>
    python reference_dropin_driver.py <reference root> ctx    <exchange dir>
    python reference_dropin_driver.py <reference root> dec    <exchange dir> <out.json>

``single``: context tp=2 and decoding tp=1,pp=2 workers in one process, all on
cuda:0; block lists come from two reference block managers; then a swap-out /
swap-in round trip driven by the reference block manager.  ``ctx`` / ``dec``:
one context worker and one decoding worker in two processes that each see ONE
GPU as cuda:0 (the Ray actor situation), the handles travelling through a file.

``ray`` is not installed: a stub whose ``remote`` returns the class unchanged is
injected (and, for a pip-installed copy of the reference, a stub of the weight
downloader sub-package its setup.py leaves out).  ``init_model`` is never
called; the KV methods need nothing of it.
"""
from __future__ import annotations

import json
import os
import sys
import tempfile
import time
import types
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

HF_CONFIG = dict(model_type="llama", hidden_size=256, num_attention_heads=8, num_key_value_heads=8, num_hidden_layers=4,
                 max_position_embeddings=2048, vocab_size=32000, intermediate_size=512)
L, H, D, BLOCK = 4, 8, 32, 16


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
    sys.path.insert(0, ref_root)
    if not (Path(ref_root) / "distserve" / "downloader").is_dir():
        # The reference's setup.py lists only its two top-level packages, so a pip-installed copy lacks the
        # ``distserve.downloader`` sub-package that worker.py imports for ``init_model`` (never called here).
        stub = types.ModuleType("distserve.downloader")
        stub.download_and_convert_weights = lambda *a, **k: (_ for _ in ()).throw(RuntimeError("weights are not part of this test"))
        sys.modules["distserve.downloader"] = stub
    import warnings

    warnings.simplefilter("ignore")
    import distserve
    import distserve.block_manager
    import distserve.worker

    return distserve


def model_config(tmp: str):
    from distserve.config import ModelConfig

    d = os.path.join(tmp, "tiny-llama")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(HF_CONFIG, f)
    return ModelConfig(d, None)


def seeded_pool(seed, shape):
    import numpy as np

    return np.random.default_rng(seed).integers(-32768, 32767, size=shape, dtype=np.int16, endpoint=True)


def fill(worker, seed):
    """Give the worker's pools seeded contents; returns the host copies (bit patterns)."""
    import torch

    hk, hv = seeded_pool([seed, 0], tuple(worker.k_cache.shape)), seeded_pool([seed, 1], tuple(worker.v_cache.shape))
    worker.k_cache.copy_(torch.from_numpy(hk).view(torch.float16))
    worker.v_cache.copy_(torch.from_numpy(hv).view(torch.float16))
    torch.cuda.synchronize()
    return hk, hv


def bits(t):
    import torch

    return t.detach().cpu().view(torch.int16).numpy()


def run_single(out_path: str) -> None:
    import numpy as np
    import torch

    import distserve
    from distserve.block_manager import BlockManager
    from distserve.config import CacheConfig, ParallelConfig
    from distserve.request import Request
    from distserve.utils import Stage
    from distserve.worker import ParaWorker
    from oracle import kv_oracle as O

    report = {"lib_path": distserve.LIB_PATH, "worker_module": distserve.worker.__file__}
    with tempfile.TemporaryDirectory() as tmp:
        mc = model_config(tmp)
        cache = CacheConfig(BLOCK, 256)
        ctx_pc, dec_pc = ParallelConfig(2, 0, 1, 0), ParallelConfig(1, 0, 2, 0)
        n_ctx, n_dec, n_cpu = 48, 40, 24

        ctx_workers = [ParaWorker(t, Stage.CONTEXT, mc, cache, ParallelConfig(2, t, 1, 0)) for t in range(2)]
        handles = [[w.init_kvcache_and_swap(n_ctx, 1) for w in ctx_workers]]
        ctx_host = {(0, t): fill(w, 100 + t) for t, w in enumerate(ctx_workers)}
        dec_workers = [ParaWorker(10 + p, Stage.DECODING, mc, cache, ParallelConfig(1, 0, 2, p)) for p in range(2)]
        dec_host = []
        for p, w in enumerate(dec_workers):
            w.init_kvcache_and_swap(n_dec, n_cpu)
            dec_host.append(list(fill(w, 200 + p)))
            w.k_swap.zero_()
            w.v_swap.zero_()
            w.register_kvcache_mem_handles(ctx_pc, handles)
        report["pool_shapes"] = {"context": list(ctx_workers[0].k_cache.shape), "decoding": list(dec_workers[0].k_cache.shape)}

        def call_dec_workers(func_name, *args):
            return [getattr(w, func_name)(*args) for w in dec_workers]

        ctx_bm = BlockManager(Stage.CONTEXT, n_ctx, 1, mc, ctx_pc, cache, lambda *a: [])
        dec_bm = BlockManager(Stage.DECODING, n_dec, n_cpu, mc, dec_pc, cache, call_dec_workers)
        # scramble both free lists the way a long-running server's are
        rng = np.random.default_rng(7)
        ctx_bm.free_gpu_blocks_list[:] = [int(x) for x in rng.permutation(n_ctx)]
        dec_bm.free_gpu_blocks_list[:] = [int(x) for x in rng.permutation(n_dec)]

        # ---- migrate_blocks, as _migrate_blocks does (distserve/single_stage_engine.py:490-536) ----
        requests, migrated = [], []
        for rid, n_tokens in enumerate([37, 128, 5, 200]):
            req = Request(0.0, rid, "", [0] * n_tokens)
            ctx_bm.allocate_blocks(req)
            dec_bm.allocate_blocks(req)
            src, dst = list(ctx_bm.get_block_table(rid)), list(dec_bm.get_block_table(rid))
            assert len(src) == len(dst) == -(-n_tokens // BLOCK)
            for w in dec_workers:
                w.migrate_blocks(src, ctx_pc, dst)
            ctx_bm.free_blocks(rid)                       # the caller recycles the sources as soon as the call returns
            for p in range(2):
                O.migrate_blocks_numpy(ctx_host, 2, 1, src, 1, 0, 2, p, dst, dec_host[p][0], dec_host[p][1], L, H)
            requests.append(req)
            migrated.append((src, dst))
        torch.cuda.synchronize()
        report["migrate_equal"] = all(np.array_equal(bits(w.k_cache), dec_host[p][0]) and np.array_equal(bits(w.v_cache), dec_host[p][1])
                                      for p, w in enumerate(dec_workers))
        report["migrated_blocks"] = sum(len(s) for s, _ in migrated)

        # ---- swap out and back in through the reference block manager (distserve/block_manager.py:288-315) ----
        swap_wait = os.environ.get("KVMIG_SWAP_WAIT", "0") not in ("", "0")
        host_swap = [[np.zeros(tuple(w.k_swap.shape), np.int16), np.zeros(tuple(w.v_swap.shape), np.int16)] for w in dec_workers]
        victim = requests[1]
        before_ids = list(dec_bm.get_block_table(victim.request_id))
        dec_bm.swap_out_requests([victim])
        cpu_ids = list(dec_bm.get_block_table(victim.request_id))
        if swap_wait:
            call_dec_workers("wait_for_all_swap_out")     # returns at once: the operator itself has waited for its copies
        else:
            torch.cuda.synchronize()                      # the worker's own event was recorded before the copies
        for p in range(2):
            O.swap_numpy(before_ids, cpu_ids, False, dec_host[p][0], dec_host[p][1], host_swap[p][0], host_swap[p][1])
        report["swap_out_equal"] = all(np.array_equal(w.k_swap.view(torch.int16).numpy(), host_swap[p][0]) and
                                       np.array_equal(w.v_swap.view(torch.int16).numpy(), host_swap[p][1])
                                       for p, w in enumerate(dec_workers))
        # the GPU blocks it left are overwritten by another request before it returns
        filler = Request(0.0, 99, "", [0] * (len(before_ids) * BLOCK))
        ctx_bm.allocate_blocks(filler)
        dec_bm.allocate_blocks(filler)
        src, dst = list(ctx_bm.get_block_table(99)), list(dec_bm.get_block_table(99))
        for p, w in enumerate(dec_workers):
            w.migrate_blocks(src, ctx_pc, dst)
            O.migrate_blocks_numpy(ctx_host, 2, 1, src, 1, 0, 2, p, dst, dec_host[p][0], dec_host[p][1], L, H)
        dec_bm.free_blocks(99)
        dec_bm.swap_in_requests([victim])
        gpu_ids = list(dec_bm.get_block_table(victim.request_id))
        if swap_wait:
            call_dec_workers("wait_for_all_swap_in")
        torch.cuda.synchronize()
        for p in range(2):
            O.swap_numpy(cpu_ids, gpu_ids, True, dec_host[p][0], dec_host[p][1], host_swap[p][0], host_swap[p][1])
        report["swap_in_equal"] = all(np.array_equal(bits(w.k_cache), dec_host[p][0]) and np.array_equal(bits(w.v_cache), dec_host[p][1])
                                      for p, w in enumerate(dec_workers))
        report["swap_wait"] = swap_wait
        report["swapped_blocks"] = len(before_ids)
    Path(out_path).write_text(json.dumps(report))


def run_ctx(exchange: str) -> None:
    """One context worker on the only GPU this process sees; publishes its handles and keeps the pools alive
    until the decoding process is done."""
    from distserve.config import CacheConfig, ParallelConfig
    from distserve.utils import Stage
    from distserve.worker import ParaWorker

    with tempfile.TemporaryDirectory() as tmp:
        mc = model_config(tmp)
        w = ParaWorker(0, Stage.CONTEXT, mc, CacheConfig(BLOCK, 256), ParallelConfig(1, 0, 1, 0))
        handles = w.init_kvcache_and_swap(64, 1)
        fill(w, 300)
        tmp_path = Path(exchange) / "handles.json.tmp"
        tmp_path.write_text(json.dumps([[list(handles[0]), list(handles[1])]]))
        tmp_path.rename(Path(exchange) / "handles.json")
        deadline = time.time() + 300
        while not (Path(exchange) / "done").exists() and time.time() < deadline:
            time.sleep(0.05)


def run_dec(exchange: str, out_path: str) -> None:
    import numpy as np
    import torch

    from distserve.config import CacheConfig, ParallelConfig
    from distserve.utils import Stage
    from distserve.worker import ParaWorker
    from oracle import kv_oracle as O

    try:
        deadline = time.time() + 300
        while not (Path(exchange) / "handles.json").exists():
            if time.time() > deadline:
                raise RuntimeError("the context process never published its handles")
            time.sleep(0.05)
        table = [[tuple(pair)] for pair in json.loads((Path(exchange) / "handles.json").read_text())]
        with tempfile.TemporaryDirectory() as tmp:
            mc = model_config(tmp)
            pc = ParallelConfig(1, 0, 1, 0)
            w = ParaWorker(1, Stage.DECODING, mc, CacheConfig(BLOCK, 256), pc)
            w.init_kvcache_and_swap(48, 1)
            hk, hv = fill(w, 400)
            w.register_kvcache_mem_handles(pc, table)
            ctx_shape = (64, L, H, BLOCK, D)
            ctx_host = {(0, 0): (seeded_pool([300, 0], ctx_shape), seeded_pool([300, 1], ctx_shape))}
            rng = np.random.default_rng(9)
            for n in (1, 17, 40):
                src = [int(x) for x in rng.integers(0, 64, size=n)]
                dst = [int(x) for x in rng.permutation(48)[:n]]
                w.migrate_blocks(src, pc, dst)
                O.migrate_blocks_numpy(ctx_host, 1, 1, src, 1, 0, 1, 0, dst, hk, hv, L, H)
            torch.cuda.synchronize()
            report = {"migrate_equal": bool(np.array_equal(bits(w.k_cache), hk) and np.array_equal(bits(w.v_cache), hv)),
                      "visible_devices": os.environ.get("CUDA_VISIBLE_DEVICES"), "device_count": torch.cuda.device_count()}
        Path(out_path).write_text(json.dumps(report))
    finally:
        (Path(exchange) / "done").write_text("1")


def main() -> None:
    ref_root, role = sys.argv[1], sys.argv[2]
    import_reference(ref_root)
    if role == "single":
        run_single(sys.argv[3])
    elif role == "ctx":
        run_ctx(sys.argv[3])
    elif role == "dec":
        run_dec(sys.argv[3], sys.argv[4])
    else:
        raise SystemExit(f"unknown role {role!r}")


if __name__ == "__main__":
    main()

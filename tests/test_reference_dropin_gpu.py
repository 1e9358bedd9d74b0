"""The reference's own worker and block manager, unmodified, running on the GPU
against this repository's operator library (``SWIFT_TRANSFORMER_LIB_PATH``
pointing at the shim): init_kvcache_and_swap -> register_kvcache_mem_handles ->
migrate_blocks -> swap_blocks -> wait_for_all_swap_*, block lists from the
reference BlockManager, pools compared with the oracle.

The reference package is looked for in ``baseline/_ref`` (where
``__graft_entry__.build()`` installs it with pip when a reference checkout is
at hand), then in ``$DISTSERVE_REFERENCE_DIR``, then in a checkout beside this
repository; without any of them the tests are skipped.
"""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
DRIVER = Path(__file__).resolve().parent / "reference_dropin_driver.py"

pytestmark = pytest.mark.gpu


def reference_root():
    for cand in (ROOT / "baseline" / "_ref", Path(os.environ.get("DISTSERVE_REFERENCE_DIR", "/nonexistent")), ROOT.parent / "reference"):
        if (cand / "distserve" / "worker.py").is_file():
            return cand
    return None


REF = reference_root()
needs_reference = pytest.mark.skipif(REF is None, reason="no reference package at hand")


def run_driver(args, env_extra, timeout=600):
    from distserve_b200 import shim_library_path

    env = dict(os.environ, SWIFT_TRANSFORMER_LIB_PATH=str(shim_library_path()), **env_extra)
    return subprocess.Popen([sys.executable, "-W", "ignore", str(DRIVER), str(REF), *args], env=env,
                            stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)


def finish(proc, timeout=600):
    try:
        out, err = proc.communicate(timeout=timeout)
    except subprocess.TimeoutExpired:
        proc.kill()          # the exact process this test started
        out, err = proc.communicate()
        raise AssertionError(f"driver did not finish: {err[-2000:]}")
    assert proc.returncode == 0, err[-3000:]
    return out


@needs_reference
@pytest.mark.parametrize("swap_wait", ["0", "1"])
def test_unmodified_reference_worker_and_block_manager_on_the_gpu(tmp_path, built_libs, swap_wait):
    """One process: context tp=2 -> decoding tp=1,pp=2 reshard through ParaWorker.migrate_blocks, then a swap-out /
    swap-in round trip through BlockManager.swap_requests -> ParaWorker.swap_blocks.  With the default the data is
    made visible by a device synchronize (the worker's own swap event is recorded before the copies); with
    KVMIG_SWAP_WAIT=1 the operator itself waits and wait_for_all_swap_* is enough."""
    out = tmp_path / "single.json"
    finish(run_driver(["single", str(out)], {"KVMIG_SWAP_WAIT": swap_wait}))
    report = json.loads(out.read_text())
    assert report["lib_path"] == str(built_libs[1])
    assert str(REF) in report["worker_module"]                    # the reference's file, not this package's mirror
    assert report["pool_shapes"] == {"context": [48, 4, 4, 16, 32], "decoding": [40, 2, 8, 16, 32]}
    assert report["migrated_blocks"] == 25 and report["swapped_blocks"] == 8
    assert report["migrate_equal"] is True
    assert report["swap_out_equal"] is True and report["swap_in_equal"] is True
    assert report["swap_wait"] is (swap_wait == "1")


@needs_reference
def test_unmodified_reference_workers_in_two_processes(tmp_path, built_libs):
    """Each worker in its own process, seeing ONE GPU as cuda:0 (two GPUs when there are two), the handles
    travelling through a file: what the reference's Ray actors do."""
    n = torch.cuda.device_count()
    exchange = tmp_path / "exchange"
    exchange.mkdir()
    out = tmp_path / "dec.json"
    ctx = run_driver(["ctx", str(exchange)], {"CUDA_VISIBLE_DEVICES": "0"})
    dec = run_driver(["dec", str(exchange), str(out)], {"CUDA_VISIBLE_DEVICES": "1" if n >= 2 else "0"})
    try:
        finish(dec)
    finally:
        (exchange / "done").write_text("1")
        finish(ctx)
    report = json.loads(out.read_text())
    assert report["migrate_equal"] is True
    assert report["device_count"] == 1

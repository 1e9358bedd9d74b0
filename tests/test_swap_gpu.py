"""Block swap between the GPU pools and pinned host pools: parity with the
oracle through the C ABI and through the worker's stream/event protocol."""
import numpy as np
import pytest
import torch

from distserve_b200 import capi
from distserve_b200.block_manager import BlockManager
from distserve_b200.config import CacheConfig, KVModelConfig, ParallelConfig
from distserve_b200.request import Request
from distserve_b200.worker import KVWorker
from oracle import kv_oracle as O
from tests.kvutil import host_pool

pytestmark = pytest.mark.gpu


def make(seed, n_gpu, n_cpu, per_block=(2, 3, 4, 8)):
    hk, hv = host_pool([seed, 0], (n_gpu, *per_block)), host_pool([seed, 1], (n_gpu, *per_block))
    sk, sv = host_pool([seed, 2], (n_cpu, *per_block)), host_pool([seed, 3], (n_cpu, *per_block))
    gk, gv = torch.from_numpy(hk).cuda(), torch.from_numpy(hv).cuda()
    pk, pv = torch.from_numpy(sk.copy()).pin_memory(), torch.from_numpy(sv.copy()).pin_memory()
    return (hk, hv, sk, sv), (gk, gv, pk, pv)


def call_swap(src, dst, is_in, dev, stream=0):
    gk, gv, pk, pv = dev
    capi.swap(src, dst, is_in, gk.data_ptr(), gv.data_ptr(), capi.PoolShape.of(*gk.shape, 2), pk.data_ptr(), pv.data_ptr(),
              pk.shape[0], stream)


def check(host, dev):
    torch.cuda.synchronize()
    hk, hv, sk, sv = host
    gk, gv, pk, pv = dev
    assert np.array_equal(gk.cpu().numpy(), hk) and np.array_equal(gv.cpu().numpy(), hv)
    assert np.array_equal(pk.numpy(), sk) and np.array_equal(pv.numpy(), sv)


def test_swap_out_and_in_match_oracle():
    host, dev = make(1, 12, 9)
    rng = np.random.default_rng(1)
    for _ in range(6):
        n = int(rng.integers(1, 7))
        g_ids = [int(x) for x in rng.permutation(12)[:n]]
        c_ids = [int(x) for x in rng.permutation(9)[:n]]
        call_swap(g_ids, c_ids, False, dev)
        O.swap_numpy(g_ids, c_ids, False, *host)
        check(host, dev)
        g2 = [int(x) for x in rng.permutation(12)[:n]]
        call_swap(c_ids, g2, True, dev)
        O.swap_numpy(c_ids, g2, True, *host)
        check(host, dev)


def test_consecutive_ids_are_coalesced_and_still_exact():
    host, dev = make(2, 16, 16)
    calls = capi.get_counter("memcpy_calls")
    call_swap([3, 4, 5, 6, 9, 10, 1], [0, 1, 2, 3, 7, 8, 15], False, dev)     # runs of 4, 2, 1
    assert capi.get_counter("memcpy_calls") - calls == 3 * 2
    O.swap_numpy([3, 4, 5, 6, 9, 10, 1], [0, 1, 2, 3, 7, 8, 15], False, *host)
    check(host, dev)
    call_swap([], [], True, dev)
    check(host, dev)


def test_swap_refusals():
    host, dev = make(3, 4, 3)
    for src, dst, is_in, text in [([0], [0, 1], True, "entries"), ([3], [0], True, "outside the host pool"),
                                  ([0], [4], True, "outside the GPU pool"), ([4], [0], False, "outside the GPU pool"),
                                  ([0], [3], False, "outside the host pool")]:
        with pytest.raises(capi.KvmigError, match=text):
            call_swap(src, dst, is_in, dev)
    check(host, dev)


def test_worker_protocol_with_block_manager():
    """BlockManager drives KVWorker exactly as it drives the reference worker
    (it passes Request objects); a flush via wait_for_all_swap_* must be
    enough for the moved data to be in place."""
    model = KVModelConfig(4, 4, 16)
    cache = CacheConfig(4, 64)
    worker = KVWorker(0, "decoding", model, cache, ParallelConfig())
    worker.init_kvcache_and_swap(24, 24)
    torch.manual_seed(4)
    worker.k_cache.copy_(torch.randn(worker.k_cache.shape, device="cuda").half())
    worker.v_cache.copy_(torch.randn(worker.v_cache.shape, device="cuda").half())
    worker.k_swap.zero_()
    worker.v_swap.zero_()
    issued = []

    def call_all(name, *args):
        issued.append(name)
        return [getattr(worker, name)(*args)]

    bm = BlockManager("decoding", 24, 24, model, ParallelConfig(), cache, call_all)
    reqs = [Request.of_length(i, 4 * (2 + i)) for i in range(4)]     # 2,3,4,5 blocks
    for r in reqs:
        bm.allocate_blocks(r)
    snapshot = {r.request_id: (worker.k_cache[bm.get_block_table(r.request_id)].clone(),
                               worker.v_cache[bm.get_block_table(r.request_id)].clone()) for r in reqs}
    bm.swap_out_requests(reqs[:3])
    worker.wait_for_all_swap_out()
    for r in reqs[:3]:
        ids = bm.get_block_table(r.request_id)
        assert torch.equal(worker.k_swap[ids], snapshot[r.request_id][0].cpu())
        assert torch.equal(worker.v_swap[ids], snapshot[r.request_id][1].cpu())
    # overwrite the vacated GPU blocks, then bring two requests back
    worker.k_cache[list(bm.swapping_gpu_blocks_list)] = 0
    worker.v_cache[list(bm.swapping_gpu_blocks_list)] = 0
    bm.swap_in_requests([reqs[2], reqs[0]])
    worker.prepare_step([reqs[2].request_id, reqs[0].request_id])   # compute stream waits for the swap-in
    for r in (reqs[2], reqs[0]):
        ids = bm.get_block_table(r.request_id)
        assert torch.equal(worker.k_cache[ids], snapshot[r.request_id][0])
        assert torch.equal(worker.v_cache[ids], snapshot[r.request_id][1])
    assert worker.swap_event_table.keys() == {reqs[1].request_id}
    assert issued.count("swap_blocks") == 2
    worker.wait_for_all_swap_in()
    assert worker.latest_swap_in_event is None

"""Objects that the actor tests build inside spawned processes (they must be
importable by name from the child)."""
from __future__ import annotations

import os
import time


class Echo:
    def __init__(self, tag, fail_on_start=False):
        if fail_on_start:
            raise ValueError("refusing to start")
        self.tag = tag
        self.log = []

    def add(self, a, b, delay=0.0):
        time.sleep(delay)
        self.log.append((a, b))
        return a + b

    def history(self):
        return list(self.log)

    def fail(self, text):
        raise RuntimeError(text)

    def whoami(self):
        return self.tag, os.getpid(), os.environ.get("ACTOR_TEST_ENV")

    def die(self):
        os._exit(3)      # a rank that exits between steps, with no GPU work in flight


def make_kv_worker(worker_id, stage, layers, heads, head_dim, block_size, pc_list, device):
    """A KVWorker with two extra methods for the test's eyes: fill the pools
    from a seed, and read blocks back."""
    import torch

    from distserve_b200.config import CacheConfig, KVModelConfig, ParallelConfig
    from distserve_b200.worker import KVWorker

    class InspectableWorker(KVWorker):
        def fill(self, seed):
            g = torch.Generator(device="cpu").manual_seed(seed)
            for pool in (self.k_cache, self.v_cache):
                pool.copy_(torch.randn(pool.shape, generator=g).to(pool.dtype))
            torch.cuda.synchronize(self.device)

        def snapshot(self):
            return (self.k_cache.cpu().view(torch.int16).numpy(), self.v_cache.cpu().view(torch.int16).numpy())

    torch.cuda.set_device(device)
    tp, t, pp, p = pc_list
    return InspectableWorker(worker_id, stage, KVModelConfig(layers, heads, head_dim), CacheConfig(block_size, 1 << 20),
                             ParallelConfig(tp, t, pp, p), device=device)

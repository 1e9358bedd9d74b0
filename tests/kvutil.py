"""Shared helpers of the GPU parity tests: seeded pools on the device with a
host copy for the oracle, registration through the C ABI, comparison by bit
pattern."""
from __future__ import annotations

import numpy as np
import torch

from distserve_b200 import capi
from oracle import kv_oracle as O

NP_OF_SIZE = {1: np.int8, 2: np.int16, 4: np.int32, 8: np.int64}
TORCH_OF_SIZE = {1: torch.int8, 2: torch.int16, 4: torch.int32, 8: torch.int64}


def host_pool(seed, shape, elem_size=2):
    rng = np.random.default_rng(seed)
    dt = NP_OF_SIZE[elem_size]
    info = np.iinfo(dt)
    return rng.integers(info.min, info.max, size=shape, dtype=dt, endpoint=True)


class Stage:
    """All workers of one stage, living on one device of this process."""

    def __init__(self, L, H, tp, pp, num_blocks, B, D, elem_size=2, seed=0, device=0):
        self.L, self.H, self.tp, self.pp = L, H, tp, pp
        self.num_blocks, self.B, self.D, self.elem_size = num_blocks, B, D, elem_size
        self.device = torch.device("cuda", device)
        self.host = {}
        self.dev = {}
        for p in range(pp):
            for t in range(tp):
                shape = (num_blocks, L // pp, 1 if H == 1 else H // tp, B, D)     # one KV head: every rank holds it
                hk = host_pool([seed, p, t, 0], shape, elem_size)
                hv = host_pool([seed, p, t, 1], shape, elem_size)
                self.host[(p, t)] = (hk, hv)
                self.dev[(p, t)] = (torch.from_numpy(hk).to(self.device), torch.from_numpy(hv).to(self.device))

    def shape(self, key=(0, 0)):
        k = self.dev[key][0]
        return capi.PoolShape.of(*k.shape, k.element_size())

    def handles(self):
        """[pp][tp] -> (k_handle, v_handle), exported through the C ABI."""
        with torch.cuda.device(self.device):
            return [[tuple(capi.get_ipc_mem_handle(x.data_ptr(), self.shape((p, t))) for x in self.dev[(p, t)])
                     for t in range(self.tp)] for p in range(self.pp)]

    def download(self):
        return {key: (k.cpu().numpy(), v.cpu().numpy()) for key, (k, v) in self.dev.items()}


def register_all(ctx: Stage, dec: Stage, handles=None):
    handles = handles or ctx.handles()
    with torch.cuda.device(dec.device):
        for dp in range(dec.pp):
            for dt in range(dec.tp):
                for p in range(ctx.pp):
                    for t in range(ctx.tp):
                        kh, vh = handles[p][t]
                        capi.register_ipc_mem_handle(kh, vh, ctx.L, ctx.H, [ctx.tp, t, ctx.pp, p], [dec.tp, dt, dec.pp, dp])


def migrate_all(ctx: Stage, dec: Stage, src, dst, stream=0):
    """Every decoding worker pulls its share through the C ABI."""
    with torch.cuda.device(dec.device):
        for dp in range(dec.pp):
            for dt in range(dec.tp):
                k, v = dec.dev[(dp, dt)]
                capi.migrate_blocks(ctx.pp, ctx.tp, src, dec.pp, dec.tp, dp, dt, dst, k.data_ptr(), v.data_ptr(),
                                    dec.shape((dp, dt)), stream)


def oracle_all(ctx: Stage, dec: Stage, src, dst, fn=O.migrate_blocks_numpy):
    """Apply the oracle to the host copies of the decoding pools (in place)."""
    for dp in range(dec.pp):
        for dt in range(dec.tp):
            k, v = dec.host[(dp, dt)]
            fn(ctx.host, ctx.tp, ctx.pp, src, dec.tp, dt, dec.pp, dp, dst, k, v, ctx.L, ctx.H)


def assert_stage_equals_host(dec: Stage, what=""):
    got = dec.download()
    for key, (hk, hv) in dec.host.items():
        gk, gv = got[key]
        assert np.array_equal(gk, hk), f"{what}: K pool of decoding worker {key} differs from the oracle"
        assert np.array_equal(gv, hv), f"{what}: V pool of decoding worker {key} differs from the oracle"

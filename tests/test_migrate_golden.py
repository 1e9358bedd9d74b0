"""Committed digests of small seeded migrations: the oracle's sliced form must
reproduce them on CPU, the CUDA path must reproduce them on a GPU."""
import importlib.util
import json
from pathlib import Path

import pytest

from oracle import kv_oracle as O

GOLDEN = Path(__file__).resolve().parent / "golden"
spec = importlib.util.spec_from_file_location("make_migrate_golden", GOLDEN / "make_migrate_golden.py")
gen = importlib.util.module_from_spec(spec)
spec.loader.exec_module(gen)
DIGESTS = {row["name"]: row["sha256"] for row in json.loads((GOLDEN / "migrate_cases.json").read_text())}


@pytest.mark.parametrize("case", gen.CASES, ids=[c[0] for c in gen.CASES])
@pytest.mark.parametrize("form", ["numpy", "c"])
def test_oracle_reproduces_committed_digests(case, form):
    from oracle import kv_oracle_c as OC

    fn = O.migrate_blocks_numpy if form == "numpy" else OC.migrate_blocks_c
    name, L, H, (ctp, cpp), (dtp, dpp), *_ = case
    ctx, dec, src, dst = gen.build(case)
    for (p, t), (k, v) in dec.items():
        fn(ctx, ctp, cpp, src, dtp, t, dpp, p, dst, k, v, L, H)
    assert gen.digest(dec) == DIGESTS[name]


@pytest.mark.gpu
@pytest.mark.parametrize("kernel", [0, 1], ids=["auto", "vector"])
@pytest.mark.parametrize("case", gen.CASES, ids=[c[0] for c in gen.CASES])
def test_cuda_path_reproduces_committed_digests(case, kernel):
    import torch

    from distserve_b200 import capi

    name, L, H, (ctp, cpp), (dtp, dpp), B, D, elem, *_ = case
    ctx, dec, src, dst = gen.build(case)
    capi.reset_registry()
    capi.set_option("kernel", kernel)
    try:
        dev_ctx = {key: tuple(torch.from_numpy(a).cuda() for a in pair) for key, pair in ctx.items()}
        for (p, t), (k, v) in dev_ctx.items():
            shape = capi.PoolShape.of(*k.shape, elem)
            kh, vh = capi.get_ipc_mem_handle(k.data_ptr(), shape), capi.get_ipc_mem_handle(v.data_ptr(), shape)
            for dp in range(dpp):
                for dt in range(dtp):
                    capi.register_ipc_mem_handle(kh, vh, L, H, [ctp, t, cpp, p], [dtp, dt, dpp, dp])
        got = {}
        for (p, t), (k, v) in dec.items():
            dk, dv = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
            capi.migrate_blocks(cpp, ctp, src, dpp, dtp, p, t, dst, dk.data_ptr(), dv.data_ptr(),
                                capi.PoolShape.of(*dk.shape, elem))
            got[(p, t)] = (dk.cpu().numpy(), dv.cpu().numpy())
        assert gen.digest(got) == DIGESTS[name]
    finally:
        capi.set_option("kernel", 0)
        capi.reset_registry()

"""Writes migrate_cases.json: small seeded migration and swap cases with the
SHA-256 of the pools the oracle produces.  The oracle is the only source of the
expected bytes (the reference's native copy is not available to run), so these
digests pin the oracle against drift and give the CUDA path a committed target.

    python tests/golden/make_migrate_golden.py
"""
from __future__ import annotations

import hashlib
import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from oracle import kv_oracle as O  # noqa: E402

CASES = [
    # name, L, H, (ctx_tp, ctx_pp), (dec_tp, dec_pp), B, D, elem, src_blocks, dst_blocks, n, seed
    ("equal-layout", 4, 4, (1, 1), (1, 1), 4, 16, 2, 19, 17, 9, 101),
    ("gather-heads-tp2-to-tp1", 4, 8, (2, 1), (1, 1), 4, 16, 2, 23, 21, 12, 102),
    ("split-heads-tp1-to-tp2", 4, 8, (1, 1), (2, 1), 4, 16, 2, 23, 21, 12, 103),
    ("reshard-tp4pp1-to-tp2pp2", 8, 8, (4, 1), (2, 2), 4, 16, 2, 31, 29, 20, 104),
    ("layers-pp3-to-pp1", 6, 4, (1, 3), (2, 1), 2, 8, 2, 13, 11, 7, 105),
    ("fp32-odd-shape", 6, 6, (3, 2), (2, 3), 5, 3, 4, 13, 11, 7, 106),
]


def pool(seed, shape, elem):
    dt = {2: np.int16, 4: np.int32}[elem]
    info = np.iinfo(dt)
    return np.random.default_rng(seed).integers(info.min, info.max, size=shape, dtype=dt, endpoint=True)


def build(case):
    name, L, H, (ctp, cpp), (dtp, dpp), B, D, elem, nsrc, ndst, n, seed = case
    ctx = {(p, t): (pool([seed, p, t, 0], (nsrc, L // cpp, H // ctp, B, D), elem),
                    pool([seed, p, t, 1], (nsrc, L // cpp, H // ctp, B, D), elem)) for p in range(cpp) for t in range(ctp)}
    dec = {(p, t): (pool([seed, 9, p, t, 0], (ndst, L // dpp, H // dtp, B, D), elem),
                    pool([seed, 9, p, t, 1], (ndst, L // dpp, H // dtp, B, D), elem)) for p in range(dpp) for t in range(dtp)}
    rng = np.random.default_rng([seed, 77])
    src = [int(x) for x in rng.integers(0, nsrc, size=n)]
    dst = [int(x) for x in rng.permutation(ndst)[:n]]
    return ctx, dec, src, dst


def digest(pools):
    h = hashlib.sha256()
    for key in sorted(pools):
        for arr in pools[key]:
            h.update(np.ascontiguousarray(arr).tobytes())
    return h.hexdigest()


def expected(case):
    name, L, H, (ctp, cpp), (dtp, dpp), *_ = case
    ctx, dec, src, dst = build(case)
    for (p, t), (k, v) in dec.items():
        O.migrate_blocks_elementwise(ctx, ctp, cpp, src, dtp, t, dpp, p, dst, k, v, L, H)
    return digest(dec)


def main():
    out = [{"name": c[0], "sha256": expected(c)} for c in CASES]
    (HERE / "migrate_cases.json").write_text(json.dumps(out, indent=1))
    print(len(out), "cases")


if __name__ == "__main__":
    main()

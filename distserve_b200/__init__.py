"""B200-native paged-KV block migration and swap behind DistServe's operator API.

The package holds the CUDA library (``lib/libkvmig.so``, C ABI in
``include/kvmig.h``), the operator shim (``lib/libst_pybinding.so``) and the
host-side mirror of the reference classes that sit directly on that boundary
(``worker.KVWorker`` for ``distserve/worker.py``'s ParaWorker KV methods,
``block_manager.BlockManager`` for ``distserve/block_manager.py``).

There is no CPU fallback: every compute entry point needs the built libraries
and a CUDA device, and fails loudly without them.
"""
from __future__ import annotations

from pathlib import Path

_LIB_DIR = Path(__file__).resolve().parent / "lib"


def kvmig_library_path() -> Path:
    """Path of the C-ABI library; raises if it has not been built."""
    p = _LIB_DIR / "libkvmig.so"
    if not p.exists():
        raise RuntimeError(f"{p} is missing: build it with `python -m distserve_b200.build`")
    return p


def shim_library_path() -> Path:
    """Path of the operator shim (what SWIFT_TRANSFORMER_LIB_PATH should point at)."""
    p = _LIB_DIR / "libst_pybinding.so"
    if not p.exists():
        raise RuntimeError(f"{p} is missing: build it with `python -m distserve_b200.build`")
    return p


_ops_loaded = False


def load_ops() -> None:
    """Register torch.ops.block_migration_ops.* and torch.ops.swapping_ops.swap
    (what distserve/__init__.py:16 does with SwiftTransformer's library)."""
    global _ops_loaded
    if _ops_loaded:
        return
    import torch

    torch.ops.load_library(str(shim_library_path()))
    _ops_loaded = True

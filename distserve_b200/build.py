"""Builds the two shared libraries in-tree, next to this file, under ``lib/``:

* ``libkvmig.so``        — CUDA kernels + C ABI (``include/kvmig.h``), sm_100a only,
  no dependency on torch;
* ``libst_pybinding.so`` — the operator shim that registers the operator names the
  reference's Python layer calls and forwards to ``libkvmig.so``.

``python -m distserve_b200.build`` rebuilds whatever is older than its sources.
nvcc cross-compiles without a GPU, so this runs on a CPU-only machine.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "lib"
INCLUDE = ROOT / "include"

KVMIG_SO = LIB / "libkvmig.so"
SHIM_SO = LIB / "libst_pybinding.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xptxas", "-v",
    "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build libkvmig.so")
    return cand


def _stale(target: Path, sources) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in sources)


def _run(cmd, log_name: str) -> None:
    proc = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    (LIB / log_name).write_text("$ " + " ".join(str(c) for c in cmd) + "\n" + proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"build step failed ({log_name}):\n{proc.stdout}\n{proc.stderr}")


def build_kvmig(force: bool = False) -> Path:
    src = CSRC / "kvmig.cu"
    hdr = INCLUDE / "kvmig.h"
    LIB.mkdir(exist_ok=True)
    if force or _stale(KVMIG_SO, [src, hdr, CSRC / "kvmig_kernels.cuh"]):
        _run([_nvcc(), *NVCC_FLAGS, "-o", KVMIG_SO, src], "libkvmig.build.log")
    return KVMIG_SO


def build_shim(force: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension

    src = CSRC / "st_pybinding.cpp"
    hdr = INCLUDE / "kvmig.h"
    LIB.mkdir(exist_ok=True)
    if force or _stale(SHIM_SO, [src, hdr, KVMIG_SO]):
        torch_lib = Path(torch.__file__).resolve().parent / "lib"
        cuda_home = Path(_nvcc()).resolve().parent.parent
        cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC",
               f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
        for inc in cpp_extension.include_paths():
            cmd += ["-isystem", inc]
        cmd += ["-isystem", cuda_home / "include", "-o", SHIM_SO, src,
                f"-L{LIB}", "-lkvmig", f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch",
                "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}", "-Wl,--no-as-needed"]
        _run(cmd, "libst_pybinding.build.log")
    return SHIM_SO


def build_all(force: bool = False):
    return build_kvmig(force), build_shim(force)


if __name__ == "__main__":
    k, s = build_all(force="--force" in sys.argv)
    print(k)
    print(s)

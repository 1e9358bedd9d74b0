"""Compiles oracle/kv_oracle.c with gcc into oracle/_build/libkvoracle.so.

    python oracle/build_oracle.py

Test infrastructure: nothing in the shipped package depends on the result.
"""
from __future__ import annotations

import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_build" / "libkvoracle.so"


def build(force: bool = False) -> Path:
    src = HERE / "kv_oracle.c"
    if not force and OUT.exists() and OUT.stat().st_mtime >= src.stat().st_mtime:
        return OUT
    OUT.parent.mkdir(exist_ok=True)
    cmd = ["gcc", "-O3", "-fopenmp", "-fPIC", "-shared", "-Wall", "-o", str(OUT), str(src)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"gcc failed:\n{proc.stdout}\n{proc.stderr}")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))

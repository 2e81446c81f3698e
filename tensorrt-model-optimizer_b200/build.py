"""Ahead-of-time build of the CUDA library for sm_100a.

Compiles every ``csrc/*.cu`` with nvcc into ``b200q/_lib/libb200q.so`` (in-tree, next to the
Python package that loads it through ctypes).  Nothing is compiled at import time.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT_DIR = HERE / "b200q" / "_lib"
OBJ_DIR = HERE / "build"
LIB = OUT_DIR / "libb200q.so"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
# No fast-math: every result is specified in IEEE round-to-nearest arithmetic.
CFLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _compile(src: Path, headers: list[Path], verbose: bool) -> Path:
    obj = OBJ_DIR / (src.stem + ".o")
    if _stale(obj, [src, *headers]):
        cmd = [NVCC, *ARCH, *CFLAGS, "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        (OBJ_DIR / (src.stem + ".ptxas.txt")).write_text(res.stderr)
        if res.returncode != 0:
            sys.stderr.write(res.stderr)
            raise RuntimeError(f"nvcc failed for {src.name}")
        if verbose:
            print(f"compiled {src.name}")
    return obj


def build(verbose: bool = False) -> Path:
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "b200q.h"]
    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(lambda s: _compile(s, headers, verbose), sources))
    if _stale(LIB, objs):
        cmd = [NVCC, *ARCH, "-shared", "-o", str(LIB), *map(str, objs)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stderr)
            raise RuntimeError("link failed")
        if verbose:
            print(f"linked {LIB}")
    return LIB


if __name__ == "__main__":
    build(verbose=True)

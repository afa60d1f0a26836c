"""Builds librecpulse_b200.so in-tree with nvcc for sm_100a.

    python -m recpulse_b200.build [--verbose]

The library has no Python or PyTorch dependency; it links the CUDA runtime
statically, resolves the driver's tensor-map encoder at run time and looks NCCL up
with dlopen only when a sharded entry point is first used.  Translation units are
compiled side by side (one nvcc per source) and linked at the end.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "_obj")
LIB = os.path.join(PKG, "librecpulse_b200.so")
HEADER = os.path.join(PKG, "..", "include", "recpulse_b200.h")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.c")))


def _inputs() -> list[str]:
    """Everything a translation unit can include: any change rebuilds."""
    return _sources() + sorted(glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))) + [HEADER]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    return any(os.path.getmtime(f) > built for f in _inputs())


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile when sources are newer than the library; returns the library path."""
    if not force and not _stale():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        if os.path.exists(LIB):
            return LIB          # no compiler on this box: keep the prebuilt library
        raise RuntimeError("nvcc not found and no prebuilt librecpulse_b200.so")
    os.makedirs(OBJ, exist_ok=True)
    headers_time = max(os.path.getmtime(f) for f in _inputs() if not f.endswith((".cu", ".c")))

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ, os.path.basename(src) + ".o")
        if not force and os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(src), headers_time):
            return obj
        cmd = [nvcc, *ARCH, "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-Wall", "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd))
        subprocess.run(cmd, check=True)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, _sources()))
    subprocess.run([nvcc, *ARCH, "-shared", "-o", LIB, *objs, "-ldl"], check=True)
    return LIB


if __name__ == "__main__":
    build(force=True, verbose="--verbose" in sys.argv)
    print(LIB)

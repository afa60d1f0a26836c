"""Builds librecpulse_b200.so in-tree with nvcc for sm_100a.

    python -m recpulse_b200.build [--verbose]

The library has no Python or PyTorch dependency; it links the CUDA runtime
statically and resolves the driver's tensor-map encoder at run time.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "librecpulse_b200.so")
SOURCES = ["gemm_dispatch.cu", "host_pipeline.cu", "op_matmul.c"]
HEADERS = ["gemm_simt.cuh", "gemm_umma.cuh", "gemm_dmma.cuh", "gemm_tf32x3.cuh", "reduce_cols.cuh", "rpb_common.h",
           os.path.join("..", "..", "include", "recpulse_b200.h")]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > built for f in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile when sources are newer than the library; returns the library path."""
    if not force and not _stale():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        if os.path.exists(LIB):
            return LIB          # no compiler on this box: keep the prebuilt library
        raise RuntimeError("nvcc not found and no prebuilt librecpulse_b200.so")
    cmd = [nvcc, *ARCH, "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-Wall", "-shared",
           "-o", LIB, *[os.path.join(CSRC, s) for s in SOURCES], "-ldl"]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    build(force=True, verbose="--verbose" in sys.argv)
    print(LIB)

"""Builds libfhob.so (the C-ABI library) in-tree with nvcc for sm_100a.

Usage: python flash-hob_b200/build.py [--force] [--verbose]
The library lands next to the Python host module (fhob/libfhob.so) so it
travels with the source tree; nothing is installed into site-packages.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "fhob" / "libfhob.so"
SOURCES = ["fhob_api.cu", "simt_kernels.cu", "tc_kernels.cu", "tc_first_order.cu", "static_scratch.cu"]
HEADERS = ["fhob_common.cuh", "sm100_ptx.cuh", "tc_common.cuh", "../../include/fhob.h"]


def nvcc_path() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = Path(cuda_home) / "bin" / "nvcc"
    return str(cand) if cand.exists() else "nvcc"


def is_stale() -> bool:
    if not OUT.exists():
        return True
    t = OUT.stat().st_mtime
    deps = [CSRC / s for s in SOURCES] + [(CSRC / h).resolve() for h in HEADERS] + [Path(__file__)]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not is_stale():
        return OUT
    cmd = [
        nvcc_path(), "-shared", "-Xcompiler", "-fPIC", "-O3", "-std=c++17", "-lineinfo",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-o", str(OUT),
    ] + [str(CSRC / s) for s in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))

"""Builds libfhob.so (the C-ABI library) in-tree with nvcc for sm_100a.

Usage: python flash-hob_b200/build.py [--force] [--verbose]
The library lands next to the Python host module (fhob/libfhob.so) so it
travels with the source tree; nothing is installed into site-packages.
Each source file is compiled to an object of its own (in parallel, and only
when it or a header changed), then the objects are linked.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
OUT = HERE / "fhob" / "libfhob.so"
SOURCES = ["fhob_api.cu", "simt_kernels.cu", "tc_kernels.cu", "tc_first_order.cu", "static_scratch.cu"]
HEADERS = ["fhob_common.cuh", "sm100_ptx.cuh", "tc_common.cuh", "../../include/fhob.h"]
FLAGS = ["-Xcompiler", "-fPIC", "-O3", "-std=c++17", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a"]


def nvcc_path() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = Path(cuda_home) / "bin" / "nvcc"
    return str(cand) if cand.exists() else "nvcc"


def _newest_header() -> float:
    return max(p.stat().st_mtime for p in [(CSRC / h).resolve() for h in HEADERS] + [Path(__file__)])


def is_stale() -> bool:
    if not OUT.exists():
        return True
    t = OUT.stat().st_mtime
    return _newest_header() > t or any((CSRC / s).stat().st_mtime > t for s in SOURCES)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not is_stale():
        return OUT
    OBJ.mkdir(exist_ok=True)
    nvcc, hdr = nvcc_path(), _newest_header()
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src: str) -> Path:
        obj = OBJ / (Path(src).stem + ".o")
        if (force or verbose or not obj.exists()
                or obj.stat().st_mtime < max(hdr, (CSRC / src).stat().st_mtime)):
            subprocess.run([nvcc, "-c", *FLAGS, *extra, "-o", str(obj), str(CSRC / src)], check=True)
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    subprocess.run([nvcc, "-shared", *FLAGS, "-o", str(OUT)] + [str(o) for o in objs], check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))

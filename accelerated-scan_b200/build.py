"""Builds libascan_b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python accelerated-scan_b200/build.py [--force] [--verbose]

The shared library is written next to the Python package
(accelerated_scan/libascan_b200.so).  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "accelerated_scan", "libascan_b200.so")
SOURCES = ["api.cu", "planner.cpp", "inst_f32.cu", "inst_bf16.cu", "inst_f16.cu", "inst_c64.cu"]
HEADERS = sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))) + [
    os.path.join("..", "..", "include", "ascan_b200.h")]
OBJ_DIR = os.path.join(HERE, "build", "obj")


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; it is required to build libascan_b200.so")


def needs_build() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return OUT
    # one nvcc process per translation unit, all at once, then one link
    os.makedirs(OBJ_DIR, exist_ok=True)
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]
    if verbose:
        flags += ["-Xptxas", "-v"]
    jobs = []
    for src in SOURCES:
        obj = os.path.join(OBJ_DIR, os.path.splitext(src)[0] + ".o")
        cmd = [_nvcc()] + flags + ["-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            print(" ".join(cmd))
        jobs.append((cmd, obj, subprocess.Popen(cmd)))
    failed = [cmd for cmd, _, proc in jobs if proc.wait() != 0]
    if failed:
        raise RuntimeError("nvcc failed: " + " ".join(failed[0]))
    link = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", OUT] + [obj for _, obj, _ in jobs]
    subprocess.run(link, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))

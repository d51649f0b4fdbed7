"""Builds ``libphasekv_b200.so`` (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m phasekv_b200.build [--force] [--verbose]

The library is plain CUDA behind ``extern "C"`` entry points (include/phasekv_b200.h); it links
against nothing but the CUDA runtime, so the build is a single nvcc invocation.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_PATH = os.path.join(HERE, "libphasekv_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--shared",
    "-cudart", "shared",
    # No --use_fast_math: the quantiser relies on IEEE division and round-half-even.
]


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _inputs() -> list[str]:
    inc = os.path.join(HERE, "..", "include", "phasekv_b200.h")
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [inc]


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(p) > built for p in _inputs())


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA library of phasekv_b200 cannot be built")
    return nvcc


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return LIB_PATH
    extra = os.environ.get("PKV_NVCC_FLAGS", "").split()  # e.g. -DPKV_MMA_WARPS=16 for tuning experiments
    cmd = [find_nvcc(), *NVCC_FLAGS, *extra, *(["-Xptxas", "-v"] if verbose else []), "-o", LIB_PATH, *sources()]
    # nvcc hands host code to the compiler named by CC/CXX only if told to; use the system g++.
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    proc = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("nvcc failed building libphasekv_b200.so")
    if verbose:
        sys.stderr.write(proc.stdout + proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register/shared-memory usage")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))

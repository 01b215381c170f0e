"""Builds the CUDA library in-tree: csrc/*.cu -> libinkq.so (sm_100a only).

    python qwen3.ink.cpp_b200/build.py            # or  __graft_entry__.build()

nvcc cross-compiles without a GPU.  The ptxas resource report (registers, spills,
shared memory per kernel) is written to build/libinkq.ptxas.txt (not tracked).
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libinkq.so")
SHIM = os.path.join(HERE, "libinkq_refshim.so")


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target: str, sources) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_cuda(force: bool = False, verbose: bool = False) -> str:
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    deps = srcs + glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        [os.path.join(ROOT, "include", "inkq.h")]
    if not force and not _stale(LIB, deps):
        return LIB
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-Xptxas", "-v", "-Xcompiler", "-fPIC", "-shared", "-ccbin", "g++",
           "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-o", LIB] + srcs
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    res = subprocess.run(cmd, capture_output=True, text=True, env=env)
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    with open(os.path.join(HERE, "build", "libinkq.ptxas.txt"), "w") as f:
        f.write(res.stderr)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed")
    if verbose:
        print(res.stderr)
    return LIB


def build_shim(force: bool = False) -> str:
    """Host-side C++ drop-in layer (reference-named functions and the linear class helpers)."""
    srcs = sorted(glob.glob(os.path.join(HERE, "host", "*.cc")))
    deps = srcs + glob.glob(os.path.join(HERE, "host", "*.h")) + [os.path.join(ROOT, "include", "inkq.h")]
    if not srcs:
        return ""
    if not force and not _stale(SHIM, deps) and not _stale(SHIM, [LIB]):
        return SHIM
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-I", os.path.join(ROOT, "include"),
           "-I", os.path.join(HERE, "host"), "-o", SHIM] + srcs + ["-L", HERE, "-linkq", "-Wl,-rpath,$ORIGIN"]
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    res = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("g++ failed building the host shim")
    return SHIM


def build_all(force: bool = False) -> None:
    build_cuda(force)
    build_shim(force)


if __name__ == "__main__":
    build_cuda(force="--force" in sys.argv, verbose=True)
    build_shim(force="--force" in sys.argv)
    print("built", LIB)

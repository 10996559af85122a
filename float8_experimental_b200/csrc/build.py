"""Builds libf8b200.so (the C-ABI kernel library) in-tree with nvcc for sm_100a.

Usage: python -m float8_experimental_b200.csrc.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libf8b200.so")
SOURCES = ["capi.cu", "cast.cu", "gemm.cu", "norm.cu", "reduce.cu"]
# Single-GPU extra: the cluster-multicast GEMM lives in a library of its own, so that runs on
# several GPUs can leave its source and binary out altogether (it includes gemm.cu).
MC_LIB_PATH = os.path.join(LIB_DIR, "libf8b200_mc.so")
MC_SOURCES = ["capi.cu", "gemm_mc.cu"]
HEADERS = ["common.cuh", os.path.join("..", "..", "include", "f8b200.h")]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if os.path.exists(cand):
        return cand
    found = shutil.which("nvcc")
    if found is None:
        raise RuntimeError("nvcc not found: set CUDA_HOME or put nvcc on PATH")
    return found


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(HERE, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > built for d in deps)


def _compile(sources, out_path, verbose, extra=()):
    cmd = [
        _nvcc(),
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-O3", "-std=c++17", "-lineinfo",
        "-Xcompiler", "-fPIC", "-shared", *extra,
        "-o", out_path,
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(HERE, s) for s in sources]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed building {os.path.basename(out_path)}")


def build_mc(force: bool = False, verbose: bool = False):
    """Compiles the single-GPU multicast GEMM library when its source is present; returns its
    path, or None when the source was left out."""
    src = os.path.join(HERE, "gemm_mc.cu")
    if not os.path.exists(src):
        return None
    deps = [os.path.join(HERE, s) for s in MC_SOURCES + ["gemm.cu"] + HEADERS] + [os.path.abspath(__file__)]
    if not force and os.path.exists(MC_LIB_PATH) and all(os.path.getmtime(d) <= os.path.getmtime(MC_LIB_PATH) for d in deps):
        return MC_LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    # hidden visibility: only the f8b200_mc_* entry points leave this library, so the copy of gemm.cu
    # it includes cannot interpose the symbols of libf8b200.so
    _compile(MC_SOURCES, MC_LIB_PATH, verbose, extra=("-Xcompiler", "-fvisibility=hidden"))
    return MC_LIB_PATH


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles the library if it is missing or older than its sources; returns its path."""
    build_mc(force, verbose)
    if not force and not _stale():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    _compile(SOURCES, LIB_PATH, verbose)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))

"""Builds the CUDA library of the sampler in-tree: ``ferro_b200/lib/libferro_sampler_b200.so``.

nvcc cross-compiles for sm_100a without a GPU.  The library has no dependency on PyTorch; the CUDA runtime is
linked statically so it can live in one process with any other CUDA user.
"""
from __future__ import annotations

import os
import shutil
import subprocess

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libferro_sampler_b200.so")
SOURCES = ["fsb_stream.cu", "fsb_fullrow.cu", "fsb_support.cu", "fsb_shim.cpp", "fsb_request.cpp"]
HEADERS = ["fsb_internal.h", "fsb_device.cuh", os.path.join("..", "..", "include", "ferro_sampler_b200.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-cudart", "static", "-shared",
]


def nvcc_path() -> str:
    p = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(p):
        raise FileNotFoundError("nvcc not found; the sampler library cannot be built on this machine")
    return p


def is_fresh() -> bool:
    if not os.path.exists(LIB_PATH):
        return False
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    return all(os.path.getmtime(d) <= t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and is_fresh():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [nvcc_path(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-x", "cu"]
    cmd += [os.path.join(CSRC, f) for f in SOURCES]
    cmd += ["-o", LIB_PATH]
    subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == "__main__":
    import sys
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))

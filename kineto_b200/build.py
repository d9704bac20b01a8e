"""Builds libk2j.so (the CUDA library behind include/k2j.h) in-tree with nvcc for sm_100a."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libk2j.so")
SRC = os.path.join(HERE, "csrc", "k2j.cu")
SRC_NOALLOC = os.path.join(HERE, "csrc", "k2j_noalloc.cu")
SRC_NAMES = os.path.join(HERE, "csrc", "k2j_names.cpp")
DEPS = [SRC, SRC_NOALLOC, SRC_NAMES] + [os.path.join(HERE, "csrc", f) for f in ("k2j_kernels.cuh", "k2j_format.cuh", "k2j_sink.cuh", "k2j_sort.cuh", "k2j_pow10.h", "k2j_cupti_sizes.h")] + [
    os.path.join(os.path.dirname(HERE), "include", "k2j.h")]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(d) > t for d in DEPS)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    cmd = [nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "--shared", "-Xcompiler", "-fPIC", "-Xptxas", "-v", "-o", LIB, SRC, SRC_NOALLOC, SRC_NAMES, "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed")
    return LIB


if __name__ == "__main__":
    build(force=True, verbose=True)

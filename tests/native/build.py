"""Builds the TEST-ONLY native library `tests/native/libissm_b200_selftest.so` (sm_100a): the tcgen05
building-block self-check and the bounded-wait check.  None of it is linked into the product library.

    python -m tests.native.build [--force]
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "umma_selftest.cu")
LIB = os.path.join(HERE, "libissm_b200_selftest.so")
DEPS = [SRC, os.path.join(HERE, "..", "..", "dest3d_b200", "csrc", "umma.cuh")]


def build(force=False):
    if not force and os.path.exists(LIB) and all(os.path.getmtime(d) <= os.path.getmtime(LIB) for d in DEPS):
        return LIB
    nvcc = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
           "-shared", SRC, "-o", LIB]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building the self-test library")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))

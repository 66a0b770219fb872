"""Builds the C-ABI shared library `libissm_b200.so` for sm_100a with nvcc, in-tree.

    python -m dest3d_b200.build            # build if sources are newer than the library
    python -m dest3d_b200.build --force
"""
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libissm_b200.so")
SOURCES = ["issm_abi.cu", "issm_simt.cu", "issm_norm.cu", "issm_tensor.cu", "issm_tensor_bwd.cu", "umma_selftest.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared", "-Xptxas", "-v"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put it on PATH)")


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(PKG, "..", "include", "issm_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compile every CUDA source of the package into libissm_b200.so; returns the library path.
    The sources are compiled to objects side by side (the two tensor-core files dominate the build time),
    then linked."""
    if not force and not _stale():
        return LIB
    from concurrent.futures import ThreadPoolExecutor
    nvcc = _nvcc()
    objdir = os.path.join(PKG, "_obj")
    os.makedirs(objdir, exist_ok=True)
    cflags = [f for f in NVCC_FLAGS if f != "-shared"]

    def compile_one(src):
        obj = os.path.join(objdir, os.path.splitext(src)[0] + ".o")
        res = subprocess.run([nvcc] + cflags + ["-c", os.path.join(CSRC, src), "-o", obj], capture_output=True, text=True)
        return src, obj, res

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        results = list(pool.map(compile_one, SOURCES))
    log = "".join(f"---- {src}\n{res.stdout}{res.stderr}" for src, _, res in results)
    failed = [src for src, _, res in results if res.returncode]
    if verbose or failed:
        sys.stderr.write(log)
    if failed:
        raise RuntimeError("nvcc failed compiling " + ", ".join(failed))
    link = subprocess.run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a"] + [obj for _, obj, _ in results] +
                          ["-lcuda", "-o", LIB], capture_output=True, text=True)
    if verbose or link.returncode:
        sys.stderr.write(link.stdout + link.stderr)
    if link.returncode:
        raise RuntimeError("nvcc failed linking libissm_b200.so")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))

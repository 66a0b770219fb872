"""Builds, in-tree, the C-ABI shared library `libissm_b200.so` (CUDA kernels, sm_100a, nvcc) and the torch C++
extension `libissm_b200_torch.so` (TORCH_LIBRARY ops over that C ABI, host code only, g++).

    python -m dest3d_b200.build            # build what is older than its sources
    python -m dest3d_b200.build --force
"""
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libissm_b200.so")
TORCH_LIB = os.path.join(PKG, "libissm_b200_torch.so")
TORCH_SRC = os.path.join(CSRC, "issm_torch.cpp")
SOURCES = ["issm_abi.cu", "issm_simt.cu", "issm_norm.cu", "issm_tensor.cu", "issm_tensor_bwd.cu", "issm_pointops.cu", "issm_seqpar.cu", "issm_glue.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared", "-Xptxas", "-v"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put it on PATH)")


HEADER = os.path.join(PKG, "..", "include", "issm_b200.h")


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if not f.endswith(".cpp")] + [HEADER]
    return any(os.path.getmtime(d) > t for d in deps)


def build_torch_extension(force=False, verbose=False):
    """Compile csrc/issm_torch.cpp against the installed torch and link it to libissm_b200.so (found next to
    it at run time through an $ORIGIN rpath).  Returns the extension's path."""
    if (not force and os.path.exists(TORCH_LIB)
            and all(os.path.getmtime(d) <= os.path.getmtime(TORCH_LIB) for d in (TORCH_SRC, HEADER, LIB))):
        return TORCH_LIB
    import torch
    from torch.utils import cpp_extension as ce
    cuda_home = os.environ.get("CUDA_HOME") or "/usr/local/cuda"
    # the host compiler nvcc itself uses (g++ on PATH), so that the extension shares the process-wide libstdc++ with
    # torch: a compiler that links its own C++ runtime statically breaks exceptions thrown across the libraries
    cmd = ([os.environ.get("ISSM_B200_CXX") or shutil.which("g++") or "g++", "-O2", "-std=c++17", "-fPIC", "-shared",
            f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", TORCH_SRC]
           + [f"-I{d}" for d in ce.include_paths()] + [f"-I{os.path.join(cuda_home, 'include')}"]
           + [f"-L{d}" for d in ce.library_paths()] + ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
              f"-L{PKG}", "-lissm_b200", "-Wl,-rpath,$ORIGIN", "-o", TORCH_LIB])
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode:
        raise RuntimeError("g++ failed building libissm_b200_torch.so")
    needed = subprocess.run(["readelf", "-d", TORCH_LIB], capture_output=True, text=True).stdout
    if needed and "libstdc++" not in needed:
        os.remove(TORCH_LIB)
        raise RuntimeError("libissm_b200_torch.so was linked without the shared libstdc++ (static C++ runtime): "
                           "point ISSM_B200_CXX at the system g++")
    return TORCH_LIB


def build(force=False, verbose=False):
    """Compile every CUDA source of the package into libissm_b200.so, then the torch extension; returns the
    path of the C-ABI library.  The CUDA sources are compiled to objects side by side (the two tensor-core
    files dominate the build time), then linked."""
    _build_cabi(force, verbose)
    build_torch_extension(force, verbose)
    return LIB


def _build_cabi(force, verbose):
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

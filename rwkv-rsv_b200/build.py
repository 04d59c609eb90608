"""In-tree build of the native libraries (no pip, no JIT cache).

  librsv_b200.so   hand-written sm_100a CUDA kernels + the C ABI declared in include/rsv_b200.h
  librsv_synth.so  CPU-only seeded synthetic-checkpoint writer (csrc/synth.cpp)

`python -m rwkv_rsv_b200.build` builds both; nvcc cross-compiles without a GPU.
"""
import glob
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
ROOT = os.path.dirname(PKG)
LIB_CUDA = os.path.join(PKG, "librsv_b200.so")
LIB_SYNTH = os.path.join(PKG, "librsv_synth.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-fopenmp", "-shared", "-I", os.path.join(ROOT, "include"), "-I", CSRC,
]


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def build_synth(force=False):
    srcs = [os.path.join(CSRC, "synth.cpp"), os.path.join(CSRC, "safetensors.hpp")]
    if force or _stale(LIB_SYNTH, srcs):
        subprocess.check_call(["g++", "-O2", "-std=c++17", "-fopenmp", "-shared", "-fPIC", srcs[0], "-o", LIB_SYNTH])
    return LIB_SYNTH


def build_cuda(force=False, verbose=False):
    cu = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    deps = cu + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.hpp")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    if force or _stale(LIB_CUDA, deps):
        extra = os.environ.get("RSV_NVCC_EXTRA", "").split()  # e.g. -DRSV_DS_DEBUG: phase time stamps of the batch-1 decode kernel
        cmd = [_nvcc()] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + cu + ["-o", LIB_CUDA]
        env = dict(os.environ)
        env["CXX"] = "g++"
        subprocess.check_call(cmd + ["-ccbin", "g++"], env=env)
    return LIB_CUDA


def build_all(force=False, verbose=False):
    return build_synth(force), build_cuda(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built", LIB_SYNTH, LIB_CUDA)

"""Builds libvmcuda.so (the CUDA engine and its C ABI) in-tree for sm_100a with nvcc.

    python -m visualmesh_b200.build            # build if sources are newer than the library
    python -m visualmesh_b200.build --force

-fmad=false and -ffp-contract=off are part of the contract: the projection arithmetic must round every operation
the way the reference CPU engine does. The graph-convolution kernels call fmaf() explicitly.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libvmcuda.so")
SOURCES = ["engine.cu", "hostmesh.cpp"]
HEADERS = ["kernels.cuh", "conv_tc.cuh", "device_math.cuh", "host_math.hpp", "libm_tables.hpp", os.path.join("..", "..", "include", "vmcuda.h")]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    for f in SOURCES + HEADERS:
        p = os.path.join(CSRC, f)
        if os.path.exists(p) and os.path.getmtime(p) > t:
            return True
    return False


def build(force=False, verbose=False):
    if not force and not needs_build():
        return LIB
    srcs = [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "-fmad=false",
           "-Xcompiler", "-fPIC,-ffp-contract=off,-fvisibility=hidden", "-shared", "-o", LIB] + srcs
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    subprocess.run(cmd, check=True, cwd=CSRC)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))

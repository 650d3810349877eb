"""Builds libvmcuda.so (the CUDA engine and its C ABI) in-tree for sm_100a with nvcc.

    python -m visualmesh_b200.build            # rebuild what is older than its sources
    python -m visualmesh_b200.build --force [-v]

Every translation unit is compiled to an object file of its own (in parallel) and the objects are linked into the
library; a unit is recompiled when it or one of the headers it includes is newer than its object.
-fmad=false and -ffp-contract=off are part of the contract: the projection arithmetic must round every operation
the way the reference CPU engine does. The graph-convolution kernels call fmaf() explicitly.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_build")
LIB = os.path.join(HERE, "libvmcuda.so")
ABI_HEADER = os.path.join("..", "..", "include", "vmcuda.h")
# translation unit -> headers it includes (directly or not)
UNITS = {
    "engine.cu": ["kernels.cuh", "tile_plan.cuh", "device_math.cuh", "host_math.hpp", "libm_tables.hpp", "conv_dispatch.hpp", "conv_args.hpp",
                  ABI_HEADER],
    "conv_ffma.cu": ["conv_ffma.cuh", "conv_common.cuh", "conv_dispatch.hpp", "conv_args.hpp", ABI_HEADER],
    "conv_tc.cu": ["conv_tc.cuh", "conv_common.cuh", "conv_dispatch.hpp", "conv_args.hpp", ABI_HEADER],
    "conv_staged.cu": ["conv_staged.cuh", "tile_plan.cuh", "conv_tc.cuh", "conv_common.cuh", "conv_dispatch.hpp", "conv_args.hpp", ABI_HEADER],
    "hostmesh.cpp": ["host_math.hpp", ABI_HEADER],
}


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def _obj(unit):
    return os.path.join(OBJ, os.path.splitext(unit)[0] + ".o")


def _stale(unit):
    obj = _obj(unit)
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > t for f in [unit] + UNITS[unit]
               if os.path.exists(os.path.join(CSRC, f)))


def needs_build():
    """The library is missing or older than one of its sources (object files may be absent: they do not travel)."""
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    files = {f for u in UNITS for f in [u] + UNITS[u]}
    return any(os.path.getmtime(os.path.join(CSRC, f)) > t for f in files if os.path.exists(os.path.join(CSRC, f)))


def build(force=False, verbose=False):
    if not force and not needs_build():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "-fmad=false",
             "-Xcompiler", "-fPIC,-ffp-contract=off,-fvisibility=hidden"]
    if verbose:
        flags += ["-Xptxas", "-v"]

    def compile_unit(unit):
        out = subprocess.run([_nvcc()] + flags + ["-c", os.path.join(CSRC, unit), "-o", _obj(unit)], cwd=CSRC,
                             capture_output=True, text=True)
        return unit, out

    todo = [u for u in UNITS if force or _stale(u)]
    with ThreadPoolExecutor(max_workers=max(1, min(len(todo), os.cpu_count() or 1))) as pool:
        for unit, out in pool.map(compile_unit, todo):
            if verbose or out.returncode != 0:
                sys.stderr.write(f"---- {unit}\n{out.stdout}{out.stderr}")
            if out.returncode != 0:
                raise subprocess.CalledProcessError(out.returncode, f"nvcc -c {unit}")
    subprocess.run([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB] + [_obj(u) for u in UNITS],
                   check=True, cwd=CSRC)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))

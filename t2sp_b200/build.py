"""Builds libt2sp_b200.so in-tree with nvcc for sm_100a (no JIT cache, no pip install).

Run as `python -m t2sp_b200.build` or through `__graft_entry__.build()`. The shared
library carries the CUDA kernels and the C ABI declared in include/t2sp_b200/runtime.h.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libt2sp_b200.so")

SOURCES = ["umma_launch.cu", "host_rt.cpp", "errors.cpp", "halide_rt.cpp", "ops.cpp", "noalloc.cu"]


def _nvcc():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build t2sp_b200")
    return nvcc


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps += [os.path.join(ROOT, "include", "t2sp_b200", f) for f in os.listdir(os.path.join(ROOT, "include", "t2sp_b200"))]
    return any(os.path.getmtime(d) > t for d in deps if os.path.isfile(d))


def build(force=False, verbose=False):
    if not force and not needs_build():
        return LIB
    cmd = [
        _nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-Xcompiler", "-fPIC,-fvisibility=default", "-shared", "-cudart", "static",
        "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-x", "cu",
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    cmd += ["-o", LIB]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building libt2sp_b200.so")
    if verbose:
        sys.stderr.write(res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))

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

EXTRA_LINK = ["-ldl"]
SOURCES = ["launch_core.cu", "launch_core_x3.cu", "launch_pair.cu", "launch_x3pair.cu", "launch_x3tm.cu", "launch_mttkrp.cu", "umma_launch.cu", "host_rt.cpp", "errors.cpp", "halide_rt.cpp", "ops.cpp", "multigpu.cpp", "noalloc.cu"]


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
    """Compiles the sources side by side into objects (a scratch folder outside the tree), then links."""
    if not force and not needs_build():
        return LIB
    import concurrent.futures
    import hashlib
    import tempfile
    obj_dir = os.path.join(tempfile.gettempdir(), "t2sp_b200_obj_" + hashlib.sha1(ROOT.encode()).hexdigest()[:10])
    os.makedirs(obj_dir, exist_ok=True)
    common = [
        _nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-Xcompiler", "-fPIC,-fvisibility=default", "-cudart", "static",
        "-I", os.path.join(ROOT, "include"), "-I", CSRC,
    ]
    if verbose:
        common += ["-Xptxas", "-v"]
    newest_header = max(os.path.getmtime(os.path.join(d, f))
                        for d in (CSRC, os.path.join(ROOT, "include", "t2sp_b200"))
                        for f in os.listdir(d) if f.endswith((".h", ".cuh")))

    def compile_one(src):
        path = os.path.join(CSRC, src)
        obj = os.path.join(obj_dir, src + ".o")
        if not force and os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(path), newest_header):
            return obj, None
        res = subprocess.run(common + ["-x", "cu", "-c", path, "-o", obj], capture_output=True, text=True)
        return obj, res

    objs = []
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        for obj, res in pool.map(compile_one, SOURCES):
            if res is not None and res.returncode != 0:
                sys.stderr.write(res.stdout + res.stderr)
                raise RuntimeError("nvcc failed building libt2sp_b200.so")
            if res is not None and verbose:
                sys.stderr.write(res.stderr)
            objs.append(obj)
    res = subprocess.run(common + ["-shared"] + objs + ["-o", LIB] + EXTRA_LINK, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed linking libt2sp_b200.so")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))

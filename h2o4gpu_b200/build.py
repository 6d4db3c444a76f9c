"""Builds libh2o4gpu_kmeans.so for sm_100a with nvcc, in-tree (h2o4gpu_b200/lib/).

Usage: python -m h2o4gpu_b200.build [--force] [--verbose]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIBDIR, "libh2o4gpu_kmeans.so")
SOURCES = ["kmeans_api.cu", "kmeans_noalloc.cu"]


def _nccl_include():
    for p in ("/usr/include",):
        if os.path.exists(os.path.join(p, "nccl.h")):
            return []
    try:
        import nvidia.nccl  # type: ignore
        inc = os.path.join(os.path.dirname(nvidia.nccl.__file__), "include")
        if os.path.exists(os.path.join(inc, "nccl.h")):
            return ["-I" + inc]
    except Exception:
        pass
    return []


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(HERE, "..", "include", "h2o4gpu_kmeans.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    if not force and not _stale():
        return LIB
    os.makedirs(LIBDIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-shared", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
           "-o", LIB] + _nccl_include() + [os.path.join(CSRC, s) for s in SOURCES] + ["-ldl"]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(LIB)

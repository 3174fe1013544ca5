"""Builds ruquant_b200/librq_b200.so (the C-ABI library of include/rq_b200.h) with nvcc for sm_100a, in-tree.

    python -m ruquant_b200.build [--force] [-v]

RQ_NVCC_EXTRA in the environment adds compiler flags (e.g. -DRQ_TRACE for the kernels' timeline diagnostics);
RQ_B200_LIB names another output file (the package loads the same variable), for side-by-side builds.

nvcc cross-compiles without a GPU.  The library links the CUDA runtime statically and has no other dependency
(no torch, no libcuda at link time: the one driver entry point it needs is fetched through the runtime).
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.environ.get("RQ_B200_LIB") or os.path.join(HERE, "librq_b200.so")
SOURCES = ["rq_api.cu", "rq_act.cu", "rq_prepack.cu", "rq_gemv.cu", "rq_gemm_tc.cu", "rq_static.cu", "rq_wquant.cu", "rq_rank.cu"]
NVCC_FLAGS = ["-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-fmad=false",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-cudart", "static"]


def _newest_source():
    t = 0.0
    for root in (CSRC, os.path.join(HERE, "..", "include")):
        for name in os.listdir(root):
            t = max(t, os.path.getmtime(os.path.join(root, name)))
    return t


def build(force=False, verbose=False):
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_source():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objs = []
    procs = []
    for src in SOURCES:
        path = os.path.join(CSRC, src)
        if not os.path.exists(path):
            continue
        # a side-by-side build keeps its objects next to its own output file
        obj = (os.path.join(CSRC, src[:-3] + ".o") if not os.environ.get("RQ_B200_LIB")
               else os.path.join(os.path.dirname(os.path.abspath(LIB)), src[:-3] + "." + os.path.basename(LIB) + ".o"))
        cmd = ([nvcc] + NVCC_FLAGS + os.environ.get("RQ_NVCC_EXTRA", "").split() + (["-Xptxas", "-v"] if verbose else [])
               + ["-c", path, "-o", obj])
        procs.append((cmd, subprocess.Popen(cmd)))
        objs.append(obj)
    for cmd, p in procs:
        if p.wait() != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    link = [nvcc, "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs
    subprocess.check_call(link)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))

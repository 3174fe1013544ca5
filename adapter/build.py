"""Compiles the ggml-cuda adapter (rq-w4a4.cu) against the reference's vendored ggml headers and links it with the test
harness (ggml_shim.cu) and librq_b200.so into adapter/_build/librq_ggml_shim.so.

    python adapter/build.py

The ggml headers are not part of this repository: they are taken from the reference tree (third_party/llama.cpp/ggml),
looked for at $RQ_REFERENCE_DIR or beside this repository (../reference).  Where the tree is absent nothing is built and
the adapter's tests skip; the built library travels with the repository's other built files.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT_DIR = os.path.join(HERE, "_build")
SHIM_SO = os.path.join(OUT_DIR, "librq_ggml_shim.so")
ADAPTER_O = os.path.join(OUT_DIR, "rq-w4a4.o")


def reference_ggml():
    base = os.environ.get("RQ_REFERENCE_DIR") or os.path.normpath(os.path.join(ROOT, "..", "reference"))
    ggml = os.path.join(base, "third_party", "llama.cpp", "ggml")
    return ggml if os.path.exists(os.path.join(ggml, "src", "ggml-cuda", "common.cuh")) else None


def build(force=False):
    ggml = reference_ggml()
    if ggml is None:
        return None
    srcs = [os.path.join(HERE, n) for n in ("rq-w4a4.cu", "rq-w4a4.cuh", "ggml_shim.cu")] + [os.path.join(ROOT, "include", "rq_b200.h")]
    if not force and os.path.exists(SHIM_SO) and os.path.getmtime(SHIM_SO) >= max(os.path.getmtime(s) for s in srcs):
        return SHIM_SO
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    flags = ["-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-Xcompiler", "-fPIC",
             "-I" + os.path.join(ggml, "include"), "-I" + os.path.join(ggml, "src"), "-I" + os.path.join(ggml, "src", "ggml-cuda"),
             "-I" + os.path.join(ROOT, "include"), "-I" + HERE]
    shim_o = os.path.join(OUT_DIR, "ggml_shim.o")
    subprocess.check_call([nvcc] + flags + ["-c", os.path.join(HERE, "rq-w4a4.cu"), "-o", ADAPTER_O])
    subprocess.check_call([nvcc] + flags + ["-c", os.path.join(HERE, "ggml_shim.cu"), "-o", shim_o])
    lib_dir = os.path.join(ROOT, "ruquant_b200")
    subprocess.check_call([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", SHIM_SO, ADAPTER_O, shim_o,
                           "-L" + lib_dir, "-lrq_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../ruquant_b200",
                           "-Xlinker", "-z", "-Xlinker", "defs"])
    return SHIM_SO


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))

"""Builds libes_b200.so (sm_100a) in-tree with nvcc.

usage: python -m einsummable_b200.build [--force] [--trace]

--trace builds lib/libes_b200_trace.so instead: the same library with the contraction kernel's
clock trace compiled in (see einsummable_b200/trace.py); the product library is not touched.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libes_b200.so")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")

SOURCES = ["api.cc", "scalarop.cc", "einsum.cc", "codegen.cc", "jit.cc", "kernels.cu", "contraction.cu", "attention.cu", "noalloc.cu", "exchange.cu", "program.cc", "storage.cc", "wire.cc"]


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(ROOT, "include", "es_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps)


TRACE_LIB = os.path.join(LIB_DIR, "libes_b200_trace.so")


def build(force=False, verbose=False, trace=False):
    if not trace and not force and not _stale():
        return LIB
    os.makedirs(LIB_DIR, exist_ok=True)
    nvcc = os.path.join(CUDA_HOME, "bin", "nvcc")
    cmd = [
        nvcc, "-std=c++17", "-O3", "-lineinfo",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-ccbin", "/usr/bin/g++",
        "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function",
        "-Xptxas", "-v" if verbose else "-O3",
        "-shared", "-cudart", "static",
        "-I", os.path.join(ROOT, "include"), "-I", CSRC,
        "-o", TRACE_LIB if trace else LIB,
    ] + (["-DES_B200_TRACE"] if trace else []) + [os.path.join(CSRC, s) for s in SOURCES] + [
        "-L", os.path.join(CUDA_HOME, "lib64"), "-lnvrtc",
        "-Xlinker", "-rpath," + os.path.join(CUDA_HOME, "lib64"),
    ]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building libes_b200.so")
    if verbose:
        sys.stderr.write(res.stdout + res.stderr)
    return TRACE_LIB if trace else LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, trace="--trace" in sys.argv))

"""Builds the CUDA library in-tree: csrc/*.cu -> dciknn_cuda_b200/libdci_b200.so.

nvcc only (no torch headers): the library exposes the C ABI of
include/dci_b200.h and is loaded with ctypes.  sm_100a is the only target.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libdci_b200.so")

NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-shared", "-Xcompiler", "-fPIC"]


def _sources():
    srcs = []
    for root, _, files in os.walk(CSRC):
        srcs += [os.path.join(root, f) for f in files if f.endswith((".cu", ".cuh", ".h"))]
    srcs.append(os.path.join(os.path.dirname(HERE), "include", "dci_b200.h"))
    return srcs


def build(force=False, verbose=False):
    srcs = _sources()
    if not force and os.path.exists(LIB):
        t = os.path.getmtime(LIB)
        if all(os.path.getmtime(s) <= t for s in srcs):
            return LIB
    cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + \
          [os.path.join(CSRC, "dci_b200.cu"), "-o", LIB]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))

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


SHIM = os.path.join(HERE, "_dci_b200.so")


def build_torch_shim(force=False):
    """Compiles csrc/torch_shim.cpp (pybind11 + torch headers, host code only) into
    dciknn_cuda_b200/_dci_b200.so, linked against libdci_b200.so next to it."""
    src = os.path.join(CSRC, "torch_shim.cpp")
    header = os.path.join(os.path.dirname(HERE), "include", "dci_b200.h")
    if not force and os.path.exists(SHIM) and all(os.path.getmtime(p) <= os.path.getmtime(SHIM) for p in (src, header)):
        return SHIM
    build(force=False)
    import sysconfig
    import torch
    from torch.utils import cpp_extension
    inc = cpp_extension.include_paths(device_type="cuda")
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-DTORCH_EXTENSION_NAME=_dci_b200",
           "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           "-I" + sysconfig.get_paths()["include"]] + ["-I" + p for p in inc] + \
          [src, "-o", SHIM, "-L" + HERE, "-ldci_b200", "-L" + torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch",
           "-ltorch_python", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + torch_lib]
    subprocess.run(cmd, check=True)
    return SHIM


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
    print(build_torch_shim(force=True))

"""Build the reference project's own CUDA sources for the GPU box (TEST INFRASTRUCTURE ONLY).

The reference (src/dci_cuda_kernel.cu, src/util_kernel.cu, include/dci.h) is
compiled where it lies, unmodified, together with oracle/ref_harness.cu, into
oracle/_ref/libdci_ref.so.  A second library, libdci_ref_racefixed.so, is built
from a temporary patched copy in which the per-thread top-k scratch offset
`blockIdx.x * k + threadIdx.x * k` (dci_cuda_kernel.cu:514-549, six uses) is
replaced by `(blockIdx.x * blockDim.x + threadIdx.x) * k`, which removes the
overlap between blocks and makes the reference's output deterministic.  The
patched copy lives in a temporary directory and is deleted after the build;
reference sources are never copied into this repository.

The outputs travel to the GPU box with the working tree (they are git-ignored).
Nothing here runs at test time on the GPU box, where the reference checkout
does not exist.
"""
import os
import re
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
REF_SO = os.path.join(OUT, "libdci_ref.so")
REF_FIXED_SO = os.path.join(OUT, "libdci_ref_racefixed.so")

_RACE = re.compile(r"blockIdx\.x\s*\*\s*num_neighbours\s*\+\s*threadIdx\.x\s*\*\s*num_neighbours")


def _nvcc(kernel_src, util_src, include_dir, out):
    cmd = ["nvcc", "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
           "-shared", "-Xcompiler", "-fPIC", "-w", "-I", include_dir,
           kernel_src, util_src, os.path.join(HERE, "ref_harness.cu"),
           "-lcublas", "-o", out]
    subprocess.run(cmd, check=True)


def build_reference(ref_root=None, force=False):
    """Returns the list of libraries built, or [] when the reference checkout is absent.
    ref_root defaults to $DCI_REFERENCE_ROOT, else a checkout named `reference` next to this
    repository."""
    sibling = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    ref_root = ref_root or os.environ.get("DCI_REFERENCE_ROOT", sibling)
    ksrc = os.path.join(ref_root, "src", "dci_cuda_kernel.cu")
    usrc = os.path.join(ref_root, "src", "util_kernel.cu")
    inc = os.path.join(ref_root, "include")
    if not (os.path.exists(ksrc) and os.path.exists(usrc)):
        return []
    os.makedirs(OUT, exist_ok=True)
    harness = os.path.join(HERE, "ref_harness.cu")
    fresh = all(os.path.exists(p) and os.path.getmtime(p) > os.path.getmtime(harness)
                for p in (REF_SO, REF_FIXED_SO))
    if fresh and not force:
        return [REF_SO, REF_FIXED_SO]
    _nvcc(ksrc, usrc, inc, REF_SO)
    tmp = tempfile.mkdtemp(prefix="dci_ref_racefixed_")
    try:
        text = open(ksrc).read()
        patched, count = _RACE.subn("(blockIdx.x * blockDim.x + threadIdx.x) * num_neighbours", text)
        if count != 6:
            raise RuntimeError("expected 6 scratch-offset expressions to patch, found %d" % count)
        pk = os.path.join(tmp, "dci_cuda_kernel.cu")
        with open(pk, "w") as f:
            f.write(patched)
        _nvcc(pk, usrc, inc, REF_FIXED_SO)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    return [REF_SO, REF_FIXED_SO]


if __name__ == "__main__":
    print(build_reference(force="--force" in sys.argv))

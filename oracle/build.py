"""Build recipe for the test oracle (TEST INFRASTRUCTURE ONLY).

`build_oracle()` compiles oracle/dci_oracle.c with gcc into
oracle/libdci_oracle.so.  `build_reference()` (see oracle/build_ref.py)
compiles the reference's own CUDA sources; it needs the reference checkout
and is skipped when that is absent.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libdci_oracle.so")


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_oracle(force=False):
    src = os.path.join(HERE, "dci_oracle.c")
    if not force and not _stale(ORACLE_SO, [src]):
        return ORACLE_SO
    cmd = ["gcc", "-O2", "-std=c11", "-fopenmp", "-ffp-contract=off", "-fno-fast-math",
           "-mfma", "-shared", "-fPIC", "-Wall", "-Wextra", src, "-lm", "-o", ORACLE_SO]
    subprocess.run(cmd, check=True)
    return ORACLE_SO


if __name__ == "__main__":
    print(build_oracle(force=True))

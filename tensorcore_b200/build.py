"""Builds libtensorcore.so and the decode harness for sm_100a with nvcc (in-tree, under
tensorcore_b200/lib/).  Usage: ``python -m tensorcore_b200.build``."""
from __future__ import annotations

import os
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIB_DIR = os.path.join(_HERE, "lib")


def build(verbose: bool = False, jobs: int | None = None) -> str:
    """Runs make in csrc/; returns the path of libtensorcore.so.  Raises on failure."""
    jobs = jobs or max(1, (os.cpu_count() or 2))
    proc = subprocess.run(["make", "-C", CSRC, f"-j{jobs}", "all"], stdout=subprocess.PIPE,
                          stderr=subprocess.STDOUT, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout)
    if proc.returncode != 0:
        raise RuntimeError("building libtensorcore.so failed")
    out = os.path.join(LIB_DIR, "libtensorcore.so")
    if not os.path.exists(out):
        raise RuntimeError(f"{out} missing after build")
    return out


if __name__ == "__main__":
    print(build(verbose=True))

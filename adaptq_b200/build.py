"""Compile the CUDA library in-tree: adaptq_b200/libadaptq_b200.so (sm_100a only)."""
from __future__ import annotations

import os
import shutil
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(_HERE, "csrc", "adaptq_b200.cu")
LIB = os.path.join(_HERE, "libadaptq_b200.so")
# the same sources with -DADAPTQ_CHECKED: device-side index checks that record a status
# instead of trapping, guard bytes behind every device buffer (see csrc/common.cuh)
LIB_CHECKED = os.path.join(_HERE, "libadaptq_b200_checked.so")


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; the AdapTQ B200 library cannot be built")


def sources():
    d = os.path.join(_HERE, "csrc")
    inc = os.path.join(os.path.dirname(_HERE), "include")
    return [os.path.join(d, f) for f in sorted(os.listdir(d))] + \
           [os.path.join(inc, f) for f in sorted(os.listdir(inc))]


def is_stale(lib: str = LIB) -> bool:
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    return any(os.path.getmtime(s) > t for s in sources())


def build_library(force: bool = False, verbose: bool = False, checked: bool = False) -> str:
    """nvcc -gencode arch=compute_100a,code=sm_100a ... -> libadaptq_b200.so
    (checked=True: libadaptq_b200_checked.so, compiled with -DADAPTQ_CHECKED)"""
    lib = LIB_CHECKED if checked else LIB
    if not force and not is_stale(lib):
        return lib
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-Xcompiler", "-fPIC", "-shared", "-diag-suppress", "1886", "-o", lib, SRC]
    if checked:
        cmd.insert(1, "-DADAPTQ_CHECKED=1")
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    subprocess.check_call(cmd)
    return lib


if __name__ == "__main__":
    import sys
    print(build_library(force=True, verbose=True, checked="--checked" in sys.argv))

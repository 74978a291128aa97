"""Builds libcvcuda_b200.so in-tree with nvcc, for sm_100a only.

Usage: ``python cv-cuda_b200/build.py [--force] [--verbose]``
"""
from __future__ import annotations

import argparse
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libcvcuda_b200.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
SOURCES = ["library.cu", "cvcuda_ops.cpp", "random_crop.cpp"]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = glob.glob(os.path.join(CSRC, "*")) + glob.glob(os.path.join(ROOT, "include", "cvcuda_b200", "*"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not (force or _stale()):
        return LIB
    srcs = [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    cmd = [
        NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        # the goldens are defined by un-fused float arithmetic: never contract a*b+c into an FMA
        "--fmad=false", "--ftz=false", "--prec-div=true", "--prec-sqrt=true",
        "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "-shared",
        "-I" + os.path.join(ROOT, "include"), "-I" + CSRC,
        "-Xlinker", "--version-script=" + os.path.join(CSRC, "exports.map"),
        "-o", LIB, *srcs, "-ldl",
    ]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print registers / spills / shared memory per kernel")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
    sys.exit(0)

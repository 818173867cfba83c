"""Compile the CUDA sources into `deconver_b200/libndc_b200.so` for sm_100a with nvcc.

The library is built in-tree (next to this file) so that it travels with the source tree.
nvcc cross-compiles without a GPU.  Run as `python -m deconver_b200._build [--force]`.
"""

import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
INCLUDE = os.path.join(ROOT, "include")
LIB = os.path.join(PKG, "libndc_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def sources():
    deps = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC))
            if f.endswith((".cu", ".cuh"))]
    deps.append(os.path.join(INCLUDE, "ndc_b200.h"))
    return deps


def is_stale():
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    return any(os.path.getmtime(s) > built for s in sources())


def build_library(force=False, verbose=False, extra_flags=()):
    """Build the shared library if it is missing or older than a source file."""
    if not (force or is_stale()):
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc, *NVCC_FLAGS, *extra_flags, "-I", INCLUDE, "-I", CSRC, "-o", LIB,
           os.path.join(CSRC, "ndc_abi.cu")]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd, cwd=ROOT)
    return LIB


if __name__ == "__main__":
    flags = ["-Xptxas", "-v"] if "--ptxas" in sys.argv else []
    print(build_library(force="--force" in sys.argv, verbose=True, extra_flags=flags))

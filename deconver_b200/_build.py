"""Compile the CUDA sources into `deconver_b200/libndc_b200.so` for sm_100a with nvcc.

The library is built in-tree (next to this file) so that it travels with the source tree.
nvcc cross-compiles without a GPU.  The tiled kernels are compiled as six translation units
(forward / backward of volumes / backward of images, each for float32 and bfloat16) next to the
ABI unit and the instance-norm and bias units, in parallel, then linked.  Run as `python -m deconver_b200._build [--force]`.
"""

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
INCLUDE = os.path.join(ROOT, "include")
LIB = os.path.join(PKG, "libndc_b200.so")
OBJ = os.path.join(PKG, "_obj")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xfatbin=-compress-all",
]

# (object name, source, extra defines)
UNITS = [("abi", "ndc_abi.cu", []), ("inorm", "ndc_inorm.cu", []), ("bias", "ndc_bias.cu", [])] + [
    ("dw4_p%d_t%d" % (part, t), "ndc_dw4_inst.cu", ["-DNDC_DW4_PART=%d" % part, "-DNDC_DW4_T=%d" % t])
    for part in (1, 2, 0) for t in (0, 1)   # the longest units first
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
    os.makedirs(OBJ, exist_ok=True)

    def compile_unit(unit):
        name, src, defines = unit
        obj = os.path.join(OBJ, name + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra_flags, *defines, "-I", INCLUDE, "-I", CSRC, "-c",
               os.path.join(CSRC, src), "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        return obj, res

    with ThreadPoolExecutor(max_workers=min(len(UNITS), os.cpu_count() or 1)) as pool:
        results = list(pool.map(compile_unit, UNITS))
    for _, res in results:
        if res.stdout and (verbose or res.returncode):
            print(res.stdout, end="", flush=True)
    failed = [res for _, res in results if res.returncode]
    if failed:
        raise subprocess.CalledProcessError(failed[0].returncode, failed[0].args)
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + [o for o, _ in results]
    if verbose:
        print(" ".join(link), flush=True)
    subprocess.check_call(link, cwd=ROOT)
    return LIB


if __name__ == "__main__":
    flags = ["-Xptxas", "-v"] if "--ptxas" in sys.argv else []
    print(build_library(force="--force" in sys.argv, verbose=True, extra_flags=flags))

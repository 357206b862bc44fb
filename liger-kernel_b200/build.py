"""Build libflce_b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python liger-kernel_b200/build.py [--force] [--verbose]

nvcc cross-compiles, so no GPU is needed to build.
"""

import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "liger_kernel_b200", "libflce_b200.so")
SOURCES = [os.path.join(CSRC, "flce_b200.cu")]


def _deps():
    deps = [os.path.join(ROOT, "include", "flce_b200.h")]
    for name in sorted(os.listdir(CSRC)):
        deps.append(os.path.join(CSRC, name))
    return deps


def needs_build():
    if not os.path.exists(OUT):
        return True
    built = os.path.getmtime(OUT)
    return any(os.path.getmtime(d) > built for d in _deps())


TRACE_OUT = os.path.join(HERE, "liger_kernel_b200", "libflce_b200_trace.so")


def build(force=False, verbose=False, trace=False):
    """trace=True builds a second library with -DFLCE_CLOCK_TRACE: the three warp roles of the main loop count the cycles
    they spend waiting on each barrier (read back with flce_b200_debug_clock_trace; used by bench_gemm.py --trace)."""
    out = TRACE_OUT if trace else OUT
    if not trace and not force and not needs_build():
        return OUT
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [
        nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
        "-shared", "-Xcompiler", "-fPIC", "-I", os.path.join(ROOT, "include"), "-I", CSRC,
        "-o", out,
    ] + (["-DFLCE_CLOCK_TRACE"] if trace else []) + SOURCES
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    subprocess.run(cmd, check=True)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--trace", action="store_true", help="also build libflce_b200_trace.so (cycle accounting in the main loop)")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
    if a.trace:
        print(build(force=True, verbose=a.verbose, trace=True))
    sys.exit(0)

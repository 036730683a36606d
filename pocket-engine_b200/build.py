"""Builds libplora.so (the C-ABI library: host registry + sm_100a kernels) in-tree with nvcc.

Usage: python pocket-engine_b200/build.py [--force] [--verbose]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libplora.so")
LIB_BOUNDS = os.path.join(HERE, "libplora_bounds.so")  # the range-checked build (-DPLORA_BOUNDS), used by tests
SOURCES = ["plora_host.cpp", "plora_read.cpp", "plora_manager.cpp", "plora_kernels.cu", "plora_mma.cu", "plora_fp8.cu", "plora_site.cu", "plora_static.cu", "plora_xchg.cu", "plora_gemm.cu"]
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-Wall,-Wextra", "-shared", "-cudart", "static",
]


def stale(lib=LIB):
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f != "plora_compat.cu"] + \
        [os.path.join(HERE, "..", "include", "plora.h")]
    return any(os.path.getmtime(d) > t for d in deps)


COMPAT = os.path.join(HERE, "plora_compat.fatbin")


def build_compat(force=False):
    """The drop-in kernel image under the reference's own kernel names (for POCKET_KERNELS=<fatbin>)."""
    src = os.path.join(CSRC, "plora_compat.cu")
    if not force and os.path.exists(COMPAT) and os.path.getmtime(COMPAT) >= os.path.getmtime(src):
        return COMPAT
    r = subprocess.run(["nvcc", "--fatbin", "-std=c++17", "-O3", "-lineinfo", "-gencode",
                        "arch=compute_100a,code=sm_100a", src, "-o", COMPAT], capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("nvcc failed building plora_compat.fatbin")
    return COMPAT


def _nvcc(lib, extra, verbose):
    cmd = ["nvcc"] + FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + \
        [os.path.join(CSRC, s) for s in SOURCES] + ["-o", lib]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed building " + os.path.basename(lib))


def build(force=False, verbose=False, bounds=True):
    build_compat(force)
    if force or stale(LIB):
        _nvcc(LIB, [], verbose)
    if bounds and (force or stale(LIB_BOUNDS)):
        _nvcc(LIB_BOUNDS, ["-DPLORA_BOUNDS"], False)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(LIB)

"""Builds librocal_b200.so (CUDA kernels + C-ABI + host pipeline) in-tree for sm_100a.

    python -m rocal_b200.build [--force] [--verbose] [--debug-bounds]

--debug-bounds builds librocal_b200_bounds.so instead: the same sources with RB200_DEBUG_BOUNDS defined, in which the
kernels check every sample's source rectangle and every staging copy against the arena size the caller states and
report through the status word (include/rb200_kernels.h, "Sizes and the bounds-checking build"). Load it by setting
RB200_LIBRARY to its path.

nvcc cross-compiles without a GPU. The library links the CUDA runtime statically, so it loads
in any process whether or not another CUDA runtime (e.g. torch's) is already present.
"""
import glob
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "librocal_b200.so")
OBJ_DIR = os.path.join(PKG, "build")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall",
          "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(CSRC, "kernels"),
          "-I" + os.path.join(CSRC, "host")]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cu")) + glob.glob(os.path.join(CSRC, "host", "*.cpp")))


def headers():
    return (glob.glob(os.path.join(CSRC, "kernels", "*.cuh")) + glob.glob(os.path.join(CSRC, "host", "*.h")) +
            glob.glob(os.path.join(ROOT, "include", "*.h")))


LIB_BOUNDS = os.path.join(PKG, "librocal_b200_bounds.so")


def build(force=False, verbose=False, debug_bounds=False):
    lib = LIB_BOUNDS if debug_bounds else LIB
    obj_dir = OBJ_DIR + ("_bounds" if debug_bounds else "")
    defines = ["-DRB200_DEBUG_BOUNDS"] if debug_bounds else []
    os.makedirs(obj_dir, exist_ok=True)
    hdr_time = max([os.path.getmtime(h) for h in headers()] + [os.path.getmtime(__file__)])
    objs, procs = [], []
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src) + ".o")
        objs.append(obj)
        if (not force and os.path.exists(obj) and os.path.getmtime(obj) > os.path.getmtime(src)
                and os.path.getmtime(obj) > hdr_time):
            continue
        cmd = [NVCC] + ARCH + COMMON + defines + (["-Xptxas", "-v"] if verbose else []) + ["-x", "cu", "-c", src, "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(out)
        if p.returncode != 0:
            failed = True
            sys.stderr.write("nvcc failed for %s\n" % src)
    if failed:
        raise RuntimeError("rocal_b200: nvcc build failed")
    if procs or force or not os.path.exists(lib):
        cmd = [NVCC] + ARCH + ["-shared", "-o", lib] + objs + ["-Xlinker", "--exclude-libs,ALL", "-lpthread"]
        subprocess.run(cmd, check=True)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, debug_bounds="--debug-bounds" in sys.argv))

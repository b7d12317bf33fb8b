"""Build recipe of the CPU oracle. TEST INFRASTRUCTURE ONLY — the product never imports this.

    python oracle/build.py            # liboracle.so (+ _ref/libref.so when the reference tree is present)

liboracle.so   the CPU restatement in oracle.c (gcc, -ffp-contract=off so that every written
               operation rounds once; -mavx2 -mfma -mf16c are the reference's own CPU flags,
               rocAL/CMakeLists.txt:375).
_ref/libref.so reference-owned CPU code compiled where it lies (never copied):
               rocAL/source/meta_data/bounding_box_graph.cpp, rocAL/source/parameters/
               parameter_{factory,random_crop_decoder,crop,random_crop}.cpp + ref_driver.cpp, against
               the stand-in headers in ref_stubs/. Only built when REFERENCE_ROOT exists.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REFERENCE_ROOT = os.environ.get("ROCAL_REFERENCE_ROOT", "/root/reference")

ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libref.so")

CFLAGS = ["-O3", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off", "-fno-fast-math",
          "-mavx2", "-mfma", "-mf16c", "-fvisibility=hidden", "-Wall", "-Wno-unused-function"]


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources if os.path.exists(s))


def build_oracle(force=False):
    srcs = [os.path.join(HERE, "oracle.c"), os.path.join(HERE, "..", "include", "rb200_kernels.h")]
    if force or _stale(ORACLE_SO, srcs):
        cmd = ["gcc", "-std=gnu11"] + CFLAGS + [srcs[0], "-o", ORACLE_SO, "-lm"]
        subprocess.run(cmd, check=True)
    return ORACLE_SO


def reference_available():
    return os.path.isfile(os.path.join(REFERENCE_ROOT, "rocAL", "source", "meta_data", "bounding_box_graph.cpp"))


def build_ref(force=False):
    """Returns the path of _ref/libref.so, or None when the reference tree is absent and no
    prebuilt library exists."""
    if not reference_available():
        return REF_SO if os.path.exists(REF_SO) else None
    r = os.path.join(REFERENCE_ROOT, "rocAL")
    srcs = [os.path.join(r, "source", "meta_data", "bounding_box_graph.cpp"),
            os.path.join(r, "source", "parameters", "parameter_factory.cpp"),
            os.path.join(r, "source", "parameters", "parameter_random_crop_decoder.cpp"),
            os.path.join(r, "source", "parameters", "parameter_crop.cpp"),
            os.path.join(r, "source", "parameters", "parameter_random_crop.cpp"),
            os.path.join(HERE, "ref_driver.cpp")]
    if force or _stale(REF_SO, srcs):
        os.makedirs(REF_DIR, exist_ok=True)
        cmd = ["g++", "-std=c++17", "-O3", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off",
               "-mavx2", "-mfma", "-mf16c", "-w",
               "-DENABLE_HIP=0", "-DENABLE_OPENCL=0", "-DENABLE_SIMD=0", "-DDBGLOG=0", "-DWRNLOG=0",
               "-DDBGINFO=0", "-DDBG_TIMING=1",
               "-I" + os.path.join(HERE, "ref_stubs"), "-I" + os.path.join(r, "include"),
               "-I" + os.path.join(r, "include", "api")] + srcs + ["-o", REF_SO]
        subprocess.run(cmd, check=True)
    return REF_SO


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))

"""Build recipe of the CPU oracle. TEST INFRASTRUCTURE ONLY — the product never imports this.

    python oracle/build.py            # liboracle.so (+ _ref/libref.so when the reference tree is present)

liboracle.so   the CPU restatement in oracle.c (gcc, -ffp-contract=off so that every written
               operation rounds once; -mavx2 -mfma -mf16c are the reference's own CPU flags,
               rocAL/CMakeLists.txt:375).
_ref/libref.so reference-owned CPU code compiled where it lies (never copied):
               rocAL/source/meta_data/bounding_box_graph.cpp, rocAL/source/parameters/
               parameter_{factory,random_crop_decoder,crop,rocal_crop,random_crop}.cpp,
               rocAL/source/meta_data/randombboxcrop_reader.cpp + ref_driver.cpp + ref_bbox_crop_driver.cpp,
               against the stand-in headers in ref_stubs/. Only built when the reference tree exists.
_ref/libref_hip.so the reference's own pixel kernels, rocAL/rocAL_hip/rocal_hip_kernels.cpp, compiled for the
               host where they lie against ref_stubs/hip/ (vector types, thread indices set by a launch
               loop) + ref_hip_driver.cpp. Built with -ffp-contract=fast --param=avoid-fma-max-bits=0:
               the HIP compiler contracts a*b+c inside an expression by default, and that parameter makes
               gcc fuse every such candidate (its x86 tuning otherwise skips the ones on a loop-carried
               sum), so the host build rounds where the device build does.

The reference tree is found through the --reference argument, the environment variable
ROCAL_REFERENCE_ROOT, or as a directory named `reference` beside this repository's checkout; without any
of them only prebuilt _ref libraries are used.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REFERENCE_ROOT = os.environ.get("ROCAL_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")

ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libref.so")
REF_HIP_SO = os.path.join(REF_DIR, "libref_hip.so")

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


def set_reference_root(path):
    global REFERENCE_ROOT
    REFERENCE_ROOT = path or ""


def reference_available():
    return bool(REFERENCE_ROOT) and os.path.isfile(os.path.join(REFERENCE_ROOT, "rocAL", "source", "meta_data", "bounding_box_graph.cpp"))


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
            os.path.join(r, "source", "parameters", "parameter_rocal_crop.cpp"),
            os.path.join(r, "source", "parameters", "parameter_random_crop.cpp"),
            os.path.join(r, "source", "meta_data", "randombboxcrop_reader.cpp"),
            os.path.join(HERE, "ref_driver.cpp"), os.path.join(HERE, "ref_bbox_crop_driver.cpp")]
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


def build_ref_hip(force=False):
    """Returns the path of _ref/libref_hip.so, or None when the reference tree is absent and no
    prebuilt library exists."""
    if not reference_available():
        return REF_HIP_SO if os.path.exists(REF_HIP_SO) else None
    hip = os.path.join(REFERENCE_ROOT, "rocAL", "rocAL_hip")
    srcs = [os.path.join(hip, "rocal_hip_kernels.cpp"), os.path.join(HERE, "ref_hip_driver.cpp")]
    deps = srcs + [os.path.join(HERE, "ref_stubs", "hip", h) for h in ("hip_runtime.h", "hip_runtime_api.h", "hip_fp16.h")]
    if force or _stale(REF_HIP_SO, deps):
        os.makedirs(REF_DIR, exist_ok=True)
        cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-ffp-contract=fast", "--param=avoid-fma-max-bits=0",
               "-mavx2", "-mfma", "-mf16c", "-w", "-I" + os.path.join(HERE, "ref_stubs"), "-I" + hip] + srcs + ["-o", REF_HIP_SO]
        subprocess.run(cmd, check=True)
    return REF_HIP_SO


if __name__ == "__main__":
    if "--reference" in sys.argv:
        set_reference_root(sys.argv[sys.argv.index("--reference") + 1])
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))
    print(build_ref_hip(force="--force" in sys.argv))

"""The host side of the library under the sanitizers, on a machine without a GPU. The whole host layer (graph planning,
loader thread, ring of output slots, feeding from a second thread, boxes, random bbox crop, error and shutdown paths) is
compiled with g++ against a stand-in for the CUDA runtime and for the kernel entry points
(tests/harness/fake_cuda_runtime.cpp: "device" memory is heap memory, streams run in line) and driven through the
rocAL-signature API by tests/harness/pipeline_host_harness.cpp - once with -fsanitize=address,undefined (every table and
buffer the host code sizes is watched, leaks included) and once with -fsanitize=thread (the producer / loader /
consumer hand-offs)."""
import glob
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "rocal_b200", "csrc", "host")
CUDA_INCLUDE = os.environ.get("CUDA_INCLUDE", "/usr/local/cuda/include")


def _build(tmp, name, sanitize):
    exe = str(tmp / name)
    src = [os.path.join(ROOT, "tests", "harness", "pipeline_host_harness.cpp"),
           os.path.join(ROOT, "tests", "harness", "fake_cuda_runtime.cpp")] + sorted(glob.glob(os.path.join(HOST, "*.cpp")))
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=" + sanitize, "-I", CUDA_INCLUDE,
           "-I", os.path.join(ROOT, "include"), "-I", HOST, "-I", os.path.join(ROOT, "rocal_b200", "csrc", "kernels")] + src + \
          ["-o", exe, "-lpthread", "-ldl"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return exe


@pytest.fixture(scope="module")
def harnesses(tmp_path_factory):
    if not os.path.exists(os.path.join(CUDA_INCLUDE, "cuda_runtime.h")):
        pytest.skip("the CUDA runtime header is needed to compile the host layer")
    d = tmp_path_factory.mktemp("san")
    # the two builds take most of a minute each: run them side by side
    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(2) as ex:
        a = ex.submit(_build, d, "asan", "address,undefined")
        t = ex.submit(_build, d, "tsan", "thread")
        return a.result(), t.result()


def test_host_layer_under_address_and_undefined_behaviour_sanitizers(harnesses):
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1")
    r = subprocess.run([harnesses[0], "60"], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0 and "ok 60" in r.stdout, r.stderr[-4000:]
    assert "Sanitizer" not in r.stderr and "runtime error" not in r.stderr, r.stderr[-4000:]


def test_host_layer_under_thread_sanitizer(harnesses):
    r = subprocess.run([harnesses[1], "60"], capture_output=True, text=True, timeout=600)
    if "unexpected memory mapping" in r.stderr:
        pytest.skip("the thread sanitizer cannot map its shadow memory on this kernel")
    assert r.returncode == 0 and "ok 60" in r.stdout, r.stderr[-4000:]
    assert "ThreadSanitizer" not in r.stderr, r.stderr[-4000:]

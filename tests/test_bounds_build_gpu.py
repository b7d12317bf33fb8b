"""The bounds-checking build of the library (`python -m rocal_b200.build --debug-bounds`): its kernels check every
sample's source rectangle and every staging copy against the arena size the caller states, report through the status
word and skip what would leave the arena. Each test runs a child process that loads that build through RB200_LIBRARY,
because a process binds one build of the library."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BOUNDS_LIB = os.path.join(ROOT, "rocal_b200", "librocal_b200_bounds.so")


def _run(args, timeout):
    assert os.path.exists(BOUNDS_LIB), "build it first: python -m rocal_b200.build --debug-bounds"
    env = dict(os.environ, RB200_LIBRARY=BOUNDS_LIB, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable] + args, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, (r.stdout[-3000:], r.stderr[-3000:])
    return r.stdout


@pytest.mark.gpu
def test_out_of_bounds_samples_are_reported_and_skipped():
    out = _run([os.path.join(ROOT, "tests", "harness", "bounds_build_check.py")], 600)
    assert "bounds build check passed" in out
    for name in ("resample stream rows", "resample stream pairs", "resample tile", "resample direct", "resample triangular", "pointwise vector", "pointwise scalar",
                 "warp affine", "output size refused"):
        assert "ok " + name in out, out


@pytest.mark.gpu
def test_differential_and_pipeline_suites_under_the_bounds_build():
    """The randomised differential test and the operator tests through the pipeline run clean under the checking
    build: same results, and the library-wide status word is still 0 at the end."""
    code = ("import sys, pytest\n"
            "rc = pytest.main(['-q', '-x', '-m', 'gpu', '-p', 'no:cacheprovider', 'tests/test_differential_gpu.py', "
            "'tests/test_api_ops_gpu.py', 'tests/test_normalize_gpu.py'])\n"
            "from rocal_b200._lib import lib, version\n"
            "assert version().endswith('+bounds'), version()\n"
            "st = lib.rb200k_device_status()\n"
            "print('status word', st)\n"
            "sys.exit(int(rc) or st)\n")
    out = _run(["-c", code], 1500)
    assert "status word 0" in out, out[-2000:]


def test_bounds_build_exports_the_same_abi():
    """CPU: when the checking build is present it exports every entry point the release build does."""
    import ctypes
    if not os.path.exists(BOUNDS_LIB):
        pytest.skip("the bounds-checking build has not been made")
    rel = os.path.join(ROOT, "rocal_b200", "librocal_b200.so")
    names = subprocess.run(["nm", "-D", "--defined-only", rel], capture_output=True, text=True, check=True).stdout.split("\n")
    names = [l.split()[-1] for l in names if " T " in l and (" rb200" in l or " rocal" in l)]
    assert len(names) > 100
    dbg = ctypes.CDLL(BOUNDS_LIB)
    for nm in names:
        assert hasattr(dbg, nm), nm
    dbg.rb200k_version.restype = ctypes.c_char_p
    assert dbg.rb200k_version().decode().endswith("+bounds")

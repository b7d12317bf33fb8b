"""amd.rocal.random for the supported subset (rocAL_pybind/amd/rocal/random.py)."""
import ctypes

from . import _capi as C


def coin_flip(*inputs, probability=0.5, device=None):
    """Per-sample 0/1 with P(1) = probability: rocalCreateIntRand({0,1}, {1-p, p})."""
    values = (ctypes.c_int * 2)(0, 1)
    freqs = (ctypes.c_double * 2)(1 - probability, probability)
    return C.Param(C.create_int_rand(values, freqs, 2), True)


def uniform(*inputs, range=(-1.0, 1.0), device=None):
    """Per-sample float, uniform in range: rocalCreateFloatUniformRand."""
    return C.Param(C.create_float_uniform_rand(float(range[0]), float(range[1])), False)

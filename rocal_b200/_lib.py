"""ctypes binding of librocal_b200.so — the C-ABI declared in include/rb200_kernels.h and
include/rb200.h. There is no fallback: if the library is missing, importing this module fails."""
import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# RB200_LIBRARY names another build of the same library (the bounds-checking one, a sanitizer build)
LIB_PATH = os.environ.get("RB200_LIBRARY") or os.path.join(_PKG, "librocal_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        "rocal_b200: %s not found. Build it with `python -m rocal_b200.build` (needs nvcc); "
        "there is no CPU fallback." % LIB_PATH)

lib = ctypes.CDLL(LIB_PATH)

c_void_p, c_int, c_char_p, c_uint64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_uint64


class ResampleParams(ctypes.Structure):
    _fields_ = [("out", c_void_p), ("out_w", ctypes.c_int32), ("out_h", ctypes.c_int32),
                ("out_dtype", ctypes.c_int32), ("out_layout", ctypes.c_int32),
                ("normalize", ctypes.c_int32), ("fill_padding", ctypes.c_int32),
                ("mul", ctypes.c_float * 3), ("add", ctypes.c_float * 3), ("interpolation", ctypes.c_int32), ("path", ctypes.c_int32),
                ("overlap", ctypes.c_int32), ("strip_rows", ctypes.c_int32), ("status", ctypes.c_void_p),
                ("arena_bytes", ctypes.c_uint64), ("out_bytes", ctypes.c_uint64)]


class PointwiseParams(ctypes.Structure):
    _fields_ = [("out", c_void_p), ("out_w", ctypes.c_int32), ("out_h", ctypes.c_int32),
                ("out_dtype", ctypes.c_int32), ("out_layout", ctypes.c_int32),
                ("color_op", ctypes.c_int32), ("normalize", ctypes.c_int32),
                ("fill_padding", ctypes.c_int32), ("reverse_channels", ctypes.c_int32),
                ("mul", ctypes.c_float * 3), ("add", ctypes.c_float * 3), ("arith", ctypes.c_int32),
                ("overlap", ctypes.c_int32), ("status", ctypes.c_void_p),
                ("arena_bytes", ctypes.c_uint64), ("out_bytes", ctypes.c_uint64)]


class WarpParams(ctypes.Structure):
    _fields_ = [("out", c_void_p), ("out_w", ctypes.c_int32), ("out_h", ctypes.c_int32),
                ("fill_padding", ctypes.c_int32), ("overlap", ctypes.c_int32), ("status", ctypes.c_void_p),
                ("arena_bytes", ctypes.c_uint64), ("out_bytes", ctypes.c_uint64)]


class BoxEncoderParams(ctypes.Structure):
    _fields_ = [("anchors", c_void_p), ("num_anchors", ctypes.c_int32), ("criteria", ctypes.c_float),
                ("means", ctypes.c_float * 4), ("inv_stds", ctypes.c_float * 4),
                ("offset", ctypes.c_int32), ("scale", ctypes.c_float)]


class BoxMatcherParams(ctypes.Structure):
    _fields_ = [("anchors", c_void_p), ("num_anchors", ctypes.c_int32), ("high_threshold", ctypes.c_float),
                ("low_threshold", ctypes.c_float), ("allow_low_quality_matches", ctypes.c_int32)]


class BoxWindow(ctypes.Structure):
    _fields_ = [("l", ctypes.c_float), ("t", ctypes.c_float), ("r", ctypes.c_float), ("b", ctypes.c_float),
                ("mirror_h", ctypes.c_int32), ("mirror_v", ctypes.c_int32), ("reserved", ctypes.c_int32 * 2)]


class NormalizeParams(ctypes.Structure):
    _fields_ = [("out", c_void_p), ("out_w", ctypes.c_int32), ("out_h", ctypes.c_int32), ("out_dtype", ctypes.c_int32),
                ("axis_mask", ctypes.c_int32), ("compute_mean", ctypes.c_int32), ("compute_stddev", ctypes.c_int32),
                ("fill_padding", ctypes.c_int32), ("mean", ctypes.c_float * 3), ("stddev", ctypes.c_float * 3),
                ("scale", ctypes.c_float), ("shift", ctypes.c_float),
                ("arena_bytes", ctypes.c_uint64), ("out_bytes", ctypes.c_uint64)]


lib.rb200k_normalize_scratch_bytes.argtypes = [c_int, c_int, c_int, c_int]
lib.rb200k_normalize_scratch_bytes.restype = ctypes.c_size_t
lib.rb200k_normalize.argtypes = [c_void_p, c_void_p, c_void_p, c_int, ctypes.POINTER(NormalizeParams), c_void_p, ctypes.c_size_t, c_void_p]
lib.rb200k_normalize.restype = c_int
lib.rb200k_transpose.argtypes = [c_void_p, c_void_p, c_int, ctypes.POINTER(ctypes.c_int32), c_void_p, ctypes.POINTER(ctypes.c_int32), c_void_p]
lib.rb200k_transpose.restype = c_int
lib.rb200k_resample.argtypes = [c_void_p, c_void_p, c_void_p, c_int, ctypes.POINTER(ResampleParams), c_void_p]
lib.rb200k_resample.restype = c_int
lib.rb200k_pointwise.argtypes = [c_void_p, c_void_p, c_void_p, c_int, ctypes.POINTER(PointwiseParams), c_void_p]
lib.rb200k_pointwise.restype = c_int
lib.rb200k_resample_probe.argtypes = [c_void_p, c_void_p, c_void_p, c_int, ctypes.POINTER(ResampleParams), c_void_p, c_uint64, c_int]
lib.rb200k_resample_probe.restype = c_int
lib.rb200k_pointwise_probe.argtypes = [c_void_p, c_void_p, c_void_p, c_int, ctypes.POINTER(PointwiseParams), c_void_p, c_uint64, c_int]
lib.rb200k_pointwise_probe.restype = c_int
lib.rb200k_device_status.restype = c_int
lib.rb200k_warp_affine.argtypes = [c_void_p, c_void_p, c_int, ctypes.POINTER(WarpParams), c_void_p]
lib.rb200k_warp_affine.restype = c_int
lib.rb200k_box_encode.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, ctypes.POINTER(BoxEncoderParams),
                                  c_void_p, c_void_p, c_void_p]
lib.rb200k_box_encode.restype = c_int
lib.rb200k_box_iou_match.argtypes = [c_void_p, c_void_p, c_int, c_int, ctypes.POINTER(BoxMatcherParams), c_void_p, c_void_p]
lib.rb200k_box_iou_match.restype = c_int
lib.rb200k_box_transform.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
lib.rb200k_box_transform.restype = c_int
lib.rb200k_last_error.restype = c_char_p
lib.rb200k_launch_count.restype = c_uint64
lib.rb200k_version.restype = c_char_p


class Rb200Error(RuntimeError):
    pass


def check(rc, what):
    if rc != 0:
        raise Rb200Error("%s failed (%d): %s" % (what, rc, lib.rb200k_last_error().decode()))


def launch_count():
    return int(lib.rb200k_launch_count())


def version():
    return lib.rb200k_version().decode()

"""ctypes front of oracle/liboracle.so (the CPU restatement) and oracle/_ref/libref.so
(reference-owned CPU code compiled from the reference tree). TEST INFRASTRUCTURE ONLY.

Takes the same numpy tables as the CUDA path (layouts of include/rb200_kernels.h) and returns
numpy arrays, so a parity test is `np.array_equal(gpu.cpu().numpy(), oracle(...))`.
"""
import ctypes
import math
import os

import numpy as np

from . import build as _build

_HERE = os.path.dirname(os.path.abspath(__file__))

FP32, FP16, UINT8 = 0, 1, 2
NHWC, NCHW = 0, 1
_NP = {FP32: np.float32, FP16: np.float16, UINT8: np.uint8}


class _ResampleParams(ctypes.Structure):
    _fields_ = [("out", ctypes.c_void_p), ("out_w", ctypes.c_int32), ("out_h", ctypes.c_int32),
                ("out_dtype", ctypes.c_int32), ("out_layout", ctypes.c_int32),
                ("normalize", ctypes.c_int32), ("fill_padding", ctypes.c_int32),
                ("mul", ctypes.c_float * 3), ("add", ctypes.c_float * 3), ("interpolation", ctypes.c_int32), ("path", ctypes.c_int32),
                ("overlap", ctypes.c_int32), ("strip_rows", ctypes.c_int32), ("status", ctypes.c_void_p),
                ("arena_bytes", ctypes.c_uint64), ("out_bytes", ctypes.c_uint64)]


class _PointwiseParams(ctypes.Structure):
    _fields_ = [("out", ctypes.c_void_p), ("out_w", ctypes.c_int32), ("out_h", ctypes.c_int32),
                ("out_dtype", ctypes.c_int32), ("out_layout", ctypes.c_int32),
                ("color_op", ctypes.c_int32), ("normalize", ctypes.c_int32),
                ("fill_padding", ctypes.c_int32), ("reverse_channels", ctypes.c_int32),
                ("mul", ctypes.c_float * 3), ("add", ctypes.c_float * 3), ("arith", ctypes.c_int32),
                ("overlap", ctypes.c_int32), ("status", ctypes.c_void_p),
                ("arena_bytes", ctypes.c_uint64), ("out_bytes", ctypes.c_uint64)]


class _WarpParams(ctypes.Structure):
    _fields_ = [("out", ctypes.c_void_p), ("out_w", ctypes.c_int32), ("out_h", ctypes.c_int32),
                ("fill_padding", ctypes.c_int32), ("overlap", ctypes.c_int32), ("status", ctypes.c_void_p),
                ("arena_bytes", ctypes.c_uint64), ("out_bytes", ctypes.c_uint64)]


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(_build.build_oracle())
        _lib.orc_resample.restype = ctypes.c_int
        _lib.orc_pointwise.restype = ctypes.c_int
        _lib.orc_warp_affine.restype = ctypes.c_int
        _lib.orc_box_encode.restype = ctypes.c_int
    return _lib


def ref():
    """The reference-built library, or None when neither the reference tree nor a prebuilt copy exists."""
    global _ref
    if _ref is None:
        path = _build.build_ref()
        if path is None:
            return None
        _ref = ctypes.CDLL(path)
    return _ref


def set_threads(n):
    """OpenMP thread count for subsequent oracle calls (used by the CPU-baseline timing)."""
    os.environ["OMP_NUM_THREADS"] = str(n)
    try:
        omp = ctypes.CDLL("libgomp.so.1")
        omp.omp_set_num_threads(int(n))
    except OSError:
        pass


def _out_array(n, out_w, out_h, dtype, layout, fill):
    shape = (n, 3, out_h, out_w) if layout == NCHW else (n, out_h, out_w, 3)
    return np.zeros(shape, dtype=_NP[dtype]) if fill else np.full(shape, 0, dtype=_NP[dtype])


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def resample(arena, samples, out_w, out_h, out_dtype=FP32, out_layout=NCHW, mul=None, add=None,
             fill_padding=True, out=None, interpolation=0):
    n = len(samples)
    if out is None:
        out = _out_array(n, out_w, out_h, out_dtype, out_layout, True)
    p = _ResampleParams()
    p.out = out.ctypes.data
    p.out_w, p.out_h, p.out_dtype, p.out_layout = out_w, out_h, out_dtype, out_layout
    p.normalize = 1 if mul is not None else 0
    p.fill_padding = 1 if fill_padding else 0
    p.interpolation = int(interpolation)
    for c in range(3):
        p.mul[c] = float(mul[c]) if mul is not None else 1.0
        p.add[c] = float(add[c]) if add is not None else 0.0
    rc = lib().orc_resample(_ptr(arena), _ptr(samples), ctypes.c_int(n), ctypes.byref(p))
    assert rc == 0
    return out


def pointwise(arena, samples, out_w, out_h, color_op=0, out_dtype=UINT8, out_layout=NHWC, mul=None, add=None,
              reverse_channels=False, fill_padding=True, out=None):
    n = len(samples)
    if out is None:
        out = _out_array(n, out_w, out_h, out_dtype, out_layout, True)
    p = _PointwiseParams()
    p.out = out.ctypes.data
    p.out_w, p.out_h, p.out_dtype, p.out_layout = out_w, out_h, out_dtype, out_layout
    p.color_op = color_op
    p.normalize = 1 if mul is not None else 0
    p.fill_padding = 1 if fill_padding else 0
    p.reverse_channels = 1 if reverse_channels else 0
    for c in range(3):
        p.mul[c] = float(mul[c]) if mul is not None else 1.0
        p.add[c] = float(add[c]) if add is not None else 0.0
    rc = lib().orc_pointwise(_ptr(arena), _ptr(samples), ctypes.c_int(n), ctypes.byref(p))
    assert rc == 0
    return out


def warp_affine(arena, samples, out_w, out_h, fill_padding=True, out=None):
    n = len(samples)
    if out is None:
        out = np.zeros((n, out_h, out_w, 3), dtype=np.uint8)
    p = _WarpParams()
    p.out = out.ctypes.data
    p.out_w, p.out_h = out_w, out_h
    p.fill_padding = 1 if fill_padding else 0
    rc = lib().orc_warp_affine(_ptr(arena), _ptr(samples), ctypes.c_int(n), ctypes.byref(p))
    assert rc == 0
    return out


class _NormalizeParams(ctypes.Structure):
    _fields_ = [("out", ctypes.c_void_p), ("out_w", ctypes.c_int32), ("out_h", ctypes.c_int32), ("out_dtype", ctypes.c_int32),
                ("axis_mask", ctypes.c_int32), ("compute_mean", ctypes.c_int32), ("compute_stddev", ctypes.c_int32),
                ("fill_padding", ctypes.c_int32), ("mean", ctypes.c_float * 3), ("stddev", ctypes.c_float * 3),
                ("scale", ctypes.c_float), ("shift", ctypes.c_float)]


def normalize(arena, samples, out_w, out_h, axis_mask=3, mean=None, stddev=None, scale=1.0, shift=0.0, out_dtype=FP32,
              fill_padding=True):
    """orc_normalize: statistics are computed where mean / stddev is None, else per-channel constants. Returns
    [n][out_h][out_w][3] float32 or float16."""
    n = len(samples)
    out = np.zeros((n, out_h, out_w, 3), dtype=_NP[out_dtype])
    p = _NormalizeParams()
    p.out = out.ctypes.data
    p.out_w, p.out_h, p.out_dtype, p.axis_mask = out_w, out_h, out_dtype, axis_mask
    p.compute_mean, p.compute_stddev = int(mean is None), int(stddev is None)
    p.fill_padding = 1 if fill_padding else 0
    for c in range(3):
        p.mean[c] = float(mean[c]) if mean is not None else 0.0
        p.stddev[c] = float(stddev[c]) if stddev is not None else 1.0
    p.scale, p.shift = float(scale), float(shift)
    lib().orc_normalize.restype = ctypes.c_int
    rc = lib().orc_normalize(_ptr(arena), _ptr(samples), ctypes.c_int(n), ctypes.byref(p))
    assert rc == 0
    return out


def transpose(arena, samples, perm, out_dims):
    """orc_transpose: uint8 [n][out_dims...] with every sample's permuted window at the origin of its slot."""
    n = len(samples)
    out = np.zeros((n,) + tuple(int(v) for v in out_dims), dtype=np.uint8)
    pm = np.asarray(perm, dtype=np.int32)
    od = np.asarray(out_dims, dtype=np.int32)
    lib().orc_transpose.restype = ctypes.c_int
    rc = lib().orc_transpose(_ptr(arena), _ptr(samples), ctypes.c_int(n), _ptr(pm), _ptr(out), _ptr(od))
    assert rc == 0
    return out


def _box_call(fn, boxes, labels, offsets, anchors, criteria, means, stds, offset, scale):
    n = len(offsets) - 1
    a = anchors.shape[0]
    boxes = np.ascontiguousarray(boxes, dtype=np.float32)
    labels = np.ascontiguousarray(labels, dtype=np.int32)
    offsets = np.ascontiguousarray(offsets, dtype=np.int32)
    anchors = np.ascontiguousarray(anchors, dtype=np.float32)
    means = np.ascontiguousarray(means, dtype=np.float32)
    stds = np.ascontiguousarray(stds, dtype=np.float32)
    ob = np.zeros((n, a, 4), dtype=np.float32)
    ol = np.zeros((n, a), dtype=np.int32)
    rc = fn(_ptr(boxes), _ptr(labels), _ptr(offsets), ctypes.c_int(n), _ptr(anchors), ctypes.c_int(a),
            ctypes.c_float(criteria), _ptr(means), _ptr(stds), ctypes.c_int(1 if offset else 0),
            ctypes.c_float(scale), _ptr(ob), _ptr(ol))
    assert rc == 0
    return ob, ol


def box_encode(boxes, labels, offsets, anchors, criteria=0.5, means=(0, 0, 0, 0), stds=(0.1, 0.1, 0.2, 0.2),
               offset=True, scale=1.0):
    """The restatement (oracle.c)."""
    return _box_call(lib().orc_box_encode, boxes, labels, offsets, anchors, criteria, means, stds, offset, scale)


def ref_box_encode(boxes, labels, offsets, anchors, criteria=0.5, means=(0, 0, 0, 0), stds=(0.1, 0.1, 0.2, 0.2),
                   offset=True, scale=1.0):
    """The reference's own BoundingBoxGraph::update_box_encoder_meta_data (needs _ref/libref.so)."""
    r = ref()
    if r is None:
        raise RuntimeError("oracle/_ref/libref.so is not available")
    r.ref_box_encode.restype = ctypes.c_int
    return _box_call(r.ref_box_encode, boxes, labels, offsets, anchors, criteria, means, stds, offset, scale)


def _match_call(fn, boxes, offsets, anchors, high, low, allow):
    n = len(offsets) - 1
    a = anchors.shape[0]
    boxes = np.ascontiguousarray(boxes, dtype=np.float32)
    offsets = np.ascontiguousarray(offsets, dtype=np.int32)
    anchors = np.ascontiguousarray(anchors, dtype=np.float32)
    out = np.zeros((n, a), dtype=np.int32)
    fn.restype = ctypes.c_int
    rc = fn(_ptr(boxes), _ptr(offsets), ctypes.c_int(n), _ptr(anchors), ctypes.c_int(a), ctypes.c_float(high),
            ctypes.c_float(low), ctypes.c_int(1 if allow else 0), _ptr(out))
    assert rc == 0
    return out


def box_iou_match(boxes, offsets, anchors, high_threshold=0.5, low_threshold=0.4, allow_low_quality_matches=True):
    """The restatement (oracle.c) of the box IoU matcher: matched box index per anchor, -1 / -2 below the thresholds."""
    return _match_call(lib().orc_box_iou_match, boxes, offsets, anchors, high_threshold, low_threshold,
                       allow_low_quality_matches)


def ref_box_iou_match(boxes, offsets, anchors, high_threshold=0.5, low_threshold=0.4, allow_low_quality_matches=True):
    """The reference's own BoundingBoxGraph::update_box_iou_matcher (needs _ref/libref.so)."""
    r = ref()
    if r is None:
        raise RuntimeError("oracle/_ref/libref.so is not available")
    return _match_call(r.ref_box_iou_match, boxes, offsets, anchors, high_threshold, low_threshold,
                       allow_low_quality_matches)


def resize_dst_size(src_w, src_h, dst_w, dst_h, mode, max_w=0, max_h=0, cap_w=1 << 30, cap_h=1 << 30):
    ow, oh = ctypes.c_uint(), ctypes.c_uint()
    lib().orc_resize_dst_size(ctypes.c_uint(src_w), ctypes.c_uint(src_h), ctypes.c_uint(dst_w), ctypes.c_uint(dst_h),
                              ctypes.c_int(mode), ctypes.c_uint(max_w), ctypes.c_uint(max_h), ctypes.c_uint(cap_w),
                              ctypes.c_uint(cap_h), ctypes.byref(ow), ctypes.byref(oh))
    return ow.value, oh.value


def crop_fixed(in_w, in_h, crop_w, crop_h, anchor_x, anchor_y):
    x, y, w, h = ctypes.c_uint(), ctypes.c_uint(), ctypes.c_uint(), ctypes.c_uint()
    lib().orc_crop_fixed(ctypes.c_uint(in_w), ctypes.c_uint(in_h), ctypes.c_uint(crop_w), ctypes.c_uint(crop_h),
                         ctypes.c_float(anchor_x), ctypes.c_float(anchor_y), ctypes.byref(x), ctypes.byref(y),
                         ctypes.byref(w), ctypes.byref(h))
    return x.value, y.value, w.value, h.value


# ---- numpy restatement of the parameter generators ----------------------------------------

def seed_sequence(seed, count=1024):
    """The seed table of ParameterFactory::set_seed (parameter_factory.cpp:114-119): std::seed_seq{seed}
    .generate() over `count` 32-bit words, as specified in the C++ standard [rand.util.seedseq]."""
    v = [seed & 0xFFFFFFFF]
    n, s = count, 1
    b = [0x8b8b8b8b] * n
    t = 11 if n >= 623 else 7 if n >= 68 else 5 if n >= 39 else 3 if n >= 7 else (n - 1) // 2
    p, q = (n - t) // 2, (n - t) // 2 + t
    m = max(s + 1, n)
    M = 0xFFFFFFFF

    def T_(x):
        return x ^ (x >> 27)

    for k in range(m):
        r1 = (1664525 * T_(b[k % n] ^ b[(k + p) % n] ^ b[(k - 1) % n])) & M
        if k == 0:
            r2 = (r1 + s) & M
        elif k <= s:
            r2 = (r1 + (k % n) + v[k - 1]) & M
        else:
            r2 = (r1 + (k % n)) & M
        b[(k + p) % n] = (b[(k + p) % n] + r1) & M
        b[(k + q) % n] = (b[(k + q) % n] + r2) & M
        b[k % n] = r2
    for k in range(m, m + n):
        r3 = (1566083941 * T_((b[k % n] + b[(k + p) % n] + b[(k - 1) % n]) & M)) & M
        r4 = (r3 - (k % n)) & M
        b[(k + p) % n] ^= r3
        b[(k + q) % n] ^= r4
        b[k % n] = r4
    return np.array(b, dtype=np.int64)


class UniformRand:
    """UniformRand<T> (parameter_random.h:37-116): std::mt19937(seed); one draw at construction; each
    renewal draws `batch` values val/max*(end-start)+start in double, cast to T."""

    def __init__(self, start, end, seed, batch, integer=False):
        self._rs = np.random.RandomState()
        self._rs.seed(int(seed) & 0xFFFFFFFF)   # init_genrand, the seeding of std::mt19937(seed)
        self.start, self.end = (start, max(end, start))
        self.batch, self.integer = batch, integer
        self._raw(1)

    def _raw(self, k):
        return self._rs.randint(0, 1 << 32, size=k, dtype=np.uint64).astype(np.float64)

    def renew(self):
        raw = self._raw(self.batch)
        if self.start == self.end:
            v = np.full(self.batch, self.start, dtype=np.float64)
        else:
            s, e = (float(self.start), float(self.end)) if self.integer else (float(np.float32(self.start)), float(np.float32(self.end)))
            v = raw / 4294967295.0 * (e - s) + s
        return np.trunc(v).astype(np.int32) if self.integer else v.astype(np.float32)


class CustomRand:
    """CustomRand<int> (parameter_random.h:118-239): cumulative distribution + upper_bound."""

    def __init__(self, values, freqs, seed, batch):
        self._rs = np.random.RandomState()
        self._rs.seed(int(seed) & 0xFFFFFFFF)
        self.values = np.asarray(values)
        f = np.asarray(freqs, dtype=np.float64)
        f = np.where(f >= 0, f, 0)
        self.cdf = np.cumsum(f / f.sum())
        self.batch = batch
        if len(self.values) > 1:
            self._rs.randint(0, 1 << 32, size=1, dtype=np.uint64)

    def renew(self):
        if len(self.values) == 1:
            return np.full(self.batch, self.values[0])
        raw = self._rs.randint(0, 1 << 32, size=self.batch, dtype=np.uint64).astype(np.float64) / 4294967295.0
        idx = np.searchsorted(self.cdf, raw, side="right")
        return self.values[idx]


# ---- random-resized-crop windows of the fused JPEG crop source ----------------------------

class _Mt19937:
    """Raw 32-bit outputs of std::mt19937(seed)."""

    def __init__(self, seed):
        self._rs = np.random.RandomState()
        self._rs.seed(int(seed) & 0xFFFFFFFF)

    def __call__(self):
        return int(self._rs.randint(0, 1 << 32, size=1, dtype=np.uint64)[0])


def _uniform_real_f32(gen, a, b):
    """std::uniform_real_distribution<float>(a, b)(mt19937) as libstdc++ evaluates it: one 32-bit draw, converted
    to float (round to nearest), divided by 2^32, pulled below 1 when the conversion rounded up to 2^32
    (std::generate_canonical<float, 24>), then canonical * (b - a) + a in float."""
    f32 = np.float32
    c = f32(f32(gen()) / f32(4294967296.0))
    if c >= f32(1.0):
        c = np.nextafter(f32(1.0), f32(0.0))
    return f32(f32(c * f32(f32(b) - f32(a))) + f32(a))


def _uniform_int(gen, lo, hi):
    """std::uniform_int_distribution<int>(lo, hi)(mt19937) as libstdc++ (GCC 11 and later) evaluates it for a
    32-bit engine: the multiply-and-reject method on a 64-bit product."""
    span = (hi - lo + 1) & 0xFFFFFFFF
    if span == 0:
        return lo + gen()
    prod = gen() * span
    low = prod & 0xFFFFFFFF
    if low < span:
        threshold = ((1 << 32) - span) % span
        while low < threshold:
            prod = gen() * span
            low = prod & 0xFFFFFFFF
    return lo + (prod >> 32)


_libm = None


def _libm_f32(name, x):
    """logf / expf of the C library (std::log / std::exp on a float)."""
    global _libm
    if _libm is None:
        _libm = ctypes.CDLL("libm.so.6")
        for fn in ("logf", "expf"):
            getattr(_libm, fn).restype = ctypes.c_float
            getattr(_libm, fn).argtypes = [ctypes.c_float]
    return np.float32(getattr(_libm, name)(float(np.float32(x))))


def _roundf_int(x):
    """(int)roundf(x) for a non-negative float below 2^23: halves away from zero."""
    return int(np.floor(np.float64(x) + 0.5))


def random_crop_window(height, width, sample_seed, aspect=(3.0 / 4, 4.0 / 3), area=(0.08, 1.0), num_attempts=10):
    """RocalRandomCropDecParam::generate_crop_window (parameter_random_crop_decoder.cpp:41-101) for one image:
    returns (x, y, w, h). Every intermediate keeps the C type of the reference's expression."""
    f32 = np.float32
    H, W = int(height), int(width)
    if H <= 0 or W <= 0:
        return (0, 0, 1, 1)
    gen = _Mt19937(sample_seed)
    a_lo, a_hi = f32(aspect[0]), f32(aspect[1])
    s_lo, s_hi = f32(area[0]), f32(area[1])
    log_lo, log_hi = _libm_f32("logf", a_lo), _libm_f32("logf", a_hi)
    max_hw = f32(f32(1.0) / a_lo)
    min_area = f32(f32(W * H) * s_lo)
    max_w = max(1, int(f32(f32(H) * a_hi)))
    max_h = max(1, int(f32(f32(W) * max_hw)))
    if f32(H * max_w) < min_area:
        ch, cw = H, max_w
    elif f32(W * max_h) < min_area:
        ch, cw = max_h, W
    else:
        left = num_attempts
        ch = cw = 1
        while left > 0:
            scale = _uniform_real_f32(gen, s_lo, s_hi)
            target = f32(scale * f32(H * W))
            ratio = _libm_f32("expf", _uniform_real_f32(gen, log_lo, log_hi))
            cw = max(1, _roundf_int(np.sqrt(f32(target * ratio))))
            ch = max(1, _roundf_int(np.sqrt(f32(target / ratio))))
            got = f32(f32(cw) / f32(ch))
            if cw <= W and ch <= H and a_lo <= got <= a_hi:
                break
            left -= 1
        if left <= 0:
            max_area = f32(f32(s_hi * f32(W)) * f32(H))
            whole = f32(f32(W) / f32(H))
            if whole > a_hi:
                ch, cw = H, max_w
            elif whole < a_lo:
                ch, cw = max_h, W
            else:
                ch, cw = H, W
            shrink = min(f32(1.0), f32(max_area / f32(cw * ch)))
            side = np.sqrt(f32(shrink))
            cw = max(1, int(f32(f32(cw) * side)))
            ch = max(1, int(f32(f32(ch) * side)))
    x = _uniform_int(gen, 0, W - cw)
    y = _uniform_int(gen, 0, H - ch)
    return (x, y, cw, ch)


def random_crop_windows(batch_seed, shapes_hw, aspect=(3.0 / 4, 4.0 / 3), area=(0.08, 1.0), num_attempts=10):
    """The windows of one batch: sample seeds = std::seed_seq{batch_seed}.generate()
    (RocalRandomCropDecParam::generate_random_seeds, parameter_random_crop_decoder.cpp:104-108), then one
    window per (height, width). Returns an (n, 4) uint32 array of x, y, w, h."""
    shapes = np.asarray(shapes_hw, dtype=np.int64).reshape(-1, 2)
    seeds = seed_sequence(int(batch_seed), count=len(shapes))
    out = np.zeros((len(shapes), 4), dtype=np.uint32)
    for i, (h, w) in enumerate(shapes):
        out[i] = random_crop_window(h, w, int(seeds[i]), aspect, area, num_attempts)
    return out


def ref_random_crop_windows(shapes_hw, aspect=(3.0 / 4, 4.0 / 3), area=(0.08, 1.0), num_attempts=10):
    """The reference build's windows for one batch and the batch seed its std::random_device drew:
    (batch_seed, (n, 4) uint32 array). None when the reference build is absent."""
    r = ref()
    if r is None:
        return None
    shapes = np.ascontiguousarray(np.asarray(shapes_hw, dtype=np.int32).reshape(-1, 2))
    out = np.zeros((len(shapes), 4), dtype=np.uint32)
    r.ref_random_crop_windows.restype = ctypes.c_uint
    seed = r.ref_random_crop_windows(_ptr(shapes), ctypes.c_int(len(shapes)), ctypes.c_float(aspect[0]),
                                     ctypes.c_float(aspect[1]), ctypes.c_float(area[0]), ctypes.c_float(area[1]),
                                     ctypes.c_int(num_attempts), _ptr(out))
    return int(seed), out


# ---- random-area crop windows of RandomCrop / CropResize -----------------------------------

class _SingleValue:
    """A single-value parameter (create_single_value_param): renew() changes nothing."""

    def __init__(self, v):
        self.v = np.float32(v)

    def renew(self):
        return self.v


class _UniformOne:
    """UniformRand<float> without an array: renew() draws one value (parameter_random.h:37-116)."""

    def __init__(self, lo, hi, seed):
        self._u = UniformRand(lo, hi, seed, 1)

    def renew(self):
        return np.float32(self._u.renew()[0])


def random_area_window(w, h, area, aspect, x_drift, y_drift):
    """RocalRandomCropParam::fill_crop_dims for one image (parameter_random_crop.cpp:48-97): up to five (area,
    aspect) renewals for a window strictly smaller than the image, placed by x_drift and y_drift (the latter renewed
    twice); else the central crop clamped to the aspect range 0.75 .. 1.333. Parameters are objects with renew()
    returning the new float value. Returns (x, y, cw, ch)."""
    f32 = np.float32
    w, h = int(w), int(h)
    lo, hi = f32(0.7500), f32(1.333)
    cw = ch = 0
    for _ in range(5):
        a, r = area.renew(), aspect.renew()
        target = float(f32(f32(a * f32(h)) * f32(w)))                 # float product, then held in a double
        cw = int(np.sqrt(np.float64(target) * np.float64(r)))
        ch = int(np.sqrt(np.float64(target) * np.float64(f32(f32(1) / r))))
        if ch < h and cw < w:
            xd = x_drift.renew()
            y_drift.renew()
            yd = y_drift.renew()
            return (int(f32(xd * f32(w - cw))), int(f32(yd * f32(h - ch))), cw, ch)
    ratio = f32(f32(w) / f32(h))
    if ratio < lo:
        cw = w
        ch = int(f32(f32(cw) / lo))
    elif ratio > hi:
        ch = h
        cw = int(f32(f32(ch) * hi))
    else:
        cw, ch = w, h
    return ((w - cw) // 2, (h - ch) // 2, cw, ch)


def random_area_windows(wh, fixed=None, seed=None, first_entry=0):
    """Windows for a batch, in sample order. fixed = (area, aspect, x_drift, y_drift) single values, or seed = the
    ParameterFactory seed whose table entries first_entry .. first_entry+3 start the default ranges of x_drift
    (0.01..0.99), y_drift (0.01..0.99), area (0.08..0.99) and aspect (0.75..1.333), the order in which the class
    creates them."""
    wh = np.asarray(wh).reshape(-1, 2)
    if fixed is not None:
        area, aspect, xd, yd = [_SingleValue(v) for v in fixed]
    else:
        table = seed_sequence(int(seed), 1024)
        e = [int(table[(first_entry + k) % 1024]) for k in range(4)]
        xd = _UniformOne(0.01, 0.99, e[0])
        yd = _UniformOne(0.01, 0.99, e[1])
        area = _UniformOne(0.08, 0.99, e[2])
        aspect = _UniformOne(0.7500, 1.333, e[3])
    return np.array([random_area_window(w, h, area, aspect, xd, yd) for w, h in wh], dtype=np.uint32)


def ref_random_area_windows(wh, fixed=None, seed=0):
    """The reference build's windows, and the index of the first seed-table entry its parameters took."""
    r = ref()
    if r is None:
        return None
    wh = np.ascontiguousarray(np.asarray(wh, dtype=np.uint32).reshape(-1, 2))
    out = np.zeros((len(wh), 4), dtype=np.uint32)
    f4 = np.asarray(fixed if fixed is not None else (0, 0, 0, 0), dtype=np.float32)
    r.ref_random_area_windows.restype = ctypes.c_uint
    first = r.ref_random_area_windows(_ptr(wh), ctypes.c_int(len(wh)), ctypes.c_int(1 if fixed is not None else 0), _ptr(f4),
                                      ctypes.c_uint(seed), _ptr(out))
    return out, int(first)


# ---- the reference's own pixel kernels, compiled for the host (oracle/_ref/libref_hip.so) ----------

_ref_hip = None


def ref_hip():
    """The host build of rocAL/rocAL_hip/rocal_hip_kernels.cpp, or None when neither the reference tree nor a
    prebuilt copy exists."""
    global _ref_hip
    if _ref_hip is None:
        path = _build.build_ref_hip()
        if path is None:
            return None
        _ref_hip = ctypes.CDLL(path)
    return _ref_hip


def _hip_resize(fn, arena, src_w, src_h, src_stride, src_offset, dst_w, dst_h, channels):
    n = len(src_w)
    u32 = lambda a: np.ascontiguousarray(a, dtype=np.uint32)   # noqa: E731
    sw, sh, ss, dw, dh = u32(src_w), u32(src_h), u32(src_stride), u32(dst_w), u32(dst_h)
    so = np.ascontiguousarray(src_offset, dtype=np.uint64)
    mw, mh = int(dw.max()), int(dh.max())
    out = np.zeros((n, mh, mw, 3) if channels == 3 else (n, mh, mw), dtype=np.uint8)
    arena = np.ascontiguousarray(arena, dtype=np.uint8)
    fn.restype = ctypes.c_int
    rc = fn(_ptr(arena), ctypes.c_size_t(arena.size), ctypes.c_int(n), _ptr(sw), _ptr(sh), _ptr(ss), _ptr(so), _ptr(dw), _ptr(dh),
            ctypes.c_uint(mw), ctypes.c_uint(mh), _ptr(out))
    assert rc == 0
    return out


def ref_hip_resize_bilinear(arena, src_w, src_h, src_stride, src_offset, dst_w, dst_h):
    """resize_bilinear_pkd_hip_tensor (rocal_hip_kernels.cpp:446-485) on interleaved RGB images: returns
    [n][max dst_h][max dst_w][3] uint8, sample i valid in its dst_h[i] x dst_w[i] corner."""
    return _hip_resize(ref_hip().ref_hip_resize_bilinear_pkd3, arena, src_w, src_h, src_stride, src_offset, dst_w, dst_h, 3)


def ref_hip_resize_generic(arena, src_w, src_h, src_stride, src_offset, dst_w, dst_h):
    """resize_generic_pln1_hip_tensor (rocal_hip_kernels.cpp:514-589, the triangular filter) on single-channel
    planes: returns [n][max dst_h][max dst_w] uint8."""
    return _hip_resize(ref_hip().ref_hip_resize_generic_pln1, arena, src_w, src_h, src_stride, src_offset, dst_w, dst_h, 1)


def ref_hip_copy_int8(images, nchw, fp16, mul, add, reverse_channels=False):
    """Hip_CopyInt8ToNCHW_* / Hip_CopyInt8ToNHWC_* (rocal_hip_kernels.cpp:40-217) on a [n][h][w][3] uint8 batch."""
    images = np.ascontiguousarray(images, dtype=np.uint8)
    n, h, w, _ = images.shape
    out = np.zeros((n, 3, h, w) if nchw else (n, h, w, 3), dtype=np.float16 if fp16 else np.float32)
    m, a = np.asarray(mul, dtype=np.float32), np.asarray(add, dtype=np.float32)
    fn = ref_hip().ref_hip_copy_int8
    fn.restype = ctypes.c_int
    rc = fn(_ptr(images), ctypes.c_int(n), ctypes.c_int(h), ctypes.c_int(w), ctypes.c_int(1 if nchw else 0),
            ctypes.c_int(1 if fp16 else 0), _ptr(m), _ptr(a), ctypes.c_int(1 if reverse_channels else 0), _ptr(out))
    assert rc == 0
    return out


# ---- crop windows of RocalCropParam ---------------------------------------------------------------------

def rocal_crop_windows(wh, mode, crop_w, crop_h, f):
    """RocalCropParam::fill_crop_dims (parameter_rocal_crop.cpp:49-85) for a batch of input sizes wh = n x {w, h}.
    mode 0: fixed anchors f = (anchor_x, anchor_y); mode 1: absolute corner f = (x1, y1) (a corner at or beyond the
    image falls back to 0); mode 2: random branch with the factor values f = (width, height, x drift, y drift) already
    drawn. Returns n x {x1, y1, crop_w, crop_h, x2, y2} uint32, x2 / y2 clipped to the image as the class does."""
    f32 = np.float32
    wh = np.asarray(wh, dtype=np.int64).reshape(-1, 2)
    out = np.zeros((len(wh), 6), dtype=np.uint32)
    for i, (w, h) in enumerate(wh):
        w, h = int(w), int(h)
        if mode in (0, 1):
            cw = crop_w if (0 < crop_w <= w) else w
            ch = crop_h if (0 < crop_h <= h) else h
            if mode == 0:
                x1 = int(np.rint(f32(f32(f[0]) * f32(w - cw))))
                y1 = int(np.rint(f32(f32(f[1]) * f32(h - ch))))
            else:
                x1 = 0 if int(f[0]) >= w else int(f[0])
                y1 = 0 if int(f[1]) >= h else int(f[1])
        else:
            cw = int(f32(f32(f[0]) * f32(w)))
            ch = int(f32(f32(f[1]) * f32(h)))
            x1 = int(f32(f32(f[2]) * f32(w - cw)))
            y1 = int(f32(f32(f[3]) * f32(h - ch)))
        out[i] = (x1, y1, cw, ch, min(x1 + cw, w), min(y1 + ch, h))
    return out


def ref_rocal_crop_windows(wh, mode, crop_w, crop_h, f):
    """The reference class itself (needs _ref/libref.so)."""
    r = ref()
    if r is None:
        return None
    wh = np.ascontiguousarray(np.asarray(wh, dtype=np.uint32).reshape(-1, 2))
    out = np.zeros((len(wh), 6), dtype=np.uint32)
    f4 = np.zeros(4, dtype=np.float32)
    f4[:len(f)] = f
    r.ref_rocal_crop_windows.restype = ctypes.c_int
    rc = r.ref_rocal_crop_windows(_ptr(wh), ctypes.c_int(len(wh)), ctypes.c_int(mode), ctypes.c_uint(crop_w), ctypes.c_uint(crop_h),
                                  _ptr(f4), _ptr(out))
    assert rc == 0
    return out


# ---- bounding boxes that follow the augmentations (the reference's meta nodes) ------------------------
# Boxes are float32 ltrb in the coordinate space of the node's input; each function takes and returns
# (boxes [total][4], labels [total], offsets [n+1]).

def _split(boxes, labels, offsets):
    boxes = np.asarray(boxes, dtype=np.float32).reshape(-1, 4)
    labels = np.asarray(labels, dtype=np.int32)
    return [(boxes[offsets[i]:offsets[i + 1]].copy(), labels[offsets[i]:offsets[i + 1]].copy()) for i in range(len(offsets) - 1)]


def _join(per):
    counts = [len(b) for b, _ in per]
    boxes = np.concatenate([np.asarray(b, dtype=np.float32).reshape(-1, 4) for b, _ in per]) if per else np.zeros((0, 4), np.float32)
    labels = np.concatenate([np.asarray(l, dtype=np.int32) for _, l in per]) if per else np.zeros(0, np.int32)
    return boxes, labels, np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)


def _covered_fraction(box, crop, entire=False):
    """MetaNode::BBoxIntersectionOverUnion (include/meta_data/meta_node.h:42-58): intersection / area of the box
    (the default), or the true IoU when `entire`; float32 products, the quotient widened to double."""
    f32 = np.float32
    xa, ya = max(box[0], crop[0]), max(box[1], crop[1])
    xb, yb = min(box[2], crop[2]), min(box[3], crop[3])
    inter = f32(max(f32(0), f32(xb - xa)) * max(f32(0), f32(yb - ya)))
    a1 = f32(f32(box[3] - box[1]) * f32(box[2] - box[0]))
    a2 = f32(f32(crop[3] - crop[1]) * f32(crop[2] - crop[0]))
    with np.errstate(divide="ignore", invalid="ignore"):
        return float(f32(inter / f32(f32(a1 + a2) - inter))) if entire else float(f32(inter / a1))


def meta_crop(boxes, labels, offsets, windows, mirror=None, resize_to=None, iou_threshold=0.25):
    """CropMetaNode / CropMirrorNormalizeMetaNode / ResizeCropMirrorMetaNode (meta_node_crop.cpp:44-79,
    meta_node_crop_mirror_normalize.cpp:53-90, meta_node_resize_crop_mirror.cpp:55-100): a box is kept when at least
    iou_threshold of its area lies in the window {x1, y1, w, h}; kept boxes are clipped, shifted to the window's
    origin, mirrored about the window's width and (resize_to = (w, h)) scaled by resize / window. A sample left
    without boxes gets the whole window with label 0."""
    f32 = np.float32
    per = []
    for i, (b, l) in enumerate(_split(boxes, labels, offsets)):
        x1, y1, cw, ch = [f32(v) for v in windows[i][:4]]
        crop = (x1, y1, f32(x1 + cw), f32(y1 + ch))
        kb, kl = [], []
        for q, lab in zip(b, l):
            if _covered_fraction(q, crop) >= float(f32(iou_threshold)):
                nl, nt = f32(max(crop[0], q[0]) - crop[0]), f32(max(crop[1], q[1]) - crop[1])
                nr, nb = f32(min(crop[2], q[2]) - crop[0]), f32(min(crop[3], q[3]) - crop[1])
                if mirror is not None and mirror[i] == 1:
                    nl, nr = f32(cw - nr), f32(cw - nl)
                if resize_to is not None:
                    sx, sy = f32(f32(resize_to[0]) / cw), f32(f32(resize_to[1]) / ch)
                    nl, nt, nr, nb = f32(nl * sx), f32(nt * sy), f32(nr * sx), f32(nb * sy)
                kb.append((nl, nt, nr, nb))
                kl.append(lab)
        if not kb:
            kb, kl = [(f32(0), f32(0), cw, ch)], [0]
        per.append((kb, kl))
    return _join(per)


def meta_flip(boxes, labels, offsets, roi_wh, h_flip, v_flip):
    """FlipMetaNode (meta_node_flip.cpp:30-62): l, r -> w - r, w - l and t, b -> h - b, h - t."""
    f32 = np.float32
    per = []
    for i, (b, l) in enumerate(_split(boxes, labels, offsets)):
        w, h = f32(roi_wh[i][0]), f32(roi_wh[i][1])
        for q in b:
            if h_flip[i]:
                q[0], q[2] = f32(w - q[2]), f32(w - q[0])
            if v_flip[i]:
                q[1], q[3] = f32(h - q[3]), f32(h - q[1])
        per.append((b, l))
    return _join(per)


def box_transform(boxes, labels, offsets, windows, rule, mirror_h=None, mirror_v=None):
    """Normalised boxes through a window and a mirror, float32 operation by operation: the form in which the library
    keeps boxes (every coordinate a fraction of the current image). rule 0: the quarter-area rule of the Crop /
    CropMirrorNormalize / ResizeCropMirror meta nodes (stand-in: the whole window, label 0); rule 1: the centre rule
    of update_random_bbox_meta_data (stand-in: an empty box, label 0). windows: [n][4] = l, t, r, b."""
    f32 = np.float32
    per = []
    for i, (b, lab) in enumerate(_split(boxes, labels, offsets)):
        l, t, r, bt = (f32(v) for v in windows[i])
        ww, wh = f32(r - l), f32(bt - t)
        kb, kl = [], []
        for q, la in zip(b, lab):
            if rule == 1:
                xc, yc = f32(f32(0.5) * f32(q[0] + q[2])), f32(f32(0.5) * f32(q[1] + q[3]))
                keep = xc > l and xc < r and yc > t and yc < bt
            else:
                xa, ya, xb, yb = max(q[0], l), max(q[1], t), min(q[2], r), min(q[3], bt)
                inter = f32(max(f32(0), f32(xb - xa)) * max(f32(0), f32(yb - ya)))
                area = f32(f32(q[3] - q[1]) * f32(q[2] - q[0]))
                with np.errstate(divide="ignore", invalid="ignore"):
                    keep = f32(inter / area) >= f32(0.25)
            if keep:
                kb.append([f32(f32(max(q[0], l) - l) / ww), f32(f32(max(q[1], t) - t) / wh),
                           f32(f32(min(q[2], r) - l) / ww), f32(f32(min(q[3], bt) - t) / wh)])
                kl.append(la)
        if not kb:
            kb, kl = [[f32(0), f32(0), f32(0), f32(0)] if rule == 1 else [f32(0), f32(0), f32(1), f32(1)]], [0]
        for q in kb:
            if mirror_h is not None and mirror_h[i]:
                q[0], q[2] = f32(f32(1) - q[2]), f32(f32(1) - q[0])
            if mirror_v is not None and mirror_v[i]:
                q[1], q[3] = f32(f32(1) - q[3]), f32(f32(1) - q[1])
        per.append((kb, kl))
    return _join(per)


def meta_rotate(boxes, labels, offsets, roi_wh, angles_deg, dst_w, dst_h):
    """RotateMetaNode (meta_node_rotate.cpp:27-103), in pixels as written: the corners of a box are rotated about the
    image centres (source: roi / 2 in float; destination: size // 2), the new box is their bounding box with
    l = min(0, .) and t = min(0, .), kept when inter / area(new box) >= 0.25 against the destination image and clipped
    to it; a sample left without boxes gets the whole destination image with label 0."""
    f32 = np.float32
    W, H = f32(dst_w), f32(dst_h)
    per = []
    for i, (b, l) in enumerate(_split(boxes, labels, offsets)):
        radian = f32(np.float64(f32(angles_deg[i])) * 3.14159265 / 180)
        r0, r1 = f32(math.cos(float(radian))), f32(math.sin(float(radian)))
        r2, r3 = f32(-1 * r1), r0
        dcx, dcy = f32(int(dst_w) // 2), f32(int(dst_h) // 2)
        scx, scy = f32(f32(roi_wh[i][0]) / 2), f32(f32(roi_wh[i][1]) / 2)
        kb, kl = [], []
        for q, lab in zip(b, l):
            x, y = f32(q[0]), f32(q[1])
            bw, bh = f32(q[2] - q[0]), f32(q[3] - q[1])

            def rot(px, py):
                return (f32(f32(f32(r0 * f32(px - scx)) + f32(r1 * f32(py - scy))) + dcx),
                        f32(f32(f32(r2 * f32(px - scx)) + f32(r3 * f32(py - scy))) + dcy))
            pts = [rot(x, y), rot(f32(x + bw), y), rot(x, f32(y + bh)), rot(f32(x + bw), f32(y + bh))]
            xs, ys = [p[0] for p in pts], [p[1] for p in pts]
            bl, bt = min(f32(0), min(xs)), min(f32(0), min(ys))
            br, bb = max(xs), max(ys)
            xa, ya, xb, yb = max(bl, f32(0)), max(bt, f32(0)), min(br, W), min(bb, H)
            inter = f32(max(f32(0), f32(xb - xa)) * max(f32(0), f32(yb - ya)))
            area = f32(f32(bb - bt) * f32(br - bl))
            with np.errstate(divide="ignore", invalid="ignore"):
                keep = f32(inter / area) >= f32(0.25)
            if keep:
                kb.append((max(f32(0), bl), max(f32(0), bt), min(W, br), min(H, bb)))
                kl.append(lab)
        if not kb:
            kb, kl = [(0, 0, W, H)], [0]
        per.append((kb, kl))
    return _join(per)


def meta_resize(boxes, labels, offsets, src_wh, dst_wh):
    """ResizeMetaNode (meta_node_resize.cpp:25-55): every coordinate times dst / src of its axis."""
    f32 = np.float32
    per = []
    for i, (b, l) in enumerate(_split(boxes, labels, offsets)):
        sx = f32(f32(dst_wh[i][0]) / f32(src_wh[i][0]))
        sy = f32(f32(dst_wh[i][1]) / f32(src_wh[i][1]))
        b[:, 0::2] = (b[:, 0::2] * sx).astype(np.float32)
        b[:, 1::2] = (b[:, 1::2] * sy).astype(np.float32)
        per.append((b, l))
    return _join(per)


def meta_ssd_random_crop(boxes, labels, offsets, windows, iou_range=(0.0, 1.0), entire_iou=False):
    """SSDRandomCropMetaNode (meta_node_ssd_random_crop.cpp:31-85): a box is kept when its centre lies in the
    closed window and its covered fraction (or IoU) lies in iou_range; kept boxes are clipped and divided by
    the window's size (they leave normalised to the crop). No stand-in box is added."""
    f32 = np.float32
    per = []
    for i, (b, l) in enumerate(_split(boxes, labels, offsets)):
        x1, y1, cw, ch = [f32(v) for v in windows[i][:4]]
        crop = (x1, y1, f32(x1 + cw), f32(y1 + ch))
        kb, kl = [], []
        for q, lab in zip(b, l):
            xc, yc = f32(f32(0.5) * f32(q[0] + q[2])), f32(f32(0.5) * f32(q[1] + q[3]))
            inside = crop[0] <= xc <= crop[2] and crop[1] <= yc <= crop[3]
            v = f32(_covered_fraction(q, crop, entire_iou))
            if f32(iou_range[0]) <= v <= f32(iou_range[1]) and inside:
                w, h = f32(crop[2] - crop[0]), f32(crop[3] - crop[1])
                kb.append((f32(f32(max(crop[0], q[0]) - crop[0]) / w), f32(f32(max(crop[1], q[1]) - crop[1]) / h),
                           f32(f32(min(crop[2], q[2]) - crop[0]) / w), f32(f32(min(crop[3], q[3]) - crop[1]) / h)))
                kl.append(lab)
        per.append((kb, kl))
    return _join(per)


def random_bbox_meta(boxes, labels, offsets, crop_xywh, roi_wh):
    """BoundingBoxGraph::update_random_bbox_meta_data (bounding_box_graph.cpp:71-118) as written: the window is
    l = x * roi_w, t = y * roi_h, r = (l + w) * roi_w, b = (t + h) * roi_h (the already scaled corner enters the
    second product); a box is kept when its centre, evaluated in double, lies strictly inside; kept boxes are
    clipped and shifted; a sample left without boxes gets one zero box with label 0."""
    f32 = np.float32
    per = []
    for i, (b, l) in enumerate(_split(boxes, labels, offsets)):
        rw, rh = f32(roi_wh[i][0]), f32(roi_wh[i][1])
        cl, ct = f32(f32(crop_xywh[i][0]) * rw), f32(f32(crop_xywh[i][1]) * rh)
        cr, cb = f32(f32(cl + f32(crop_xywh[i][2])) * rw), f32(f32(ct + f32(crop_xywh[i][3])) * rh)
        kb, kl = [], []
        for q, lab in zip(b, l):
            xc, yc = 0.5 * float(f32(q[0] + q[2])), 0.5 * float(f32(q[1] + q[3]))
            if float(cl) < xc < float(cr) and float(ct) < yc < float(cb):
                kb.append((f32(max(cl, q[0]) - cl), f32(max(ct, q[1]) - ct), f32(min(cr, q[2]) - cl), f32(min(cb, q[3]) - ct)))
                kl.append(lab)
        if not kb:
            kb, kl = [(0, 0, 0, 0)], [0]
        per.append((kb, kl))
    return _join(per)


def ref_random_bbox_meta(boxes, labels, offsets, crop_xywh, roi_wh):
    """The reference's own update_random_bbox_meta_data (needs _ref/libref.so)."""
    r = ref()
    if r is None:
        return None
    boxes = np.ascontiguousarray(boxes, dtype=np.float32).reshape(-1, 4)
    labels = np.ascontiguousarray(labels, dtype=np.int32)
    offsets = np.ascontiguousarray(offsets, dtype=np.int32)
    n = len(offsets) - 1
    crops = np.ascontiguousarray(crop_xywh, dtype=np.float32).reshape(n, 4)
    roi = np.ascontiguousarray(roi_wh, dtype=np.uint32).reshape(n, 2)
    cap = max(len(boxes), n) + n
    ob, ol, oc = np.zeros((cap, 4), np.float32), np.zeros(cap, np.int32), np.zeros(n, np.int32)
    r.ref_random_bbox_meta.restype = ctypes.c_int
    k = r.ref_random_bbox_meta(_ptr(boxes), _ptr(labels), _ptr(offsets), ctypes.c_int(n), _ptr(crops), _ptr(roi), _ptr(ob),
                               _ptr(ol), _ptr(oc))
    return ob[:k].copy(), ol[:k].copy(), np.concatenate([[0], np.cumsum(oc)]).astype(np.int32)


# ---- random-bbox-crop windows (rocalRandomBBoxCrop) -----------------------------------------------------------

class _Mt19937Seq:
    """std::mt19937 constructed from a std::seed_seq over `words`: the 624-word state is seed_seq::generate's
    output, and libstdc++ replaces an all-zero state (ignoring the low 31 bits of word 0) by 2^31."""

    def __init__(self, words):
        state = _seed_seq_generate([int(w) & 0xFFFFFFFF for w in words], 624)
        if (state[0] & 0x80000000) == 0 and not any(state[1:]):
            state[0] = 0x80000000
        self._rs = np.random.RandomState()
        self._rs.set_state(("MT19937", np.array(state, dtype=np.uint32), 624))

    def __call__(self):
        return int(self._rs.randint(0, 1 << 32, size=1, dtype=np.uint64)[0])


def _seed_seq_generate(v, n):
    """std::seed_seq{v...}.generate over n 32-bit words ([rand.util.seedseq])."""
    s = len(v)
    b = [0x8b8b8b8b] * n
    t = 11 if n >= 623 else 7 if n >= 68 else 5 if n >= 39 else 3 if n >= 7 else (n - 1) // 2
    p, q = (n - t) // 2, (n - t) // 2 + t
    m = max(s + 1, n)
    M = 0xFFFFFFFF

    def T_(x):
        return x ^ (x >> 27)

    for k in range(m):
        r1 = (1664525 * T_(b[k % n] ^ b[(k + p) % n] ^ b[(k - 1) % n])) & M
        if k == 0:
            r2 = (r1 + s) & M
        elif k <= s:
            r2 = (r1 + (k % n) + v[k - 1]) & M
        else:
            r2 = (r1 + (k % n)) & M
        b[(k + p) % n] = (b[(k + p) % n] + r1) & M
        b[(k + q) % n] = (b[(k + q) % n] + r2) & M
        b[k % n] = r2
    for k in range(m, m + n):
        r3 = (1566083941 * T_((b[k % n] + b[(k + p) % n] + b[(k - 1) % n]) & M)) & M
        r4 = (r3 - (k % n)) & M
        b[(k + p) % n] ^= r3
        b[(k + q) % n] ^= r4
        b[k % n] = r4
    return b


class BBoxCropSampler:
    """RandomBBoxCropReader::get_batch_crop_coords (randombboxcrop_reader.cpp:216-313): per sample, from that
    sample position's own generator, draw one of seven minimum-IoU options (the last keeps the whole image), a width
    and a height factor in 0.3 .. 1 whose ratio lies in 0.5 .. 2, and a position whose left edge is aligned to 8
    pixels; with all_boxes_overlap every box must reach the option's IoU with the window, and at least one box centre
    must lie strictly inside it; otherwise everything is drawn again. 128 generators serve the samples in turn
    (SeededRNG<std::mt19937, 4>, randombboxcrop_reader.h:41-72); here each is seeded through std::seed_seq from four
    consecutive outputs of std::mt19937(seed) (the reference takes those words from std::random_device)."""

    OPTIONS = (-1.0, 0.1, 0.3, 0.5, 0.7, 0.9, 0.0)

    def __init__(self, seed, all_boxes_overlap=True):
        master = _Mt19937(seed)
        self.rngs = [_Mt19937Seq([master() for _ in range(4)]) for _ in range(128)]
        self.count = 0
        self.all_boxes_overlap = all_boxes_overlap

    @staticmethod
    def _iou(box, crop):
        f32 = np.float32
        xa, ya = max(box[0], crop[0]), max(box[1], crop[1])
        xb, yb = min(box[2], crop[2]), min(box[3], crop[3])
        inter = f32(max(f32(0), f32(xb - xa)) * max(f32(0), f32(yb - ya)))
        a1 = f32(f32(box[3] - box[1]) * f32(box[2] - box[0]))
        a2 = f32(f32(crop[3] - crop[1]) * f32(crop[2] - crop[0]))
        with np.errstate(divide="ignore", invalid="ignore"):
            return f32(inter / f32(f32(a1 + a2) - inter))

    def window(self, boxes, img_w):
        """One sample: boxes [k][4] float32 ltrb as the sampler sees them; returns (x, y, w, h) float32."""
        f32 = np.float32
        gen = self.rngs[self.count % 128]
        self.count += 1
        boxes = np.asarray(boxes, dtype=np.float32).reshape(-1, 4)
        crop = None
        while True:
            option = _uniform_int(gen, 0, 6)
            if option == 6:
                crop = (f32(0), f32(0), f32(1), f32(1))
                break
            min_iou = f32(self.OPTIONS[option])
            wf = _uniform_real_f32(gen, 0.3, 1.0)
            hf = _uniform_real_f32(gen, 0.3, 1.0)
            ratio = f32(wf / hf)
            if float(ratio) < 0.5 or float(ratio) > 2.0:
                continue
            # the reference builds the position distributions from double bounds 1.0 - factor, narrowed to float
            x = _uniform_real_f32(gen, 0.0, f32(1.0 - float(wf)))
            y = _uniform_real_f32(gen, 0.0, f32(1.0 - float(hf)))
            x = f32(f32(int(_lround_f32(f32(x * f32(img_w)))) & ~7) / f32(img_w))
            crop = (x, y, f32(x + wf), f32(y + hf))
            if self.all_boxes_overlap and any(self._iou(b, crop) < min_iou for b in boxes):
                continue
            inside = 0
            for b in boxes:
                xc, yc = 0.5 * float(f32(b[0] + b[2])), 0.5 * float(f32(b[1] + b[3]))
                if float(crop[0]) < xc < float(crop[2]) and float(crop[1]) < yc < float(crop[3]):
                    inside += 1
            if inside == 0:
                continue
            break
        return (crop[0], crop[1], f32(crop[2] - crop[0]), f32(crop[3] - crop[1]))

    def windows(self, boxes, offsets, img_w):
        boxes = np.asarray(boxes, dtype=np.float32).reshape(-1, 4)
        return np.array([self.window(boxes[offsets[i]:offsets[i + 1]], int(img_w[i])) for i in range(len(offsets) - 1)],
                        dtype=np.float32)


def _lround_f32(x):
    """std::lround of a non-negative float: halves away from zero."""
    return int(np.floor(np.float64(x) + 0.5))


def ref_random_bbox_crop(boxes, offsets, img_w, seed, all_boxes_overlap=True):
    """The reference's own sampler with its generators replaced as described in ref_bbox_crop_driver.cpp."""
    r = ref()
    if r is None:
        return None
    boxes = np.ascontiguousarray(boxes, dtype=np.float32).reshape(-1, 4)
    offsets = np.ascontiguousarray(offsets, dtype=np.int32)
    img_w = np.ascontiguousarray(img_w, dtype=np.int32)
    n = len(offsets) - 1
    out = np.zeros((n, 4), dtype=np.float32)
    r.ref_random_bbox_crop.restype = ctypes.c_int
    rc = r.ref_random_bbox_crop(_ptr(boxes), _ptr(offsets), ctypes.c_int(n), _ptr(img_w), ctypes.c_uint(seed),
                                ctypes.c_int(1 if all_boxes_overlap else 0), _ptr(out))
    assert rc == 0
    return out

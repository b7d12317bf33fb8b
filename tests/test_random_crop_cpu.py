"""Random-resized-crop windows of the fused JPEG crop source (rocalFusedJpegCrop*): the numpy restatement and the
product's host sampler against golden vectors produced by the reference's own RocalRandomCropDecParam
(tests/golden/make_golden.py), and against the reference build itself when it is present."""
import ctypes
import os

import numpy as np
import pytest

from oracle import pyoracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "random_crop_windows.npz")


def _cases():
    g = np.load(GOLDEN)
    for k in range(8):
        p = g["params_%d" % k]
        yield int(g["seed_%d" % k][0]), g["shapes_%d" % k], (float(p[0]), float(p[1])), (float(p[2]), float(p[3])), int(p[4]), \
            g["windows_%d" % k]


def _product_windows(seed, shapes, aspect, area, attempts):
    from rocal_b200 import _capi as C
    shapes = np.ascontiguousarray(shapes, dtype=np.int32)
    out = np.zeros((len(shapes), 4), dtype=np.uint32)
    rc = C.random_crop_windows(seed, shapes.ctypes.data_as(ctypes.POINTER(ctypes.c_int)), len(shapes), (ctypes.c_float * 2)(*area),
                               (ctypes.c_float * 2)(*aspect), attempts, out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint)))
    assert rc == 0
    return out


def test_restatement_matches_golden():
    for seed, shapes, aspect, area, attempts, win in _cases():
        assert np.array_equal(O.random_crop_windows(seed, shapes, aspect, area, attempts), win)


def test_product_sampler_matches_golden():
    for seed, shapes, aspect, area, attempts, win in _cases():
        assert np.array_equal(_product_windows(seed, shapes, aspect, area, attempts), win)


def test_windows_are_valid():
    """Inside the image; an ordinary image with many attempts gets a window inside both ranges."""
    for seed, shapes, aspect, area, attempts, win in _cases():
        w = win.astype(np.int64)
        assert (w[:, 2] >= 1).all() and (w[:, 3] >= 1).all()
        assert (w[:, 0] + w[:, 2] <= shapes[:, 1]).all() and (w[:, 1] + w[:, 3] <= shapes[:, 0]).all()
    seed, shapes, aspect, area, attempts, win = list(_cases())[1]          # 100 attempts
    big = (shapes[:, 0] > 200) & (shapes[:, 1] > 200)
    ratio = win[big, 2] / win[big, 3]
    frac = win[big, 2] * win[big, 3] / (shapes[big, 0] * shapes[big, 1])
    assert big.sum() > 20
    assert (ratio >= aspect[0] - 1e-6).all() and (ratio <= aspect[1] + 1e-6).all()
    assert (frac >= area[0] * 0.98).all() and (frac <= area[1] * 1.02).all()


def test_restatement_matches_reference_build():
    if O.ref() is None:
        pytest.skip("reference tree not present")
    rng = np.random.Generator(np.random.PCG64(5))
    for trial in range(12):
        n = 40
        shapes = np.stack([rng.integers(1, 1000, n), rng.integers(1, 1000, n)], axis=1).astype(np.int32)
        if trial % 4 == 1:
            shapes[:, 0] = rng.integers(1, 20, n)
        if trial % 4 == 2:
            shapes[:, 1] = rng.integers(1, 20, n)
        aspect = (0.75, 4.0 / 3) if trial % 3 else (0.8, 1.25)
        attempts = 10 if trial % 2 else 1
        if trial == 3:      # empty, one-pixel and extremely thin images
            shapes[:7] = [[0, 10], [10, 0], [1, 1], [1, 2000], [2000, 1], [2, 2], [3, 1000]]
        seed, win = O.ref_random_crop_windows(shapes, aspect, (0.08, 1.0), attempts)
        assert np.array_equal(O.random_crop_windows(seed, shapes, aspect, (0.08, 1.0), attempts), win)
        assert np.array_equal(_product_windows(seed, shapes, aspect, (0.08, 1.0), attempts), win)


def test_bad_ranges_are_refused():
    from rocal_b200 import _capi as C
    shapes = np.array([[10, 10]], dtype=np.int32)
    out = np.zeros((1, 4), dtype=np.uint32)
    sp, op = shapes.ctypes.data_as(ctypes.POINTER(ctypes.c_int)), out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint))
    ok = (ctypes.c_float * 2)(0.08, 1.0)
    assert C.random_crop_windows(1, sp, 1, (ctypes.c_float * 2)(0.0, 1.0), ok, 10, op) != 0
    assert C.random_crop_windows(1, sp, 1, ok, (ctypes.c_float * 2)(2.0, 1.0), 10, op) != 0
    assert C.random_crop_windows(1, sp, 1, ok, ok, 0, op) != 0
    assert C.random_crop_windows(1, sp, 1, ok, ok, 10, op) == 0


# ---- the random-area rule of rocalRandomCrop / rocalCropResize --------------------------------

AREA_GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "random_area_windows.npz")


def _product_area_windows(wh, area, aspect, xd, yd):
    from rocal_b200 import _capi as C
    wh = np.ascontiguousarray(wh, dtype=np.uint32)
    out = np.zeros((len(wh), 4), dtype=np.uint32)
    rc = C.random_area_windows(wh.ctypes.data_as(ctypes.POINTER(ctypes.c_uint)), len(wh), area, aspect, xd, yd,
                               out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint)))
    assert rc == 0
    return out


def test_random_area_restatement_matches_golden():
    g = np.load(AREA_GOLDEN)
    for k in range(10):
        if k % 2:
            got = O.random_area_windows(g["wh_%d" % k], fixed=g["fixed_%d" % k])
        else:
            seed, first = g["seed_%d" % k]
            got = O.random_area_windows(g["wh_%d" % k], seed=int(seed), first_entry=int(first))
        assert np.array_equal(got, g["windows_%d" % k]), k


def test_random_area_product_matches_golden_and_restatement():
    """Fixed parameter values against the golden windows; random parameters created through the API against the
    restatement started from the seed-table entries they took."""
    from rocal_b200 import _capi as C
    g = np.load(AREA_GOLDEN)
    for k in range(1, 10, 2):
        f = g["fixed_%d" % k]
        ps = [C.Param(C.create_float_parameter(float(v)), False) for v in f]
        got = _product_area_windows(g["wh_%d" % k], ps[0], ps[1], ps[2], ps[3])
        win = g["windows_%d" % k].copy()
        # the window handed to the kernels is kept inside the image and at least 1x1
        wh = g["wh_%d" % k].astype(np.int64)
        exp = win.astype(np.int64)
        exp[:, 0] = np.minimum(exp[:, 0], wh[:, 0] - 1)
        exp[:, 1] = np.minimum(exp[:, 1], wh[:, 1] - 1)
        exp[:, 2] = np.maximum(1, np.minimum(exp[:, 2], wh[:, 0] - exp[:, 0]))
        exp[:, 3] = np.maximum(1, np.minimum(exp[:, 3], wh[:, 1] - exp[:, 1]))
        assert np.array_equal(got, exp), k
    C.set_seed(99)
    table = O.seed_sequence(99, 1024)
    xd = C.Param(C.create_float_uniform_rand(0.01, 0.99), False)
    first_value = np.float32(C.get_float_value(xd))
    first = None
    lo, hi = float(np.float32(0.01)), float(np.float32(0.99))
    for e in range(1024):     # which table entry did the first parameter take? (its constructor draw tells)
        rs = np.random.RandomState()
        rs.seed(int(table[e]) & 0xFFFFFFFF)
        if np.float32(float(rs.randint(0, 1 << 32, dtype=np.uint64)) / 4294967295.0 * (hi - lo) + lo) == first_value:
            first = e
            break
    assert first is not None
    yd = C.Param(C.create_float_uniform_rand(0.01, 0.99), False)
    area = C.Param(C.create_float_uniform_rand(0.08, 0.99), False)
    aspect = C.Param(C.create_float_uniform_rand(0.7500, 1.333), False)
    wh = g["wh_0"]
    got = _product_area_windows(wh, area, aspect, xd, yd)
    exp = O.random_area_windows(wh, seed=99, first_entry=first).astype(np.int64)
    exp[:, 2] = np.maximum(1, exp[:, 2])
    exp[:, 3] = np.maximum(1, exp[:, 3])
    assert np.array_equal(got, exp)


def test_random_area_restatement_matches_reference_build():
    if O.ref() is None:
        pytest.skip("reference tree not present")
    rng = np.random.Generator(np.random.PCG64(6))
    for trial in range(10):
        wh = np.stack([rng.integers(1, 900, 40), rng.integers(1, 900, 40)], axis=1).astype(np.uint32)
        if trial % 2:
            fixed = (rng.uniform(0.05, 1.3), rng.uniform(0.5, 2.0), rng.uniform(0, 1), rng.uniform(0, 1))
            win, _ = O.ref_random_area_windows(wh, fixed=fixed)
            assert np.array_equal(O.random_area_windows(wh, fixed=fixed), win)
        else:
            seed = int(rng.integers(0, 2 ** 31))
            win, first = O.ref_random_area_windows(wh, seed=seed)
            assert np.array_equal(O.random_area_windows(wh, seed=seed, first_entry=first), win)

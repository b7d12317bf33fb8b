"""The CPU oracle against the reference: golden vectors generated from reference-owned code
(tests/golden/make_golden.py), the reference build itself when present, and self-consistency
properties of the pixel restatements (whose arithmetic lives in the absent RPP library)."""
import ctypes
import os

import numpy as np
import pytest

from oracle import pyoracle as O
import synthetic as S
from rocal_b200 import tables as T

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_box_encoder_matches_golden():
    g = np.load(os.path.join(GOLDEN, "box_encoder.npz"))
    for name in ("offset", "plain", "scaled"):
        a = g[name + "_args"]
        eb, el = O.box_encode(g["boxes"], g["labels"], g["offsets"], g["anchors"], float(np.float32(a[0])), a[1:5], a[5:9],
                              bool(a[9]), float(a[10]))
        assert np.array_equal(el, g[name + "_labels"]), name
        assert np.array_equal(eb, g[name + "_boxes"]), name
        assert (el > 0).sum() > 0


def test_box_encoder_degenerate_matches_golden():
    """Zero-area and inverted boxes, degenerate anchor 0: NaN and negative IoUs follow the reference's seeding."""
    g = np.load(os.path.join(GOLDEN, "box_encoder_degenerate.npz"))
    for name, offset in (("offset", True), ("plain", False)):
        eb, el = O.box_encode(g["boxes"], g["labels"], g["offsets"], g["anchors"], 0.5, (0, 0, 0, 0), (0.1, 0.1, 0.2, 0.2),
                              offset, 1.0)
        assert np.array_equal(el, g[name + "_labels"]), name
        assert np.array_equal(eb, g[name + "_boxes"], equal_nan=True), name


def test_box_iou_matcher_matches_golden():
    g = np.load(os.path.join(GOLDEN, "box_iou_matcher.npz"))
    for name, hi, lo, allow in (("lq_05_04", 0.5, 0.4, True), ("plain_05_04", 0.5, 0.4, False), ("lq_07_03", 0.7, 0.3, True)):
        m = O.box_iou_match(g["boxes"], g["offsets"], g["anchors"], hi, lo, allow)
        assert np.array_equal(m, g[name]), name
        assert (m >= 0).sum() > 0 and (m == -2).sum() > 0
    g = np.load(os.path.join(GOLDEN, "box_encoder_degenerate.npz"))
    for name, allow in (("match_lq", True), ("match_plain", False)):
        assert np.array_equal(O.box_iou_match(g["boxes"], g["offsets"], g["anchors"], 0.5, 0.4, allow), g[name]), name


def test_box_encoder_matches_reference_build():
    if O.ref() is None:
        pytest.skip("reference tree not present: oracle/_ref/libref.so cannot be built")
    rng = S.rng_for(4)
    anchors = S.ssd300_anchors()
    boxes, labels, offs = S.random_boxes(rng, 24)
    for offset, scale, crit in ((True, 1.0, 0.5), (False, 1.0, 0.5), (True, 0.5, 0.3)):
        a = O.box_encode(boxes, labels, offs, anchors, crit, (0, 0, 0, 0), (0.1, 0.1, 0.2, 0.2), offset, scale)
        b = O.ref_box_encode(boxes, labels, offs, anchors, crit, (0, 0, 0, 0), (0.1, 0.1, 0.2, 0.2), offset, scale)
        assert np.array_equal(a[1], b[1]) and np.array_equal(a[0], b[0])


def test_box_encoder_brute_force_semantics():
    """Independent numpy statement of the matching rule on a tiny case."""
    anchors = np.array([[0, 0, .5, .5], [.5, 0, 1, .5], [0, .5, .5, 1], [.5, .5, 1, 1], [.25, .25, .75, .75]], dtype=np.float32)
    boxes = np.array([[0.0, 0.0, 0.5, 0.5], [0.3, 0.3, 0.8, 0.8], [0.0, 0.0, 0.5, 0.5]], dtype=np.float32)
    labels = np.array([3, 7, 9], dtype=np.int32)
    eb, el = O.box_encode(boxes, labels, np.array([0, 3], dtype=np.int32), anchors, 0.5, (0, 0, 0, 0), (1, 1, 1, 1), False, 1.0)
    # boxes 0 and 2 are identical and equal to anchor 0: both force-match it, the later box wins
    assert el[0, 0] == 9
    # box 1's best anchor is 4 (IoU 0.64)
    assert el[0, 4] == 7
    assert el[0, 1] == 0 and el[0, 2] == 0
    assert np.allclose(eb[0, 0], [0.25, 0.25, 0.5, 0.5])
    assert np.allclose(eb[0, 1], [0.75, 0.25, 0.5, 0.5])   # unmatched: the anchor itself as xcycwh


def test_param_rng_matches_golden():
    g = np.load(os.path.join(GOLDEN, "param_rng.npz"))
    u = O.UniformRand(0.6, 1.4, 123, 16)
    assert np.array_equal(np.concatenate([u.renew() for _ in range(3)]), g["uniform_float_seed123_0.6_1.4_b16x3"])
    u = O.UniformRand(0, 10, 77, 16, integer=True)
    assert np.array_equal(np.concatenate([u.renew() for _ in range(3)]), g["uniform_int_seed77_0_10_b16x3"])
    c = O.CustomRand(np.array([0, 1], dtype=np.int32), [0.5, 0.5], 9, 16)
    assert np.array_equal(np.concatenate([c.renew() for _ in range(3)]), g["custom_int_seed9_coin_b16x3"])
    for seed in (0, 1, 1234):
        assert np.array_equal(O.seed_sequence(seed), g["seed_seq_%d" % seed])


def test_resize_size_rules():
    # resize_shorter=256 (NOT_SMALLER, node_resize.cpp:120-137): the side whose own scale is the maximum keeps 256
    assert O.resize_dst_size(512, 256, 256, 256, 2) == (512, 256)
    assert O.resize_dst_size(300, 400, 256, 256, 2) == (256, 341)
    assert O.resize_dst_size(1080, 300, 256, 256, 2) == (922, 256)
    assert O.resize_dst_size(1080, 300, 256, 256, 2, cap_w=600) == (600, 256)
    # resize_longer (NOT_LARGER)
    assert O.resize_dst_size(400, 300, 200, 200, 3) == (200, 150)
    # stretch, default with one side given, max_size clamp
    assert O.resize_dst_size(400, 300, 100, 50, 1) == (100, 50)
    assert O.resize_dst_size(400, 300, 0, 150, 0) == (200, 150)
    assert O.resize_dst_size(400, 300, 0, 150, 0, max_w=120) == (120, 150)
    for w, h in ((300, 300), (301, 1080), (1080, 301), (777, 512)):
        assert O.resize_dst_size(w, h, 256, 256, 2) == S.resize_not_smaller(w, h, 256)


def test_min_max_resize_rule():
    """ROCAL_SCALING_MODE_MIN_MAX of ResizeMirrorNormalize (node_resize_mirror_normalize.cpp:138-160), hand-computed."""
    assert O.resize_dst_size(640, 480, 0, 0, 4, max_w=800, max_h=1333) == (1066, 800)
    assert O.resize_dst_size(1000, 300, 0, 0, 4, max_w=800, max_h=1333) == (1333, 400)      # the longer side hits the maximum
    assert O.resize_dst_size(300, 1000, 0, 0, 4, max_w=800, max_h=1333) == (400, 1333)
    assert O.resize_dst_size(500, 500, 0, 0, 4, max_w=800, max_h=1333) == (800, 800)


def test_crop_rules():
    # fixed-anchor crop (parameter_rocal_crop.cpp:51-61): centre, corners, crop larger than the image
    assert O.crop_fixed(256, 341, 224, 224, 0.5, 0.5) == (16, 58, 224, 224)
    assert O.crop_fixed(256, 341, 224, 224, 0.0, 1.0) == (0, 117, 224, 224)
    assert O.crop_fixed(200, 341, 224, 224, 0.5, 0.5) == (0, 58, 200, 224)
    assert O.crop_fixed(225, 225, 224, 224, 0.5, 0.5) == (0, 0, 224, 224)    # nearbyint(0.5) = 0 (ties to even)
    assert O.crop_fixed(227, 227, 224, 224, 0.5, 0.5) == (2, 2, 224, 224)    # nearbyint(1.5) = 2


def _images(seed, n, hr, wr, content="gradient_noise"):
    rng = S.rng_for(seed)
    return rng, S.make_images(rng, n, hr, wr, content)


def test_pointwise_properties():
    rng, (arena, hs, ws, offs) = _images(30, 5, (9, 40), (7, 60), "noise")
    n = len(hs)
    t = np.zeros(n, dtype=T.POINTWISE_SAMPLE)
    t["src_offset"], t["src_stride"], t["roi_w"], t["roi_h"] = offs, ws * 3, ws, hs
    ident = O.pointwise(arena, t, 60, 40)
    for i in range(n):
        img = arena[int(offs[i]):int(offs[i]) + hs[i] * ws[i] * 3].reshape(hs[i], ws[i], 3)
        assert np.array_equal(ident[i, :hs[i], :ws[i]], img)
        assert (ident[i, hs[i]:] == 0).all() and (ident[i, :, ws[i]:] == 0).all()
    t["flip_h"], t["flip_v"] = 1, 1
    f = O.pointwise(arena, t, 60, 40)
    for i in range(n):
        img = arena[int(offs[i]):int(offs[i]) + hs[i] * ws[i] * 3].reshape(hs[i], ws[i], 3)
        assert np.array_equal(f[i, :hs[i], :ws[i]], img[::-1, ::-1])
    # identity colour parameters leave the image unchanged; brightness follows alpha*x+beta with saturation
    t["flip_h"], t["flip_v"] = 0, 0
    t["alpha"], t["beta"], t["hue"], t["sat"] = 1.0, 0.0, 0.0, 1.0
    assert np.array_equal(O.pointwise(arena, t, 60, 40, T.COLOR_TWIST), ident)
    assert np.array_equal(O.pointwise(arena, t, 60, 40, T.COLOR_BRIGHTNESS), ident)
    t["hue"] = 360.0
    assert np.abs(O.pointwise(arena, t, 60, 40, T.COLOR_TWIST).astype(int) - ident.astype(int)).max() <= 1
    t["alpha"], t["beta"], t["hue"] = 1.9, 20.0, 0.0     # the reference's BrightnessFixed test case (unit_tests.cpp:753-756)
    b = O.pointwise(arena, t, 60, 40, T.COLOR_BRIGHTNESS)
    i = 0
    img = arena[int(offs[i]):int(offs[i]) + hs[i] * ws[i] * 3].reshape(hs[i], ws[i], 3).astype(np.float32)
    exp = np.clip(np.rint(np.float32(1.9) * img + np.float32(20.0)), 0, 255).astype(np.uint8)
    assert np.array_equal(b[i, :hs[i], :ws[i]], exp)
    # a non-zero hue field tilts the brightness offset (colour temperature): R + 30, G, B - 30
    t["alpha"], t["beta"], t["hue"] = 1.0, 0.0, 30.0
    ct = O.pointwise(arena, t, 60, 40, T.COLOR_BRIGHTNESS)[0, :hs[0], :ws[0]].astype(np.int32)
    assert np.array_equal(ct, np.clip(img.astype(np.int32) + np.array([30, 0, -30]), 0, 255))
    # gamma 1 is the identity up to the rounding of powf; gamma 2 squares the normalised value
    t["alpha"], t["hue"] = 1.0, 0.0
    assert np.abs(O.pointwise(arena, t, 60, 40, T.COLOR_GAMMA).astype(int) - ident.astype(int)).max() <= 1
    t["alpha"] = 2.0
    g2 = O.pointwise(arena, t, 60, 40, T.COLOR_GAMMA)[0, :hs[0], :ws[0]].astype(np.float64)
    assert np.abs(g2 - np.rint(img.astype(np.float64) ** 2 / 255.0)).max() <= 1
    # saturation 0 gives grey pixels (all channels equal to the value channel)
    t["alpha"], t["beta"], t["hue"], t["sat"] = 1.0, 0.0, 0.0, 0.0
    g = O.pointwise(arena, t, 60, 40, T.COLOR_TWIST)
    assert np.array_equal(g[0, :hs[0], :ws[0], 0], g[0, :hs[0], :ws[0], 1])
    assert np.array_equal(g[0, :hs[0], :ws[0], 0], img.max(axis=2).astype(np.uint8))


def test_normalize_and_fp16():
    rng, (arena, hs, ws, offs) = _images(31, 3, (20, 20), (30, 30), "noise")
    t = np.zeros(3, dtype=T.POINTWISE_SAMPLE)
    t["src_offset"], t["src_stride"], t["roi_w"], t["roi_h"] = offs, ws * 3, ws, hs
    mul, add = S.normalize_tables()
    f32 = O.pointwise(arena, t, 30, 20, T.COLOR_NONE, T.FP32, T.NCHW, mul, add)
    f16 = O.pointwise(arena, t, 30, 20, T.COLOR_NONE, T.FP16, T.NCHW, mul, add)
    img = arena[:20 * 30 * 3].reshape(20, 30, 3).astype(np.float64)
    ref = (img - np.array(S.MEAN)) / np.array(S.STD)
    assert np.allclose(f32[0].transpose(1, 2, 0), ref, rtol=1e-5, atol=2e-6)
    assert np.array_equal(f16, f32.astype(np.float16))       # round to nearest even
    # identity normalisation reproduces the crop exactly
    one = O.pointwise(arena, t, 30, 20, T.COLOR_NONE, T.FP32, T.NHWC, [1, 1, 1], [0, 0, 0])
    assert np.array_equal(one[0], img.astype(np.float32))


def test_resample_properties():
    rng, (arena, hs, ws, offs) = _images(32, 4, (17, 40), (17, 40))
    n = len(hs)
    t = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
    t["src_offset"], t["src_stride"], t["roi_w"], t["roi_h"] = offs, ws * 3, ws, hs
    t["dst_w"], t["dst_h"], t["crop_w"], t["crop_h"] = ws, hs, ws, hs
    same = O.resample(arena, t, 40, 40, T.UINT8, T.NHWC)
    for i in range(n):
        img = arena[int(offs[i]):int(offs[i]) + hs[i] * ws[i] * 3].reshape(hs[i], ws[i], 3)
        # ratio 1: every tap pair starts on the pixel itself with weight 0 on the neighbour; the last
        # row/column take the clamped tap (both taps at size-2, rocal_hip_kernels.cpp:340-343)
        assert np.array_equal(same[i, :hs[i] - 1, :ws[i] - 1], img[:-1, :-1])
        assert np.array_equal(same[i, :hs[i] - 1, ws[i] - 1], img[:-1, ws[i] - 2])
    # mirror == reversing the unmirrored result; crop == slicing the uncropped result
    t["dst_w"], t["dst_h"] = 64, 48
    t["crop_w"], t["crop_h"] = 64, 48
    full = O.resample(arena, t, 64, 48, T.UINT8, T.NHWC)
    t["mirror"] = 1
    assert np.array_equal(O.resample(arena, t, 64, 48, T.UINT8, T.NHWC), full[:, :, ::-1])
    t["mirror"] = 0
    t["crop_x"], t["crop_y"], t["crop_w"], t["crop_h"] = 5, 7, 30, 20
    assert np.array_equal(O.resample(arena, t, 30, 20, T.UINT8, T.NHWC), full[:, 7:27, 5:35])
    # a constant image stays constant under any resize
    flat = np.full(50 * 60 * 3 + 256, 93, dtype=np.uint8)
    t1 = np.zeros(1, dtype=T.RESAMPLE_SAMPLE)
    t1["src_stride"], t1["roi_w"], t1["roi_h"], t1["dst_w"], t1["dst_h"], t1["crop_w"], t1["crop_h"] = 180, 60, 50, 97, 31, 97, 31
    assert (O.resample(flat, t1, 97, 31, T.UINT8, T.NHWC) == 93).all()
    # 2x downscale of a horizontal ramp: the half-pixel centre convention averages neighbouring pixels
    ramp = np.zeros((4, 8, 3), dtype=np.uint8)
    ramp[:, :, :] = (np.arange(8) * 10)[None, :, None]
    t1["src_stride"], t1["roi_w"], t1["roi_h"], t1["dst_w"], t1["dst_h"], t1["crop_w"], t1["crop_h"] = 24, 8, 4, 4, 2, 4, 2
    o = O.resample(np.concatenate([ramp.reshape(-1), np.zeros(64, np.uint8)]), t1, 4, 2, T.UINT8, T.NHWC)
    assert list(o[0, 0, :3, 0]) == [5, 25, 45]      # (0+10)/2, (20+30)/2, (40+50)/2


def test_warp_properties():
    rng, (arena, hs, ws, offs) = _images(33, 3, (20, 40), (20, 40))
    n = len(hs)
    t = np.zeros(n, dtype=T.WARP_SAMPLE)
    t["src_offset"], t["src_stride"], t["src_w"], t["src_h"] = offs, ws * 3, ws, hs
    t["dst_w"], t["dst_h"] = ws, hs
    t["m"][:] = S.rotate_matrix(0.0)
    o = O.warp_affine(arena, t, 40, 40)
    for i in range(n):
        if hs[i] % 2 == 0 and ws[i] % 2 == 0:
            img = arena[int(offs[i]):int(offs[i]) + hs[i] * ws[i] * 3].reshape(hs[i], ws[i], 3)
            assert np.array_equal(o[i, :hs[i] - 1, :ws[i] - 1], img[:-1, :-1])
    # a shift of the whole image outside the source gives the constant-zero border everywhere
    t["m"][:, 4] = 1000.0
    assert (O.warp_affine(arena, t, 40, 40) == 0).all()
    # 180 degrees on an even-sized image maps pixel (x,y) to (W-x, H-y)
    t["m"][:] = np.array([-1, 0, 0, -1, 0, 0], dtype=np.float32)
    o = O.warp_affine(arena, t, 40, 40)
    for i in range(n):
        if hs[i] % 2 == 0 and ws[i] % 2 == 0:
            img = arena[int(offs[i]):int(offs[i]) + hs[i] * ws[i] * 3].reshape(hs[i], ws[i], 3)
            assert np.array_equal(o[i, 2:hs[i], 2:ws[i]], img[::-1, ::-1][1:hs[i] - 1, 1:ws[i] - 1])


def test_triangular_properties():
    """The triangular filter: identity at ratio 1, two-tap behaviour when up-scaling, and an independent numpy
    statement of the same sums on a small down-scale case."""
    rng = S.rng_for(31)
    arena, hs, ws, offs = S.make_images(rng, 3, (20, 40), (20, 50))
    n = 3
    t = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
    t["src_offset"], t["src_stride"] = offs, ws * 3
    t["roi_w"], t["roi_h"], t["dst_w"], t["dst_h"], t["crop_w"], t["crop_h"] = ws, hs, ws, hs, ws, hs
    out = O.resample(arena, t, 50, 40, T.UINT8, T.NHWC, interpolation=1)
    for i in range(n):
        o, h, w = int(offs[i]), int(hs[i]), int(ws[i])
        assert np.array_equal(out[i, :h, :w], arena[o:o + h * w * 3].reshape(h, w, 3))
    # independent float32 statement, sample 0 down-scaled by 2.5 x 1.6
    o, h, w = int(offs[0]), int(hs[0]), int(ws[0])
    img = arena[o:o + h * w * 3].reshape(h, w, 3)
    dw, dh = int(w / 2.5), int(h / 1.6)
    t1 = t[:1].copy()
    t1["dst_w"], t1["dst_h"], t1["crop_w"], t1["crop_h"] = dw, dh, dw, dh
    got = O.resample(arena, t1, dw, dh, T.UINT8, T.NHWC, interpolation=1)[0]
    f = np.float32

    def axis(src, dst):
        ratio = f(src) / f(dst)
        radius, scale = (ratio, f(1) / ratio) if ratio > 1 else (f(1), f(1))
        return ratio, radius, scale, (ratio - f(1)) * f(0.5) - radius, int(np.ceil(radius * f(2)))

    rw, radw, scw, offw, kw = axis(w, dw)
    rh, radh, sch, offh, kh = axis(h, dh)
    for (x, y) in ((0, 0), (dw - 1, dh - 1), (dw // 2, dh // 3), (1, dh - 2)):
        rawx = f(np.float32(x) * rw + offw)      # the fused multiply-add rounds once; so does float64 -> float32 here
        rawx = f(np.float64(x) * np.float64(rw) + np.float64(offw))
        rawy = f(np.float64(y) * np.float64(rh) + np.float64(offh))
        fx, fy = int(np.ceil(rawx)), int(np.ceil(rawy))
        wx, wy = f(fx) - rawx, f(fy) - rawy
        fx, fy = min(fx, w - 1), min(fy, h - 1)
        acc = np.zeros(3, dtype=np.float64)
        rs = f(0)
        for j in range(kh):
            rc = max(f(0), f(1) - abs(f(f(wy - radh) + f(j)) * sch))
            rs = f(rs + rc)
            cs = f(0)
            for k in range(kw):
                cc = max(f(0), f(1) - abs(f(f(wx - radw) + f(k)) * scw))
                cs = f(cs + cc)
                px = img[min(max(fy + j, 0), h - 1), min(max(fx + k, 0), w - 1)].astype(np.float64)
                acc += px * np.float64(f(cc * rc))
        val = acc / (np.float64(rs) * np.float64(cs))
        # the float64 accumulation differs from the float32 fmaf chain by far less than one grey level
        assert np.all(np.abs(got[y, x].astype(np.float64) - np.floor(np.clip(val, 0, 255))) <= 1), (x, y)


def test_other_filters_properties():
    """Bicubic, lanczos, gaussian, nearest on the generic skeleton: a constant image stays constant (normalised
    weights; truncation may cost one level), nearest up-scaling by 2 repeats every pixel, every filter differs from the
    triangular one on a textured image."""
    rng = S.rng_for(33)
    const = np.full((40, 52, 3), 137, dtype=np.uint8)
    t = np.zeros(1, dtype=T.RESAMPLE_SAMPLE)
    t["src_stride"], t["roi_w"], t["roi_h"] = 52 * 3, 52, 40
    for dst in ((17, 13), (90, 70)):
        t["dst_w"], t["dst_h"], t["crop_w"], t["crop_h"] = dst[0], dst[1], dst[0], dst[1]
        for interp in (2, 3, 4, 5):
            out = O.resample(const.reshape(-1), t, dst[0], dst[1], T.UINT8, T.NHWC, interpolation=interp)
            assert out.min() >= 136 and out.max() <= 137, (interp, dst)
    img = rng.integers(0, 256, (20, 24, 3), dtype=np.uint8)
    t["src_stride"], t["roi_w"], t["roi_h"] = 24 * 3, 24, 20
    t["dst_w"], t["dst_h"], t["crop_w"], t["crop_h"] = 48, 40, 48, 40
    up = O.resample(img.reshape(-1), t, 48, 40, T.UINT8, T.NHWC, interpolation=5)[0]
    assert np.array_equal(up, np.repeat(np.repeat(img, 2, axis=0), 2, axis=1))
    t["dst_w"], t["dst_h"], t["crop_w"], t["crop_h"] = 11, 9, 11, 9
    tri = O.resample(img.reshape(-1), t, 11, 9, T.UINT8, T.NHWC, interpolation=1)
    for interp in (2, 3, 4, 5):
        assert not np.array_equal(tri, O.resample(img.reshape(-1), t, 11, 9, T.UINT8, T.NHWC, interpolation=interp))

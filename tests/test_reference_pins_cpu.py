"""The CPU restatement against reference-owned code that runs here: the reference's own pixel kernels
(rocAL/rocAL_hip/rocal_hip_kernels.cpp compiled for the host, oracle/_ref/libref_hip.so), its crop-window
class and its random-bbox metadata update (oracle/_ref/libref.so). Each pin is checked twice: against the
committed golden vectors (always) and against the live build on larger seeded cases (when the reference tree
is present)."""
import os

import numpy as np
import pytest

from oracle import pyoracle as O
import synthetic as S
from rocal_b200 import tables as T

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _whole_image_table(ws, hs, offs, dws, dhs):
    n = len(ws)
    t = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
    t["src_offset"] = offs
    t["src_stride"] = np.asarray(ws, dtype=np.int64) * 3
    t["roi_w"], t["roi_h"] = ws, hs
    t["dst_w"], t["dst_h"] = dws, dhs
    t["crop_w"], t["crop_h"] = dws, dhs
    return t


def _valid_equal(a, b, dws, dhs):
    bad = 0
    for i in range(len(dws)):
        bad += int(np.count_nonzero(a[i, :dhs[i], :dws[i]] != b[i, :dhs[i], :dws[i]]))
    return bad


def _planes(arena, ws, hs, offs, c):
    pl, po, off = [], [], 0
    for i in range(len(ws)):
        w, h = int(ws[i]), int(hs[i])
        pl.append(arena[int(offs[i]):int(offs[i]) + w * h * 3].reshape(h, w, 3)[:, :, c].reshape(-1).copy())
        po.append(off)
        off += w * h
    return np.concatenate(pl + [np.zeros(16, np.uint8)]), np.array(po, dtype=np.uint64)


# ---- pixel arithmetic ------------------------------------------------------------------------------------

def test_bilinear_resize_matches_hip_kernel_golden():
    """orc_resample (bilinear, whole-image ROI, uint8) == resize_bilinear_pkd_hip_tensor, bit for bit."""
    g = np.load(os.path.join(GOLDEN, "hip_pixels.npz"))
    ws, hs, dws, dhs = g["src_w"], g["src_h"], g["dst_w"], g["dst_h"]
    # the kernel clamps taps to [0, size-2] (rocal_hip_kernels.cpp:340-343), which leaves a one-pixel-wide source
    # out of range; the restatement keeps the bound at 0 there, so such samples are outside the pin
    assert ws.min() >= 2 and hs.min() >= 2
    t = _whole_image_table(ws, hs, g["src_offset"], dws, dhs)
    got = O.resample(g["arena"], t, int(dws.max()), int(dhs.max()), T.UINT8, T.NHWC)
    assert _valid_equal(got, g["bilinear"], dws, dhs) == 0


def test_triangular_resize_matches_hip_kernel_golden():
    """orc_resample (triangular) on each channel == resize_generic_pln1_hip_tensor on that channel's plane."""
    g = np.load(os.path.join(GOLDEN, "hip_pixels.npz"))
    ws, hs, dws, dhs = g["src_w"], g["src_h"], g["dst_w"], g["dst_h"]
    t = _whole_image_table(ws, hs, g["src_offset"], dws, dhs)
    got = O.resample(g["arena"], t, int(dws.max()), int(dhs.max()), T.UINT8, T.NHWC, interpolation=1)
    for c in range(3):
        assert _valid_equal(got[..., c], g["triangular_c%d" % c], dws, dhs) == 0, c


def _convert_with_oracle(img, nchw, fp16, mul, add, rev):
    n, h, w, _ = img.shape
    t = np.zeros(n, dtype=T.POINTWISE_SAMPLE)
    t["src_offset"] = np.arange(n) * h * w * 3
    t["src_stride"] = w * 3
    t["roi_w"], t["roi_h"] = w, h
    return O.pointwise(np.ascontiguousarray(img).reshape(-1), t, w, h, T.COLOR_NONE, T.FP16 if fp16 else T.FP32,
                       T.NCHW if nchw else T.NHWC, list(mul), list(add), reverse_channels=bool(rev))


def test_converters_match_hip_kernels_golden():
    """orc_pointwise (copy + x*mul+add, both layouts, both types, channel reversal) == Hip_CopyInt8To*."""
    g = np.load(os.path.join(GOLDEN, "hip_pixels.npz"))
    img, mul, add = g["convert_src"], g["convert_mul"], g["convert_add"]
    for nchw in (0, 1):
        for fp16 in (0, 1):
            for rev in (0, 1):
                src = img[:, :1] if (fp16 and not nchw) else img
                got = _convert_with_oracle(src, nchw, fp16, mul, add, rev)
                ref = g["convert_nchw%d_fp16%d_rev%d" % (nchw, fp16, rev)]
                bits = np.uint16 if fp16 else np.uint32
                assert np.array_equal(got.view(bits), ref.view(bits)), (nchw, fp16, rev)


def test_pixel_restatement_matches_hip_kernels_live():
    """Larger seeded cases against the live host build of the reference kernels: the geometry of the first two
    benchmark configurations (shorter side to 256), odd widths, up- and down-scales."""
    if O.ref_hip() is None:
        pytest.skip("reference tree not present: oracle/_ref/libref_hip.so cannot be built")
    rng = S.rng_for(0)
    cases = []
    arena, hs, ws, offs = S.make_images(rng, 6, (256, 512), (256, 512))
    cases.append((arena, hs, ws, offs, [S.resize_not_smaller(int(w), int(h), 256) for w, h in zip(ws, hs)]))
    arena, hs, ws, offs = S.make_images(rng, 4, (300, 1080), (300, 1080))
    cases.append((arena, hs, ws, offs, [S.resize_not_smaller(int(w), int(h), 256) for w, h in zip(ws, hs)]))
    arena, hs, ws, offs = S.make_images(rng, 24, (2, 200), (2, 200))
    cases.append((arena, hs, ws, offs, [(int(rng.integers(1, 260)), int(rng.integers(1, 260))) for _ in range(24)]))
    total = 0
    for arena, hs, ws, offs, dst in cases:
        dws = np.array([d[0] for d in dst], dtype=np.uint32)
        dhs = np.array([d[1] for d in dst], dtype=np.uint32)
        t = _whole_image_table(ws, hs, offs, dws, dhs)
        mw, mh = int(dws.max()), int(dhs.max())
        got = O.resample(arena, t, mw, mh, T.UINT8, T.NHWC)
        ref = O.ref_hip_resize_bilinear(arena, ws, hs, ws * 3, offs, dws, dhs)
        assert _valid_equal(got, ref, dws, dhs) == 0
        got = O.resample(arena, t, mw, mh, T.UINT8, T.NHWC, interpolation=1)
        for c in range(3):
            planes, po = _planes(arena, ws, hs, offs, c)
            ref = O.ref_hip_resize_generic(planes, ws, hs, ws, po, dws, dhs)
            assert _valid_equal(got[..., c], ref, dws, dhs) == 0, c
        total += int((dws.astype(np.int64) * dhs).sum())
    assert total > 1_000_000
    img = rng.integers(0, 256, (3, 41, 57, 3), dtype=np.uint8)
    mul, add = S.normalize_tables()
    for nchw in (0, 1):
        for fp16 in (0, 1):
            if fp16 and not nchw:
                continue
            got = _convert_with_oracle(img, nchw, fp16, mul, add, 0)
            ref = O.ref_hip_copy_int8(img, nchw, fp16, mul, add, 0)
            bits = np.uint16 if fp16 else np.uint32
            assert np.array_equal(got.view(bits), ref.view(bits))


# ---- crop windows ------------------------------------------------------------------------------------------

def test_crop_windows_match_golden():
    g = np.load(os.path.join(GOLDEN, "crop_and_boxes.npz"))
    for k in range(9):
        a = g["crop_args_%d" % k]
        mode, cw, ch, f = int(a[0]), int(a[1]), int(a[2]), a[3:7].astype(np.float32)
        win = O.rocal_crop_windows(g["crop_wh_%d" % k], mode, cw, ch, f)
        assert np.array_equal(win, g["crop_windows_%d" % k]), k
        if mode == 0:
            for (w, h), row in zip(g["crop_wh_%d" % k], win):
                assert O.crop_fixed(int(w), int(h), cw, ch, float(f[0]), float(f[1])) == tuple(int(v) for v in row[:4])


def test_crop_windows_match_reference_build():
    if O.ref() is None:
        pytest.skip("reference tree not present")
    rng = np.random.Generator(np.random.PCG64(31))
    for mode in (0, 1, 2):
        for _ in range(10):
            wh = rng.integers(1, 1200, (64, 2))
            cw, ch = int(rng.integers(0, 900)), int(rng.integers(0, 900))
            f = rng.uniform(0, 1, 4).astype(np.float32) if mode != 1 else np.array([rng.integers(0, 1200), rng.integers(0, 1200), 0, 0], np.float32)
            assert np.array_equal(O.rocal_crop_windows(wh, mode, cw, ch, f), O.ref_rocal_crop_windows(wh, mode, cw, ch, f))


# ---- boxes that follow a crop -------------------------------------------------------------------------------

def test_random_bbox_meta_matches_golden():
    g = np.load(os.path.join(GOLDEN, "crop_and_boxes.npz"))
    kept = 0
    for k in range(4):
        b, l, o = O.random_bbox_meta(g["bbox_boxes_%d" % k], g["bbox_labels_%d" % k], g["bbox_offsets_%d" % k],
                                     g["bbox_crops_%d" % k], g["bbox_roi_%d" % k])
        assert np.array_equal(o, g["bbox_out_offsets_%d" % k]), k
        assert np.array_equal(l, g["bbox_out_labels_%d" % k]), k
        assert np.array_equal(b, g["bbox_out_boxes_%d" % k]), k
        kept += int((l > 0).sum())
    assert kept > 20


def test_random_bbox_meta_matches_reference_build():
    if O.ref() is None:
        pytest.skip("reference tree not present")
    rng = np.random.Generator(np.random.PCG64(32))
    for k in range(20):
        n = 16
        counts = rng.integers(0, 14, n)
        tot = int(counts.sum())
        roi = rng.integers(1, 900, (n, 2)).astype(np.uint32)
        ctr, sz = rng.uniform(0, 1, (tot, 2)), rng.uniform(0.0, 0.7, (tot, 2))
        boxes = np.concatenate([np.clip(ctr - sz / 2, 0, 1), np.clip(ctr + sz / 2, 0, 1)], 1).astype(np.float32)
        labels = rng.integers(1, 81, tot).astype(np.int32)
        offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
        crops = np.concatenate([rng.uniform(0, 0.6, (n, 2)), rng.uniform(0.2, 1, (n, 2))], 1).astype(np.float32)
        a = O.random_bbox_meta(boxes, labels, offsets, crops, roi)
        b = O.ref_random_bbox_meta(boxes, labels, offsets, crops, roi)
        for x, y in zip(a, b):
            assert np.array_equal(x, y), k


# ---- random bbox crop windows -----------------------------------------------------------------------------------

def _product_bbox_windows(seed, overlap, boxes, offsets, img_w):
    """The library's own sampler through its host-only entry point (no device is touched)."""
    import ctypes
    from rocal_b200 import _capi as C
    boxes = np.ascontiguousarray(boxes, dtype=np.float32)
    offsets = np.ascontiguousarray(offsets, dtype=np.int32)
    img_w = np.ascontiguousarray(img_w, dtype=np.int32)
    out = np.zeros((len(img_w), 4), dtype=np.float32)
    fp, ip = ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_int)
    rc = C.bbox_crop_windows(int(seed), int(overlap), 0, boxes.ctypes.data_as(fp), offsets.ctypes.data_as(ip), len(img_w),
                             img_w.ctypes.data_as(ip), out.ctypes.data_as(fp))
    assert rc == 0
    return out


def test_bbox_crop_windows_match_golden():
    """RandomBBoxCropReader::get_batch_crop_coords (randombboxcrop_reader.cpp:216-313), recorded from the reference
    build: the numpy restatement and the library's sampler both reproduce every window bit for bit."""
    g = np.load(os.path.join(GOLDEN, "crop_and_boxes.npz"))
    cropped = 0
    for k in range(3):
        seed, overlap = (int(v) for v in g["bboxcrop_args_%d" % k])
        boxes, offsets, img_w, want = (g["bboxcrop_%s_%d" % (name, k)] for name in ("boxes", "offsets", "img_w", "windows"))
        got = O.BBoxCropSampler(seed, bool(overlap)).windows(boxes, offsets, img_w)
        assert np.array_equal(got, want), k
        assert np.array_equal(_product_bbox_windows(seed, overlap, boxes, offsets, img_w), want), k
        cropped += int((want[:, 2] < 1).sum())
        # every window is a legal one: inside the image, left edge on an 8-pixel boundary
        assert np.all(want[:, :2] >= 0) and np.all(want[:, 0] + want[:, 2] <= 1.0001) and np.all(want[:, 1] + want[:, 3] <= 1.0001)
        assert np.all(np.abs(np.rint(want[:, 0] * img_w) % 8) < 1e-3)
    assert cropped > 200


def test_bbox_crop_windows_match_reference_build():
    if O.ref() is None:
        pytest.skip("reference tree not present")
    rng = np.random.Generator(np.random.PCG64(35))
    for k in range(4):
        n = 300
        counts = rng.integers(1, 9, n)
        tot = int(counts.sum())
        ctr, sz = rng.uniform(0.02, 0.98, (tot, 2)), rng.uniform(0.01, 0.8, (tot, 2))
        boxes = np.concatenate([np.clip(ctr - sz / 2, 0, 1), np.clip(ctr + sz / 2, 0, 1)], 1).astype(np.float32)
        offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
        img_w = rng.integers(16, 4000, n).astype(np.int32)
        seed, overlap = int(rng.integers(0, 2 ** 31)), k % 2
        want = O.ref_random_bbox_crop(boxes, offsets, img_w, seed, bool(overlap))
        assert np.array_equal(O.BBoxCropSampler(seed, bool(overlap)).windows(boxes, offsets, img_w), want), k
        assert np.array_equal(_product_bbox_windows(seed, overlap, boxes, offsets, img_w), want), k


def test_normalised_box_transform_agrees_with_the_pinned_rules():
    """The normalised form the library uses (pyoracle.box_transform: what the host pipeline and rb200k_box_transform are
    compared with) against the restatements that are pinned to, or written from, the reference's pixel-space code: the
    centre rule against update_random_bbox_meta_data (pinned), the quarter-area rule against the CropMetaNode
    restatement. Same boxes kept, same order, coordinates equal after the change of units."""
    rng = np.random.Generator(np.random.PCG64(36))
    n = 40
    boxes, labels, offs = S.random_boxes(rng, n, (0, 12), size_range=(0.02, 0.7))
    l, t = rng.uniform(0, 0.5, n), rng.uniform(0, 0.5, n)
    win = np.stack([l, t, l + rng.uniform(0.2, 0.5, n), t + rng.uniform(0.2, 0.5, n)], 1).astype(np.float32)
    # centre rule: the pinned function on a 1 x 1 "decoded size" works on normalised boxes; it shifts, we also divide
    xywh = np.stack([win[:, 0], win[:, 1], win[:, 2] - win[:, 0], win[:, 3] - win[:, 1]], 1).astype(np.float32)
    pb, pl, po = O.random_bbox_meta(boxes, labels, offs, xywh, np.ones((n, 2), np.uint32))
    nb, nl, no = O.box_transform(boxes, labels, offs, win, 1)
    assert np.array_equal(po, no) and np.array_equal(pl, nl)
    rep = np.repeat(xywh[:, 2:], np.diff(po), axis=0)
    assert np.allclose(pb / np.concatenate([rep, rep], 1), nb, atol=2e-6)
    # quarter-area rule: CropMetaNode works in pixels of a W x H image with an integer window
    wh = rng.integers(200, 900, (n, 2))
    pxwin = np.stack([(win[:, 0] * wh[:, 0]).astype(int), (win[:, 1] * wh[:, 1]).astype(int),
                      np.maximum(1, ((win[:, 2] - win[:, 0]) * wh[:, 0]).astype(int)),
                      np.maximum(1, ((win[:, 3] - win[:, 1]) * wh[:, 1]).astype(int))], 1)
    rep = np.repeat(wh.astype(np.float32), np.diff(offs), axis=0)
    px = (boxes * np.concatenate([rep, rep], 1)).astype(np.float32)
    cb, cl, co = O.meta_crop(px, labels, offs, [tuple(int(v) for v in w) for w in pxwin])
    nwin = np.stack([pxwin[:, 0] / wh[:, 0], pxwin[:, 1] / wh[:, 1], (pxwin[:, 0] + pxwin[:, 2]) / wh[:, 0],
                     (pxwin[:, 1] + pxwin[:, 3]) / wh[:, 1]], 1).astype(np.float32)
    nb, nl, no = O.box_transform(boxes, labels, offs, nwin, 0)
    # (a box exactly at the 0.25 threshold could fall on either side in the two units; none does for this seed)
    assert np.array_equal(co, no) and np.array_equal(cl, nl)
    rep = np.repeat(pxwin[:, 2:].astype(np.float32), np.diff(co), axis=0)
    assert np.allclose(cb / np.concatenate([rep, rep], 1), nb, atol=1e-4)
    assert int((nl > 0).sum()) > 40


def test_rotate_meta_restatement_on_hand_cases():
    """RotateMetaNode restated: no rotation keeps the right / bottom edges and, as the node is written, pulls the left /
    top edges to the image corner; a box rotated out of the destination is dropped and the sample gets the whole image."""
    boxes = np.array([[20, 10, 60, 50]], dtype=np.float32)
    b, l, o = O.meta_rotate(boxes, np.array([7], np.int32), np.array([0, 1], np.int32), [(100, 80)], [0.0], 100, 80)
    assert l.tolist() == [7] and np.allclose(b, [[0, 0, 60, 50]], atol=1e-4)
    # a quarter turn about the centre of a 100 x 100 image: x' = y, y' = 100 - x
    b, l, o = O.meta_rotate(boxes, np.array([7], np.int32), np.array([0, 1], np.int32), [(100, 100)], [90.0], 100, 100)
    assert l.tolist() == [7] and np.allclose(b, [[0, 0, 50, 80]], atol=1e-3)
    far = np.array([[0, 0, 4, 4]], dtype=np.float32)
    b, l, o = O.meta_rotate(far, np.array([7], np.int32), np.array([0, 1], np.int32), [(400, 400)], [45.0], 50, 50)
    assert l.tolist() == [0] and b.tolist() == [[0, 0, 50, 50]]


def test_meta_node_restatements_are_consistent():
    """The crop / flip / resize meta-node restatements on hand-checked cases (the node classes themselves need the
    OpenVX graph and are not compiled here)."""
    boxes = np.array([[10, 10, 50, 50], [0, 0, 8, 8], [60, 20, 100, 40]], dtype=np.float32)
    labels = np.array([3, 4, 5], dtype=np.int32)
    offs = np.array([0, 3], dtype=np.int32)
    # window x 20..80, y 0..60: box 0 keeps (30*40)/(40*40) = 0.75 of its area, box 1 nothing, box 2 half
    b, l, o = O.meta_crop(boxes, labels, offs, [(20, 0, 60, 60)])
    assert l.tolist() == [3, 5] and o.tolist() == [0, 2]
    assert b.tolist() == [[0, 10, 30, 50], [40, 20, 60, 40]]
    b, l, o = O.meta_crop(boxes, labels, offs, [(20, 0, 60, 60)], mirror=[1])
    assert b.tolist() == [[30, 10, 60, 50], [0, 20, 20, 40]]
    b, l, o = O.meta_crop(boxes, labels, offs, [(20, 0, 60, 60)], mirror=[0], resize_to=(120, 30))
    assert b.tolist() == [[0, 5, 60, 25], [80, 10, 120, 20]]
    # a window no box reaches with a quarter of its area: the whole window with label 0
    b, l, o = O.meta_crop(boxes, labels, offs, [(52, 42, 8, 8)])
    assert l.tolist() == [0] and b.tolist() == [[0, 0, 8, 8]]
    b, l, o = O.meta_flip(boxes, labels, offs, [(100, 60)], [1], [1])
    assert b.tolist() == [[50, 10, 90, 50], [92, 52, 100, 60], [0, 20, 40, 40]]
    b, l, o = O.meta_resize(boxes, labels, offs, [(100, 60)], [(50, 120)])
    assert b.tolist() == [[5, 20, 25, 100], [0, 0, 4, 16], [30, 40, 50, 80]]
    # SSD crop: centre inside (closed), output normalised to the window
    b, l, o = O.meta_ssd_random_crop(boxes, labels, offs, [(20, 0, 60, 60)])
    assert l.tolist() == [3, 5]
    assert np.allclose(b, [[0, 1 / 6, 0.5, 5 / 6], [2 / 3, 1 / 3, 1, 2 / 3]])

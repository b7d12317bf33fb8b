"""Generates the golden vectors of this folder from reference-owned code (oracle/_ref/libref.so, built from
the reference tree by oracle/build.py). Run in a container that has the reference tree:

    python tests/golden/make_golden.py                  # every file
    python tests/golden/make_golden.py random_crop      # random_crop_windows.npz and random_area_windows.npz only
    python tests/golden/make_golden.py pins             # hip_pixels.npz and crop_and_boxes.npz only

box_encoder.npz   inputs + outputs of BoundingBoxGraph::update_box_encoder_meta_data
                  (rocAL/source/meta_data/bounding_box_graph.cpp:150-220) for offset / plain encodings
box_encoder_degenerate.npz   the same on zero-area / inverted boxes and a degenerate anchor 0, plus the IoU matcher on them
box_iou_matcher.npz          BoundingBoxGraph::update_box_iou_matcher (bounding_box_graph.cpp:222-284), three settings
param_rng.npz     UniformRand<float>, UniformRand<int>, CustomRand<int> draws
                  (rocAL/include/parameters/parameter_random.h) and the std::seed_seq table of
                  ParameterFactory::set_seed (rocAL/source/parameters/parameter_factory.cpp:114-119)
random_crop_windows.npz   RocalRandomCropDecParam windows (rocAL/source/parameters/parameter_random_crop_decoder.cpp)
                  for eight batches of 96 image shapes (ordinary, very wide, very tall, tiny; one or many attempts):
                  the batch seed the reference's std::random_device drew, the shapes, the ranges and the windows
random_area_windows.npz   RocalRandomCropParam::fill_crop_dims windows (rocAL/source/parameters/parameter_random_crop.cpp:48-97,
                  the rule of rocalRandomCrop / rocalCropResize) for fixed parameter values and for the class's default
                  ranges under a ParameterFactory seed (with the index of the first seed-table entry the class took)
hip_pixels.npz    the reference's own pixel kernels (rocAL/rocAL_hip/rocal_hip_kernels.cpp, compiled for the host by
                  oracle/build.py into oracle/_ref/libref_hip.so) on small images: resize_bilinear_pkd_hip_tensor,
                  resize_generic_pln1_hip_tensor (triangular filter, one plane per channel) and the four
                  Hip_CopyInt8To* converters; inputs and outputs are stored
crop_and_boxes.npz   RocalCropParam::fill_crop_dims windows in its three modes (parameter_rocal_crop.cpp:49-85) and
                  BoundingBoxGraph::update_random_bbox_meta_data (bounding_box_graph.cpp:71-118) on normalised and
                  pixel boxes
"""
import ctypes
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import pyoracle as O          # noqa: E402
import synthetic as S     # noqa: E402


def random_crop():
    assert O.ref() is not None, "the reference tree is needed to generate golden vectors"
    rng = np.random.Generator(np.random.PCG64(777))
    out = {}
    settings = [((0.75, 4.0 / 3), (0.08, 1.0), 10), ((0.75, 1.33333), (0.08, 1.0), 100), ((0.8, 1.25), (0.08, 1.0), 10),
                ((0.75, 4.0 / 3), (0.08, 1.0), 1), ((0.5, 2.0), (0.3, 0.6), 3), ((0.75, 4.0 / 3), (0.08, 1.0), 10),
                ((0.75, 4.0 / 3), (0.08, 1.0), 10), ((1.0, 1.0), (0.9, 1.0), 2)]
    for k, (aspect, area, attempts) in enumerate(settings):
        n = 96
        shapes = np.stack([rng.integers(1, 1400, n), rng.integers(1, 1400, n)], axis=1).astype(np.int32)
        if k == 5:
            shapes[:, 0] = rng.integers(1, 16, n)       # very wide
        if k == 6:
            shapes[:, 1] = rng.integers(1, 16, n)       # very tall
        if k == 7:
            shapes = rng.integers(1, 9, (n, 2)).astype(np.int32)
        seed, win = O.ref_random_crop_windows(shapes, aspect, area, attempts)
        out["shapes_%d" % k], out["windows_%d" % k] = shapes, win
        out["params_%d" % k] = np.array([aspect[0], aspect[1], area[0], area[1], attempts], dtype=np.float64)
        out["seed_%d" % k] = np.array([seed], dtype=np.uint32)
    np.savez_compressed(os.path.join(HERE, "random_crop_windows.npz"), **out)
    print("wrote random_crop_windows.npz")


def random_area():
    assert O.ref() is not None, "the reference tree is needed to generate golden vectors"
    rng = np.random.Generator(np.random.PCG64(778))
    out = {}
    for k in range(10):
        n = 64
        wh = np.stack([rng.integers(1, 1200, n), rng.integers(1, 1200, n)], axis=1).astype(np.uint32)
        if k % 5 == 1:
            wh[:, 0] = rng.integers(1, 24, n)
        if k % 5 == 2:
            wh[:, 1] = rng.integers(1, 24, n)
        out["wh_%d" % k] = wh
        if k % 2:
            fixed = np.array([rng.uniform(0.05, 1.3), rng.uniform(0.5, 2.0), rng.uniform(0, 1), rng.uniform(0, 1)], dtype=np.float32)
            win, _ = O.ref_random_area_windows(wh, fixed=fixed)
            out["fixed_%d" % k] = fixed
        else:
            seed = int(rng.integers(0, 2 ** 31))
            win, first = O.ref_random_area_windows(wh, seed=seed)
            out["seed_%d" % k] = np.array([seed, first], dtype=np.int64)
        out["windows_%d" % k] = win
    np.savez_compressed(os.path.join(HERE, "random_area_windows.npz"), **out)
    print("wrote random_area_windows.npz")


def hip_case_images(rng, n, lo, hi):
    """n small interleaved RGB images packed one after another: (arena, widths, heights, strides, offsets)."""
    ws = rng.integers(lo, hi + 1, n).astype(np.uint32)
    hs = rng.integers(lo, hi + 1, n).astype(np.uint32)
    offs = np.zeros(n, dtype=np.uint64)
    offs[1:] = np.cumsum(ws.astype(np.uint64) * hs * 3)[:-1]
    arena = rng.integers(0, 256, int((ws.astype(np.int64) * hs * 3).sum()) + 16, dtype=np.uint8)
    # half of the images smooth (a ramp plus a little noise): interpolated values then sit near .5 boundaries
    for i in range(0, n, 2):
        w, h = int(ws[i]), int(hs[i])
        ramp = (np.add.outer(np.arange(h) * 3, np.arange(w) * 2)[:, :, None] + np.array([0, 40, 90])) % 256
        img = np.clip(ramp + rng.integers(-2, 3, (h, w, 3)), 0, 255).astype(np.uint8)
        arena[int(offs[i]):int(offs[i]) + w * h * 3] = img.reshape(-1)
    return arena, ws, hs, ws * 3, offs


def planes_of(arena, ws, hs, offs, c):
    """Channel c of every image as single-channel planes packed one after another."""
    pl, po, off = [], [], 0
    for i in range(len(ws)):
        w, h = int(ws[i]), int(hs[i])
        img = arena[int(offs[i]):int(offs[i]) + w * h * 3].reshape(h, w, 3)[:, :, c]
        pl.append(img.reshape(-1).copy())
        po.append(off)
        off += w * h
    return np.concatenate(pl + [np.zeros(16, np.uint8)]), np.array(po, dtype=np.uint64)


def hip_pixels():
    assert O.ref_hip() is not None, "the reference tree is needed to generate golden vectors"
    rng = np.random.Generator(np.random.PCG64(779))
    n = 10
    arena, ws, hs, ss, offs = hip_case_images(rng, n, 2, 36)
    dws = rng.integers(1, 44, n).astype(np.uint32)
    dhs = rng.integers(1, 44, n).astype(np.uint32)
    dws[0], dhs[0] = ws[0], hs[0]                  # identity
    dws[1], dhs[1] = ws[1] * 2, hs[1] * 2 + 1      # up-scale
    out = {"arena": arena, "src_w": ws, "src_h": hs, "src_offset": offs, "dst_w": dws, "dst_h": dhs}
    out["bilinear"] = O.ref_hip_resize_bilinear(arena, ws, hs, ss, offs, dws, dhs)
    for c in range(3):
        planes, po = planes_of(arena, ws, hs, offs, c)
        out["triangular_c%d" % c] = O.ref_hip_resize_generic(planes, ws, hs, ws, po, dws, dhs)
    img = rng.integers(0, 256, (2, 9, 13, 3), dtype=np.uint8)
    mul, add = S.normalize_tables()
    out["convert_src"], out["convert_mul"], out["convert_add"] = img, np.array(mul, np.float32), np.array(add, np.float32)
    for nchw in (0, 1):
        for fp16 in (0, 1):
            for rev in (0, 1):
                # the half-precision NHWC converter indexes rows by y*W + x*3 (rocal_hip_kernels.cpp:110), which only
                # addresses a one-row image correctly: that variant is recorded on the first row of the batch
                src = img[:, :1] if (fp16 and not nchw) else img
                out["convert_nchw%d_fp16%d_rev%d" % (nchw, fp16, rev)] = O.ref_hip_copy_int8(src, nchw, fp16, mul, add, rev)
    np.savez_compressed(os.path.join(HERE, "hip_pixels.npz"), **out)
    print("wrote hip_pixels.npz")


def crop_and_boxes():
    assert O.ref() is not None, "the reference tree is needed to generate golden vectors"
    rng = np.random.Generator(np.random.PCG64(780))
    out = {}
    for k in range(9):
        mode = k % 3
        wh = rng.integers(1, 900, (48, 2)).astype(np.uint32)
        cw, ch = int(rng.integers(0, 700)), int(rng.integers(0, 700))
        if k == 0:
            cw = ch = 224
        f = rng.uniform(0, 1, 4).astype(np.float32) if mode != 1 else np.array([rng.integers(0, 900), rng.integers(0, 900), 0, 0], np.float32)
        out["crop_wh_%d" % k], out["crop_args_%d" % k] = wh, np.array([mode, cw, ch, *f], dtype=np.float64)
        out["crop_windows_%d" % k] = O.ref_rocal_crop_windows(wh, mode, cw, ch, f)
    for k in range(4):
        n = 12
        counts = rng.integers(0, 10, n)
        tot = int(counts.sum())
        roi = rng.integers(50, 900, (n, 2)).astype(np.uint32)
        ctr, sz = rng.uniform(0, 1, (tot, 2)), rng.uniform(0.02, 0.6, (tot, 2))
        boxes = np.concatenate([np.clip(ctr - sz / 2, 0, 1), np.clip(ctr + sz / 2, 0, 1)], 1).astype(np.float32)
        if k % 2:
            rep = np.repeat(roi, counts, axis=0).astype(np.float32)
            boxes = (boxes * np.concatenate([rep, rep], 1)).astype(np.float32)
        labels = rng.integers(1, 81, tot).astype(np.int32)
        offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
        crops = np.concatenate([rng.uniform(0, 0.5, (n, 2)), rng.uniform(0.3, 1, (n, 2))], 1).astype(np.float32)
        if k < 2:
            crops[:, 2:] = 1.0
        ob, ol, oo = O.ref_random_bbox_meta(boxes, labels, offsets, crops, roi)
        for name, v in (("boxes", boxes), ("labels", labels), ("offsets", offsets), ("crops", crops), ("roi", roi),
                        ("out_boxes", ob), ("out_labels", ol), ("out_offsets", oo)):
            out["bbox_%s_%d" % (name, k)] = v
    # RandomBBoxCropReader::get_batch_crop_coords with its 128 generators re-seeded (see ref_bbox_crop_driver.cpp):
    # 160 samples each, so the generators wrap around once; case 2 has samples whose boxes are all tiny (many rejections)
    for k, (seed, overlap) in enumerate(((7, 1), (1234, 0), (99, 1))):
        n = 160
        counts = rng.integers(1, 7, n)
        tot = int(counts.sum())
        ctr = rng.uniform(0.05, 0.95, (tot, 2))
        sz = rng.uniform(0.02, 0.7 if k < 2 else 0.1, (tot, 2))
        boxes = np.concatenate([np.clip(ctr - sz / 2, 0, 1), np.clip(ctr + sz / 2, 0, 1)], 1).astype(np.float32)
        offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
        img_w = rng.integers(64, 1400, n).astype(np.int32)
        win = O.ref_random_bbox_crop(boxes, offsets, img_w, seed, bool(overlap))
        for name, v in (("boxes", boxes), ("offsets", offsets), ("img_w", img_w), ("args", np.array([seed, overlap], np.int64)),
                        ("windows", win)):
            out["bboxcrop_%s_%d" % (name, k)] = v
    np.savez_compressed(os.path.join(HERE, "crop_and_boxes.npz"), **out)
    print("wrote crop_and_boxes.npz")


def main():
    ref = O.ref()
    assert ref is not None, "the reference tree is needed to generate golden vectors"
    rng = np.random.Generator(np.random.PCG64(4242))
    anchors = S.ssd300_anchors()[::9][:960].copy()
    counts = [1, 2, 7, 33, 50, 3, 12, 1]
    per = []
    for c in counts:
        b, _, _ = S.random_boxes(rng, 1, (c, c))
        if c > 2:
            b[c // 2] = b[0]                                   # tie between boxes
            b[-1] = anchors[int(rng.integers(0, len(anchors)))]   # IoU 1 with an anchor
        per.append(b)
    boxes = np.ascontiguousarray(np.concatenate(per))
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    labels = rng.integers(1, 81, len(boxes)).astype(np.int32)
    out = {"anchors": anchors, "boxes": boxes, "labels": labels, "offsets": offsets}
    cases = [("offset", 0.5, (0, 0, 0, 0), (0.1, 0.1, 0.2, 0.2), True, 1.0),
             ("plain", 0.5, (0, 0, 0, 0), (1, 1, 1, 1), False, 1.0),
             ("scaled", 0.4, (0.05, -0.05, 0.1, 0.0), (0.1, 0.1, 0.2, 0.2), True, 2.0)]
    for name, crit, means, stds, offset, scale in cases:
        eb, el = O.ref_box_encode(boxes, labels, offsets, anchors, crit, means, stds, offset, scale)
        out[name + "_boxes"], out[name + "_labels"] = eb, el
        out[name + "_args"] = np.array([crit, *means, *stds, float(offset), scale], dtype=np.float64)
    np.savez_compressed(os.path.join(HERE, "box_encoder.npz"), **out)

    # Degenerate geometry: zero-area and inverted boxes, a degenerate anchor 0 (0/0 IoUs, negative IoUs).
    # Every sample has at least one box: the reference indexes the first IoU row of a sample unconditionally.
    rng = np.random.Generator(np.random.PCG64(4243))
    anchors = S.ssd300_anchors()[::5][:1500].copy()
    anchors[0] = (0.0, 0.0, 0.0, 0.0)
    counts = [4, 6, 1, 3]
    boxes, _, _ = S.random_boxes(rng, 1, (sum(counts), sum(counts)))
    boxes[0] = (0.3, 0.3, 0.3, 0.3)
    boxes[1] = (0.6, 0.6, 0.2, 0.2)
    boxes[4] = (0.0, 0.0, 0.0, 0.0)
    boxes[10] = (0.5, 0.2, 0.5, 0.9)
    boxes[11] = boxes[12] = (0.25, 0.25, 0.25, 0.25)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    labels = rng.integers(1, 81, len(boxes)).astype(np.int32)
    out = {"anchors": anchors, "boxes": boxes, "labels": labels, "offsets": offsets}
    for name, offset in (("offset", True), ("plain", False)):
        eb, el = O.ref_box_encode(boxes, labels, offsets, anchors, 0.5, (0, 0, 0, 0), (0.1, 0.1, 0.2, 0.2), offset, 1.0)
        out[name + "_boxes"], out[name + "_labels"] = eb, el
    for name, allow in (("match_lq", True), ("match_plain", False)):
        out[name] = O.ref_box_iou_match(boxes, offsets, anchors, 0.5, 0.4, allow)
    np.savez_compressed(os.path.join(HERE, "box_encoder_degenerate.npz"), **out)

    # Box IoU matcher on ordinary boxes (BoundingBoxGraph::update_box_iou_matcher)
    rng = np.random.Generator(np.random.PCG64(4244))
    anchors = S.ssd300_anchors()[::3][:2500].copy()
    boxes, _, offsets = S.random_boxes(rng, 6, (1, 40))
    boxes[1] = boxes[0]
    out = {"anchors": anchors, "boxes": boxes, "offsets": offsets}
    for name, hi, lo, allow in (("lq_05_04", 0.5, 0.4, True), ("plain_05_04", 0.5, 0.4, False), ("lq_07_03", 0.7, 0.3, True)):
        out[name] = O.ref_box_iou_match(boxes, offsets, anchors, hi, lo, allow)
    np.savez_compressed(os.path.join(HERE, "box_iou_matcher.npz"), **out)

    rngs = {}
    f = np.zeros(3 * 16, dtype=np.float32)
    ref.ref_uniform_rand_float(ctypes.c_uint(123), ctypes.c_float(0.6), ctypes.c_float(1.4), ctypes.c_uint(16), ctypes.c_uint(3),
                               f.ctypes.data_as(ctypes.c_void_p))
    rngs["uniform_float_seed123_0.6_1.4_b16x3"] = f
    i = np.zeros(3 * 16, dtype=np.int32)
    ref.ref_uniform_rand_int(ctypes.c_uint(77), ctypes.c_int(0), ctypes.c_int(10), ctypes.c_uint(16), ctypes.c_uint(3),
                             i.ctypes.data_as(ctypes.c_void_p))
    rngs["uniform_int_seed77_0_10_b16x3"] = i
    vals = np.array([0, 1], dtype=np.int32)
    fr = np.array([0.5, 0.5])
    c = np.zeros(3 * 16, dtype=np.int32)
    ref.ref_custom_rand_int(ctypes.c_uint(9), vals.ctypes.data_as(ctypes.c_void_p), fr.ctypes.data_as(ctypes.c_void_p),
                            ctypes.c_uint(2), ctypes.c_uint(16), ctypes.c_uint(3), c.ctypes.data_as(ctypes.c_void_p))
    rngs["custom_int_seed9_coin_b16x3"] = c
    for seed in (0, 1, 1234):
        t = np.zeros(1024, dtype=np.int64)
        ref.ref_seed_sequence(ctypes.c_uint(seed), ctypes.c_uint(1024), t.ctypes.data_as(ctypes.c_void_p))
        rngs["seed_seq_%d" % seed] = t
    np.savez_compressed(os.path.join(HERE, "param_rng.npz"), **rngs)
    print("wrote box_encoder.npz, box_encoder_degenerate.npz, box_iou_matcher.npz, param_rng.npz")


if __name__ == "__main__":
    if sys.argv[1:] == ["random_crop"]:
        random_crop()
        random_area()
    elif sys.argv[1:] == ["pins"]:
        hip_pixels()
        crop_and_boxes()
    else:
        main()
        random_crop()
        random_area()
        hip_pixels()
        crop_and_boxes()

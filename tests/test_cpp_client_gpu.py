"""A C++ program written against include/rocal_api.h with the reference's call sequence
(tests/harness/rocal_cpp_client.cpp) is compiled with g++, linked with librocal_b200.so and run on the GPU;
what it wrote is checked against the oracle. This is the drop-in boundary exercised from real C++ code:
std::vector arguments, default arguments, rocalTensor virtual calls, the slot feed contract, metadata getters."""
import os
import struct
import subprocess

import numpy as np
import pytest

from oracle import pyoracle as O
import synthetic as S
from rocal_b200 import tables as T

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_client(cuda, tmp_path):
    lib_dir = os.path.join(ROOT, "rocal_b200")
    exe = str(tmp_path / "client")
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "harness", "rocal_cpp_client.cpp"), "-L", lib_dir, "-lrocal_b200",
                    "-Wl,-rpath," + lib_dir, "-o", exe], check=True)
    rng = S.rng_for(25)
    n = 6
    arena, hs, ws, offs = S.make_images(rng, n, (300, 520), (300, 520))
    boxes, labels, boffs = S.random_boxes(rng, n, (1, 12))
    anchors = S.ssd300_anchors()
    counts = np.diff(boffs).astype(np.int32)
    with open(tmp_path / "in.bin", "wb") as f:
        f.write(struct.pack("<i", n))
        for i in range(n):
            f.write(struct.pack("<ii", int(hs[i]), int(ws[i])))
        for i in range(n):
            f.write(arena[int(offs[i]):int(offs[i]) + int(hs[i]) * int(ws[i]) * 3].tobytes())
        f.write(struct.pack("<i", len(labels)))
        f.write(counts.tobytes())
        f.write(np.ascontiguousarray(boxes, dtype=np.float32).tobytes())
        f.write(np.ascontiguousarray(labels, dtype=np.int32).tobytes())
        f.write(struct.pack("<i", len(anchors)))
        f.write(np.ascontiguousarray(anchors, dtype=np.float32).tobytes())
    # a folder of JPEG files for graph 4: two classes, five files of known sizes
    cv2 = pytest.importorskip("cv2")
    jpeg_sizes = {}
    for k, (cls, (jh, jw)) in enumerate([("ant", (120, 200)), ("ant", (300, 150)), ("bee", (90, 90)), ("bee", (240, 320)), ("bee", (64, 400))]):
        (tmp_path / "jpeg" / cls).mkdir(parents=True, exist_ok=True)
        pic = rng.integers(0, 256, (jh, jw, 3), dtype=np.uint8)
        name = "p%d.jpg" % k
        assert cv2.imwrite(str(tmp_path / "jpeg" / cls / name), pic)
        jpeg_sizes[name] = (jw, jh, 0 if cls == "ant" else 1)
    # a COCO annotation file over two of those files for graph 5: one box each, a tenth of the image in from every side
    import json
    coco = {"images": [], "annotations": [], "categories": [{"id": 3}]}
    for k, rel in enumerate(["ant/p0.jpg", "bee/p3.jpg"]):
        jw, jh, _ = jpeg_sizes[rel.split("/")[1]]
        coco["images"].append({"id": 50 + k, "file_name": rel, "width": jw, "height": jh})
        coco["annotations"].append({"id": k, "image_id": 50 + k, "category_id": 3, "iscrowd": 0,
                                    "bbox": [jw * 0.1, jh * 0.1, jw * 0.8, jh * 0.8]})
    (tmp_path / "coco.json").write_text(json.dumps(coco))
    r = subprocess.run([exe, str(tmp_path / "in.bin"), str(tmp_path / "out.bin"), str(tmp_path / "jpeg"), str(tmp_path / "coco.json")],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip() == "ok", r.stderr[-2000:]
    raw = np.fromfile(tmp_path / "out.bin", dtype=np.uint8)
    pos = 0

    def take(dtype, count):
        nonlocal pos
        a = raw[pos:pos + count * np.dtype(dtype).itemsize].view(dtype)
        pos += count * np.dtype(dtype).itemsize
        return a

    mul, add = S.normalize_tables()
    # graph 1
    got1 = take(np.float32, n * 3 * 224 * 224).reshape(n, 3, 224, 224)
    t = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
    for i in range(n):
        dw, dh = O.resize_dst_size(int(ws[i]), int(hs[i]), 256, 256, 2, cap_w=1536, cap_h=1536)
        x1, y1, cw, ch = O.crop_fixed(dw, dh, 224, 224, 0.5, 0.5)
        t[i]["src_offset"], t[i]["src_stride"] = offs[i], ws[i] * 3
        t[i]["roi_w"], t[i]["roi_h"], t[i]["dst_w"], t[i]["dst_h"] = ws[i], hs[i], dw, dh
        t[i]["crop_x"], t[i]["crop_y"], t[i]["crop_w"], t[i]["crop_h"] = x1, y1, cw, ch
    assert np.array_equal(got1, O.resample(arena, t, 224, 224, T.FP32, T.NCHW, mul, add))
    # graph 2
    got2 = take(np.float32, n * 3 * 300 * 300).reshape(n, 3, 300, 300)
    win = take(np.uint32, n * 4).reshape(n, 4).astype(np.int64)
    t2 = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
    t2["src_offset"], t2["src_stride"] = offs, ws * 3
    t2["roi_x"], t2["roi_y"], t2["roi_w"], t2["roi_h"] = win[:, 0], win[:, 1], win[:, 2], win[:, 3]
    t2["dst_w"], t2["dst_h"], t2["crop_w"], t2["crop_h"] = 300, 300, 300, 300
    assert np.array_equal(got2, O.resample(arena, t2, 300, 300, T.FP32, T.NCHW, mul, add))
    total = int(take(np.int32, 1)[0])
    b2, l2, c2 = [], [], []
    for i in range(n):
        c = int(take(np.int32, 1)[0])
        b2.append(take(np.float32, c * 4).reshape(c, 4))
        l2.append(take(np.int32, c))
        c2.append(c)
    assert sum(c2) == total and min(c2) >= 1
    b2, l2 = np.concatenate(b2), np.concatenate(l2)
    assert b2.min() >= 0.0 and b2.max() <= 1.0
    o2 = np.concatenate([[0], np.cumsum(c2)]).astype(np.int32)
    eb, el = O.box_encode(b2, l2, o2, anchors, 0.5, (0, 0, 0, 0), (0.1, 0.1, 0.2, 0.2), True, 1.0)
    gb = take(np.float32, n * len(anchors) * 4).reshape(n, len(anchors), 4)
    gl = take(np.int32, n * len(anchors)).reshape(n, len(anchors))
    assert np.array_equal(gl, el)
    assert np.allclose(gb, eb, rtol=1e-5, atol=1e-6)
    # graph 3: CropResizeFixed, ROIResize(triangular), RandomCrop(fixed parameters), Copy
    wh = np.stack([ws, hs], axis=1)
    win = O.random_area_windows(wh, fixed=(0.5, 1.25, 0.25, 0.75)).astype(np.int64)

    def stretched(wn, w, h, interpolation=0):
        tab = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
        tab["src_offset"], tab["src_stride"] = offs, ws * 3
        tab["roi_x"], tab["roi_y"], tab["roi_w"], tab["roi_h"] = wn[:, 0], wn[:, 1], wn[:, 2], wn[:, 3]
        tab["dst_w"], tab["dst_h"], tab["crop_w"], tab["crop_h"] = w, h, w, h
        return O.resample(arena, tab, w, h, T.UINT8, T.NHWC, interpolation=interpolation)

    outs = []
    for k in range(4):
        oh, ow = [int(v) for v in take(np.int32, 2)]
        outs.append((take(np.uint8, n * oh * ow * 3).reshape(n, oh, ow, 3), take(np.uint32, n * 4).reshape(n, 4)))
    sizes = take(np.int32, n * 2).reshape(n, 2)
    # graph 4: rocalFusedJpegCropSingleShard on the folder, batch 2, LAST_BATCH_PARTIAL with repeated padding
    assert int(take(np.int32, 1)[0]) == 6                         # 5 files padded to 3 batches of 2
    seen = []
    for b in range(3):
        labels4 = take(np.int32, 2)
        sizes4 = take(np.int32, 4).reshape(2, 2)
        lens4 = take(np.int32, 2)
        total4 = int(take(np.uint32, 1)[0])
        names_raw = bytes(take(np.uint8, total4)).decode()
        names4 = [names_raw[:lens4[0]], names_raw[lens4[0]:lens4[0] + lens4[1]]]
        win4 = take(np.uint32, 8).reshape(2, 4)
        seed4 = int(take(np.uint32, 1)[0])
        padded4 = int(take(np.int32, 1)[0])
        assert total4 == lens4.sum() and padded4 == (1 if b == 2 else 0)
        for i, nm in enumerate(names4):
            jw, jh, lab = jpeg_sizes[nm]
            assert labels4[i] == lab and sizes4[i].tolist() == [jw, jh]
        shapes = np.array([[jpeg_sizes[nm][1], jpeg_sizes[nm][0]] for nm in names4])
        assert np.array_equal(win4, O.random_crop_windows(seed4, shapes, (0.75, 1.33333), (0.08, 1.0), 100))
        seen += names4
    assert seen == ["p0.jpg", "p1.jpg", "p2.jpg", "p3.jpg", "p4.jpg", "p4.jpg"]
    assert int(take(np.int32, 1)[0]) == 3
    # graph 5: rocalJpegCOCOFileSourcePartialSingleShard - ids and sizes of the whole images, the sampler's windows,
    # boxes of the whole image
    ids5, sizes5 = take(np.int32, 2), take(np.int32, 4).reshape(2, 2)
    win5, seed5 = take(np.uint32, 8).reshape(2, 4), int(take(np.uint32, 1)[0])
    boxes5 = take(np.float32, 8).reshape(2, 4)
    assert ids5.tolist() == [50, 51] and sizes5.tolist() == [[200, 120], [320, 240]]
    assert np.array_equal(win5, O.random_crop_windows(seed5, np.array([[120, 200], [240, 320]]), (0.5, 2.0), (0.3, 0.8), 25))
    assert np.allclose(boxes5, [[0.1, 0.1, 0.9, 0.9]] * 2, atol=1e-5)
    assert pos == len(raw)
    assert np.array_equal(outs[0][0], stretched(win, 120, 80)) and outs[0][1][:, 2:].tolist() == [[120, 80]] * n
    fixed_roi = np.tile(np.array([[20, 30, 150, 100]], dtype=np.int64), (n, 1))
    assert np.array_equal(outs[1][0], stretched(fixed_roi, 64, 48, 1))
    for i in range(n):
        ih, iw, o = int(hs[i]), int(ws[i]), int(offs[i])
        im = arena[o:o + ih * iw * 3].reshape(ih, iw, 3)
        x, y, w, h = [int(v) for v in win[i]]
        assert np.array_equal(outs[2][0][i, :h, :w], im[y:y + h, x:x + w]) and outs[2][1][i, 2:].tolist() == [w, h]
        assert np.array_equal(outs[3][0][i, :ih, :iw], im) and outs[3][1][i, 2:].tolist() == [iw, ih]
    assert sizes.tolist() == wh.tolist()


def _pointwise_table(hs, ws, offs, windows=None, flip_h=0, alpha=1.0, beta=0.0, hue=0.0, sat=1.0):
    n = len(hs)
    t = np.zeros(n, dtype=T.POINTWISE_SAMPLE)
    t["src_offset"], t["src_stride"] = offs, ws * 3
    if windows is None:
        t["roi_w"], t["roi_h"] = ws, hs
    else:
        t["roi_x"], t["roi_y"], t["roi_w"], t["roi_h"] = windows[:, 0], windows[:, 1], windows[:, 2], windows[:, 3]
    t["flip_h"] = flip_h
    t["alpha"], t["beta"], t["hue"], t["sat"] = alpha, beta, hue, sat
    return t


def test_cpp_ops_client(cuda, tmp_path):
    """The fixed-parameter operator calls of the reference's unit tests (rocalResizeCropMirrorFixed 400x400 from a
    200x200 crop, rocalContrastFixed 30/80, rocalHueFixed 150, rocalSaturationFixed 0.3, rocalCropFixed /
    rocalCropCenterFixed 224, rocalBrightnessFixed 1.9/20, rocalColorTwistFixed, rocalFlipFixed) from C++, every output
    bit-equal to the oracle on tables built here; and boxes behind a mirrored rocalCropMirrorNormalize against the
    restatement of the reference's meta node."""
    lib_dir = os.path.join(ROOT, "rocal_b200")
    exe = str(tmp_path / "ops_client")
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "harness", "rocal_ops_client.cpp"), "-L", lib_dir, "-lrocal_b200",
                    "-Wl,-rpath," + lib_dir, "-o", exe], check=True)
    rng = S.rng_for(26)
    n = 5
    arena, hs, ws, offs = S.make_images(rng, n, (180, 420), (190, 460))
    assert hs.min() < 224 < hs.max()                     # some images are smaller than the 224 crop
    boxes, labels, boffs = S.random_boxes(rng, n, (1, 14))
    counts = np.diff(boffs).astype(np.int32)
    with open(tmp_path / "in.bin", "wb") as f:
        f.write(struct.pack("<i", n))
        for i in range(n):
            f.write(struct.pack("<ii", int(hs[i]), int(ws[i])))
        for i in range(n):
            f.write(_image(arena, offs, i, hs, ws).tobytes())
        f.write(struct.pack("<i", len(labels)))
        f.write(counts.tobytes())
        f.write(np.ascontiguousarray(boxes, dtype=np.float32).tobytes())
        f.write(np.ascontiguousarray(labels, dtype=np.int32).tobytes())
    r = subprocess.run([exe, str(tmp_path / "in.bin"), str(tmp_path / "out.bin")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip() == "ok", r.stderr[-2000:]
    # the oracle reads the same tightly packed images the client was given
    packed = np.concatenate([_image(arena, offs, i, hs, ws).reshape(-1) for i in range(n)] + [np.zeros(64, np.uint8)])
    poffs = np.concatenate([[0], np.cumsum(hs.astype(np.int64) * ws * 3)[:-1]]).astype(np.uint64)
    raw = np.fromfile(tmp_path / "out.bin", dtype=np.uint8)
    pos = 0

    def take(dtype, count):
        nonlocal pos
        a = raw[pos:pos + count * np.dtype(dtype).itemsize].view(dtype)
        pos += count * np.dtype(dtype).itemsize
        return a

    outs = []
    for k in range(9):
        oh, ow = [int(v) for v in take(np.int32, 2)]
        outs.append((take(np.uint8, n * oh * ow * 3).reshape(n, oh, ow, 3), take(np.uint32, n * 4).reshape(n, 4)))
    wh = np.stack([ws, hs], axis=1)
    max_w, max_h = int(ws.max()), int(hs.max())

    # 0: ResizeCropMirrorFixed: the 200 x 200 corner (clipped to the image) stretched to 400 x 400, mirrored
    win = O.rocal_crop_windows(wh, 1, 200, 200, (0, 0)).astype(np.int64)
    tab = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
    tab["src_offset"], tab["src_stride"] = poffs, ws * 3
    tab["roi_x"], tab["roi_y"] = win[:, 0], win[:, 1]
    tab["roi_w"], tab["roi_h"] = win[:, 4] - win[:, 0], win[:, 5] - win[:, 1]
    tab["dst_w"], tab["dst_h"], tab["crop_w"], tab["crop_h"], tab["mirror"] = 400, 400, 400, 400, 1
    assert outs[0][0].shape[1:3] == (400, 400)
    assert np.array_equal(outs[0][0], O.resample(packed, tab, 400, 400, T.UINT8, T.NHWC))
    assert outs[0][1][:, 2:].tolist() == [[400, 400]] * n

    def colour(k, op, **kw):
        exp = O.pointwise(packed, _pointwise_table(hs, ws, poffs, **kw), max_w, max_h, op)
        assert outs[k][0].shape[1:3] == (max_h, max_w), k
        for i in range(n):
            assert np.array_equal(outs[k][0][i, :hs[i], :ws[i]], exp[i, :hs[i], :ws[i]]), (k, i)
        assert outs[k][1][:, 2:].tolist() == wh.tolist(), k

    colour(1, T.COLOR_CONTRAST, alpha=30.0, beta=80.0)
    colour(2, T.COLOR_TWIST, hue=150.0)
    colour(3, T.COLOR_TWIST, sat=0.3)
    colour(6, T.COLOR_BRIGHTNESS, alpha=1.90, beta=20.0)
    colour(7, T.COLOR_TWIST, alpha=0.2, beta=10.0, hue=100.0, sat=0.25)
    colour(8, T.COLOR_NONE, flip_h=1)
    # 4 / 5: CropFixed at the corner, CropCenterFixed: pure indexing
    for k, win in ((4, O.rocal_crop_windows(wh, 1, 224, 224, (0, 0))), (5, O.rocal_crop_windows(wh, 0, 224, 224, (0.5, 0.5)))):
        win = win.astype(np.int64)
        assert outs[k][0].shape[1:3] == (224, 224)
        for i in range(n):
            x, y = int(win[i, 0]), int(win[i, 1])
            w, h = int(win[i, 4]) - x, int(win[i, 5]) - y
            im = _image(arena, offs, i, hs, ws)
            assert np.array_equal(outs[k][0][i, :h, :w], im[y:y + h, x:x + w]), (k, i)
            assert outs[k][1][i].tolist() == [0, 0, w, h], (k, i)

    # graph 2: boxes behind CropMirrorNormalize(120 x 160 window, anchors 0.25 / 0.75, mirror)
    win2 = take(np.uint32, n * 4).reshape(n, 4).astype(np.int64)
    exp_win = O.rocal_crop_windows(wh, 0, 160, 120, (0.25, 0.75)).astype(np.int64)
    assert np.array_equal(win2, np.stack([exp_win[:, 0], exp_win[:, 1], exp_win[:, 4] - exp_win[:, 0], exp_win[:, 5] - exp_win[:, 1]], 1))
    got_b, got_l, got_c = [], [], []
    for i in range(n):
        c = int(take(np.int32, 1)[0])
        got_b.append(take(np.float32, c * 4).reshape(c, 4))
        got_l.append(take(np.int32, c))
        got_c.append(c)
    assert pos == len(raw)
    _check_boxes_after_crop(boxes, labels, boffs, wh, win2, [1] * n, got_b, got_l)


def _image(arena, offs, i, hs, ws):
    o, h, w = int(offs[i]), int(hs[i]), int(ws[i])
    return arena[o:o + h * w * 3].reshape(h, w, 3)


def _check_boxes_after_crop(boxes, labels, boffs, wh, windows, mirror, got_b, got_l):
    """Boxes read back from the pipeline (normalized to the window) against the restatement of the reference's
    Crop / CropMirrorNormalize meta node run on the same boxes in pixels (meta_node_crop_mirror_normalize.cpp:53-90)."""
    n = len(wh)
    rep = np.repeat(wh, np.diff(boffs), axis=0).astype(np.float32)
    px = (np.asarray(boxes, dtype=np.float32) * np.concatenate([rep, rep], 1)).astype(np.float32)
    eb, el, eo = O.meta_crop(px, labels, boffs, windows, mirror=mirror)
    kept = 0
    for i in range(n):
        e = eb[eo[i]:eo[i + 1]] / np.array([windows[i][2], windows[i][3]] * 2, dtype=np.float32)
        assert got_l[i].tolist() == el[eo[i]:eo[i + 1]].tolist(), i
        assert np.allclose(got_b[i], e, atol=2e-6), i
        kept += int((el[eo[i]:eo[i + 1]] > 0).sum())
    assert kept >= 3

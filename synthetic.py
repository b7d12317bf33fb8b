"""Seeded synthetic inputs with the shapes and value distributions of the five benchmark
configurations (no dataset is read; these stand in for decoded JPEG batches).

Everything is drawn from numpy.random.Generator(PCG64(seed)), so a (config, seed) pair names one
exact input. The builders return host-side numpy data: a packed uint8 arena with one HWC image
after another (row pitch = width*3, each image start rounded up to 256 bytes) and the per-sample
tables of rocal_b200.tables.
"""
import importlib.util
import math
import os

import numpy as np

# The table layouts come from the package's tables.py, loaded by path: importing the package itself would load the
# CUDA library, which the CPU arm of the benchmark and the oracle-only tests must not need.
_spec = importlib.util.spec_from_file_location(
    "_rocal_b200_tables", os.path.join(os.path.dirname(os.path.abspath(__file__)), "rocal_b200", "tables.py"))
T = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(T)

MEAN = (123.675, 116.28, 103.53)
STD = (58.395, 57.12, 57.375)


def rng_for(config_index, seed=1234):
    return np.random.Generator(np.random.PCG64(seed + config_index))


def normalize_tables(mean=MEAN, std=STD):
    """The two per-channel tables the CropMirrorNormalize node builds
    (node_crop_mirror_normalize.cpp:46-70): 1/std and -(mean * (1/std)), float32."""
    inv = [np.float32(1.0) / np.float32(s) for s in std]
    mul = [np.float32(v) for v in inv]
    add = [np.float32(-(np.float32(m) * v)) for m, v in zip(mean, inv)]
    return mul, add


def _fill_image(args):
    arena, o, h, w, seed, content = args
    rng = np.random.Generator(np.random.PCG64(int(seed)))
    noise = rng.integers(0, 256, size=(h, w, 3), dtype=np.uint8)
    if content == "noise":
        img = noise
    else:
        corners = rng.integers(0, 256, size=(2, 2, 3)).astype(np.float32)
        ty = np.linspace(0.0, 1.0, h, dtype=np.float32)[:, None, None]
        tx = np.linspace(0.0, 1.0, w, dtype=np.float32)[None, :, None]
        left = corners[0, 0] * (1 - ty) + corners[1, 0] * ty          # (h,1,3)
        right = corners[0, 1] * (1 - ty) + corners[1, 1] * ty
        grad = left + (right - left) * tx                             # (h,w,3) bilinear blend of the corners
        img = ((grad.astype(np.uint16) + noise + 1) >> 1).astype(np.uint8)
    arena[o:o + h * w * 3] = img.reshape(-1)


def make_images(rng, n, h_range, w_range, content="gradient_noise", threads=None):
    """Returns (arena uint8[total], heights int32[n], widths int32[n], offsets uint64[n]).
    Sizes and one child seed per image are drawn from `rng`; the pixels of image i come from its own
    PCG64(child seed), so the result does not depend on the number of worker threads."""
    hs = rng.integers(h_range[0], h_range[1] + 1, size=n).astype(np.int32)
    ws = rng.integers(w_range[0], w_range[1] + 1, size=n).astype(np.int32)
    seeds = rng.integers(0, 2 ** 62, size=n)
    sizes = hs.astype(np.int64) * ws.astype(np.int64) * 3
    padded = (sizes + 255) // 256 * 256
    offsets = np.zeros(n, dtype=np.uint64)
    offsets[1:] = np.cumsum(padded)[:-1]
    arena = np.zeros(int(padded.sum()) + 256, dtype=np.uint8)
    jobs = [(arena, int(offsets[i]), int(hs[i]), int(ws[i]), seeds[i], content) for i in range(n)]
    threads = threads or min(16, os.cpu_count() or 1)
    if n >= 16 and threads > 1:
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(threads) as ex:
            list(ex.map(_fill_image, jobs))
    else:
        for j in jobs:
            _fill_image(j)
    return arena, hs, ws, offsets


def resize_not_smaller(src_w, src_h, size):
    """Target size of `resize_shorter=size` (scaling mode NOT_SMALLER), float32 arithmetic of
    ResizeNode::adjust_out_roi_size (node_resize.cpp:120-137)."""
    scale_w = np.float32(size) / np.float32(src_w)
    scale_h = np.float32(size) / np.float32(src_h)
    scale = max(scale_w, scale_h)
    dst_w, dst_h = size, size
    if scale_h != scale:
        dst_h = _lround(np.float32(src_h) * scale)
    if scale_w != scale:
        dst_w = _lround(np.float32(src_w) * scale)
    return int(dst_w), int(dst_h)


def _lround(v):
    v = float(np.float32(v))
    return int(math.floor(abs(v) + 0.5)) * (1 if v >= 0 else -1)


def classification_tables(rng, hs, ws, offsets, resize_shorter=256, crop=224, max_out=None):
    """Resize(shorter side) -> crop (random position) -> mirror(p=.5): one RESAMPLE_SAMPLE row per image."""
    n = len(hs)
    t = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
    for i in range(n):
        w, h = int(ws[i]), int(hs[i])
        dw, dh = resize_not_smaller(w, h, resize_shorter)
        if max_out is not None:
            dw, dh = min(dw, max_out[0]), min(dh, max_out[1])
        cw, ch = min(crop, dw), min(crop, dh)
        t[i]["src_offset"] = offsets[i]
        t[i]["src_stride"] = w * 3
        t[i]["roi_x"], t[i]["roi_y"], t[i]["roi_w"], t[i]["roi_h"] = 0, 0, w, h
        t[i]["dst_w"], t[i]["dst_h"] = dw, dh
        t[i]["crop_x"] = int(rng.integers(0, dw - cw + 1))
        t[i]["crop_y"] = int(rng.integers(0, dh - ch + 1))
        t[i]["crop_w"], t[i]["crop_h"] = cw, ch
        t[i]["mirror"] = int(rng.random() < 0.5)
    return t


def color_twist_tables(rng, hs, ws, offsets, flip_prob=0.5):
    n = len(hs)
    t = np.zeros(n, dtype=T.POINTWISE_SAMPLE)
    t["src_offset"] = offsets
    t["src_stride"] = ws * 3
    t["roi_w"], t["roi_h"] = ws, hs
    t["alpha"] = rng.uniform(0.6, 1.4, n).astype(np.float32)
    t["beta"] = rng.uniform(0.6, 1.4, n).astype(np.float32)
    t["hue"] = rng.uniform(-30.0, 30.0, n).astype(np.float32)
    t["sat"] = rng.uniform(0.5, 1.5, n).astype(np.float32)
    t["flip_h"] = (rng.random(n) < flip_prob).astype(np.int32)
    return t


def warp_tables(rng, hs, ws, offsets, out_w, out_h, angle=(-45.0, 45.0), scale=(0.8, 1.2), shift=32.0):
    """Rotation by theta (counter-clockwise on screen, the direction of meta_node_rotate.cpp:53-68),
    isotropic scale s and translation t applied source->output; the table holds the inverse map."""
    n = len(hs)
    t = np.zeros(n, dtype=T.WARP_SAMPLE)
    t["src_offset"] = offsets
    t["src_stride"] = ws * 3
    t["src_w"], t["src_h"] = ws, hs
    t["dst_w"], t["dst_h"] = out_w, out_h
    th = np.deg2rad(rng.uniform(angle[0], angle[1], n))
    s = rng.uniform(scale[0], scale[1], n)
    tx = rng.uniform(-shift, shift, n)
    ty = rng.uniform(-shift, shift, n)
    c, sn = np.cos(th), np.sin(th)
    # forward: out = s * [[c, sn], [-sn, c]] @ src + t   =>   src = (1/s) * [[c, -sn], [sn, c]] @ (out - t)
    m00, m01, m10, m11 = c / s, -sn / s, sn / s, c / s
    t["m"][:, 0], t["m"][:, 1], t["m"][:, 2], t["m"][:, 3] = m00, m01, m10, m11
    t["m"][:, 4] = -(m00 * tx + m01 * ty)
    t["m"][:, 5] = -(m10 * tx + m11 * ty)
    return t


def rotate_matrix(angle_deg):
    """Inverse-map table of a pure rotation by angle_deg (image kernel twin of meta_node_rotate.cpp:53-68)."""
    r = np.float32(angle_deg) * np.float32(math.pi / 180.0)
    c, s = np.float32(math.cos(float(r))), np.float32(math.sin(float(r)))
    return np.array([c, -s, s, c, 0.0, 0.0], dtype=np.float32)


def ssd300_anchors():
    """8732 SSD-300 default boxes as ltrb in [0,1], generated procedurally (the reference reads
    them from a coco_anchors.bin file that is not part of its tree)."""
    fig = 300
    feat = [38, 19, 10, 5, 3, 1]
    steps = [8, 16, 32, 64, 100, 300]
    scales = [21, 45, 99, 153, 207, 261, 315]
    ratios = [[2], [2, 3], [2, 3], [2, 3], [2], [2]]
    out = []
    for idx, f in enumerate(feat):
        sk1, sk2 = scales[idx] / fig, scales[idx + 1] / fig
        sk3 = math.sqrt(sk1 * sk2)
        sizes = [(sk1, sk1), (sk3, sk3)]
        for a in ratios[idx]:
            w, h = sk1 * math.sqrt(a), sk1 / math.sqrt(a)
            sizes += [(w, h), (h, w)]
        fk = fig / steps[idx]
        for w, h in sizes:
            for i in range(f):
                for j in range(f):
                    cx, cy = (j + 0.5) / fk, (i + 0.5) / fk
                    out.append((cx, cy, w, h))
    a = np.clip(np.array(out, dtype=np.float64), 0.0, 1.0)
    ltrb = np.stack([a[:, 0] - 0.5 * a[:, 2], a[:, 1] - 0.5 * a[:, 3], a[:, 0] + 0.5 * a[:, 2],
                     a[:, 1] + 0.5 * a[:, 3]], axis=1)
    return np.ascontiguousarray(ltrb.astype(np.float32))


def random_boxes(rng, n, count_range=(1, 50), size_range=(0.05, 0.9), num_labels=80):
    """Per-sample ground truth: normalized ltrb boxes fully inside [0,1]^2, labels 1..num_labels.
    Returns (boxes float32[total,4], labels int32[total], offsets int32[n+1])."""
    counts = rng.integers(count_range[0], count_range[1] + 1, size=n)
    offsets = np.zeros(n + 1, dtype=np.int32)
    offsets[1:] = np.cumsum(counts)
    total = int(offsets[-1])
    w = rng.uniform(size_range[0], size_range[1], total)
    h = rng.uniform(size_range[0], size_range[1], total)
    l = rng.uniform(0.0, 1.0, total) * (1.0 - w)
    t = rng.uniform(0.0, 1.0, total) * (1.0 - h)
    boxes = np.stack([l, t, l + w, t + h], axis=1).astype(np.float32)
    labels = rng.integers(1, num_labels + 1, size=total).astype(np.int32)
    return boxes, labels, offsets


def _iou(box, crop):
    xa, ya = max(box[0], crop[0]), max(box[1], crop[1])
    xb, yb = min(box[2], crop[2]), min(box[3], crop[3])
    inter = max(0.0, xb - xa) * max(0.0, yb - ya)
    a1 = (box[2] - box[0]) * (box[3] - box[1])
    a2 = (crop[2] - crop[0]) * (crop[3] - crop[1])
    return inter / (a1 + a2 - inter)


def ssd_random_crop(rng, boxes, labels, offsets, num_attempts=20):
    """Seeded SSD random crop: per sample pick a minimum-IoU option, rejection-sample a window
    (w,h in [0.3,1], aspect in [0.5,2]) whose IoU with every box is >= the option and that holds at
    least one box centre; boxes whose centre falls outside are dropped, the rest clipped and
    re-normalised to the window (the mask and clip steps of update_random_bbox_meta_data,
    bounding_box_graph.cpp:98-110). Returns (crops float32[n,4] ltrb, boxes, labels, offsets)."""
    options = [None, 0.1, 0.3, 0.5, 0.7, 0.9, -1.0]
    n = len(offsets) - 1
    crops = np.zeros((n, 4), dtype=np.float32)
    new_boxes, new_labels, new_offsets = [], [], [0]
    for i in range(n):
        bb = boxes[offsets[i]:offsets[i + 1]].astype(np.float64)
        ll = labels[offsets[i]:offsets[i + 1]]
        crop = (0.0, 0.0, 1.0, 1.0)
        keep = np.ones(len(bb), dtype=bool)
        done = False
        while not done:
            opt = options[int(rng.integers(0, len(options)))]
            if opt is None:
                break
            for _ in range(num_attempts):
                w, h = rng.uniform(0.3, 1.0), rng.uniform(0.3, 1.0)
                if not (0.5 <= w / h <= 2.0):
                    continue
                x, y = rng.uniform(0.0, 1.0 - w), rng.uniform(0.0, 1.0 - h)
                c = (x, y, x + w, y + h)
                if opt >= 0 and any(_iou(b, c) < opt for b in bb):
                    continue
                xc, yc = 0.5 * (bb[:, 0] + bb[:, 2]), 0.5 * (bb[:, 1] + bb[:, 3])
                k = (xc > c[0]) & (xc < c[2]) & (yc > c[1]) & (yc < c[3])
                if not k.any():
                    continue
                crop, keep, done = c, k, True
                break
        crops[i] = crop
        cw, ch = crop[2] - crop[0], crop[3] - crop[1]
        kb = bb[keep]
        out = np.stack([(np.maximum(kb[:, 0], crop[0]) - crop[0]) / cw, (np.maximum(kb[:, 1], crop[1]) - crop[1]) / ch,
                        (np.minimum(kb[:, 2], crop[2]) - crop[0]) / cw, (np.minimum(kb[:, 3], crop[3]) - crop[1]) / ch],
                       axis=1)
        new_boxes.append(out.astype(np.float32))
        new_labels.append(ll[keep])
        new_offsets.append(new_offsets[-1] + int(keep.sum()))
    return (crops, np.ascontiguousarray(np.concatenate(new_boxes)), np.ascontiguousarray(np.concatenate(new_labels)),
            np.array(new_offsets, dtype=np.int32))


def ssd_resample_tables(rng, hs, ws, offsets, crops, size=300):
    """crop window (fractions of the image) -> resize to size x size (stretch) -> mirror(p=.5)."""
    n = len(hs)
    t = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
    for i in range(n):
        w, h = int(ws[i]), int(hs[i])
        x1, y1 = int(crops[i, 0] * w), int(crops[i, 1] * h)
        x2, y2 = max(x1 + 1, int(crops[i, 2] * w)), max(y1 + 1, int(crops[i, 3] * h))
        t[i]["src_offset"] = offsets[i]
        t[i]["src_stride"] = w * 3
        t[i]["roi_x"], t[i]["roi_y"], t[i]["roi_w"], t[i]["roi_h"] = x1, y1, min(x2, w) - x1, min(y2, h) - y1
        t[i]["dst_w"], t[i]["dst_h"] = size, size
        t[i]["crop_w"], t[i]["crop_h"] = size, size
        t[i]["mirror"] = int(rng.random() < 0.5)
    return t

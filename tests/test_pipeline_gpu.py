"""The rocAL-facing pipeline (C-ABI rb200_* behind rocal_b200.Pipeline / fn) against the CPU oracle.

Each test builds a graph with the reference's call sequence for one benchmark configuration, feeds
seeded synthetic batches, and rebuilds the expected per-sample tables independently: sizes and crop
windows from the oracle's host-logic restatements, random draws read back from the parameters.
"""
import ctypes

import numpy as np
import pytest

from oracle import pyoracle as O
import synthetic as S
from rocal_b200 import tables as T

pytestmark = pytest.mark.gpu

MEAN, STD = list(S.MEAN), list(S.STD)


def _classification_pipeline(batch, out_dtype, max_side=512, seed=7, depth=2):
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    pipe = Pipeline(batch_size=batch, device_id=0, seed=seed, prefetch_queue_depth=depth)
    with pipe:
        img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_UNCOMPRESSED, max_width=max_side, max_height=max_side)
        r = fn.resize(img, resize_shorter=256)
        mirror = fn.random.coin_flip(probability=0.5)
        out = fn.crop_mirror_normalize(r, crop=[224, 224], crop_pos_x=0.5, crop_pos_y=0.5, mean=MEAN, std=STD, mirror=mirror,
                                       output_layout=types.NCHW, output_dtype=out_dtype)
        pipe.set_outputs(out)
    pipe.build()
    return pipe, out, mirror


def _expected_classification(arena, hs, ws, offs, anchors_x, anchors_y, mirror, out_dtype):
    n = len(hs)
    t = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
    for i in range(n):
        dw, dh = O.resize_dst_size(int(ws[i]), int(hs[i]), 256, 256, 2, cap_w=1536, cap_h=1536)
        x1, y1, cw, ch = O.crop_fixed(dw, dh, 224, 224, float(anchors_x[i]), float(anchors_y[i]))
        t[i]["src_offset"], t[i]["src_stride"] = offs[i], ws[i] * 3
        t[i]["roi_w"], t[i]["roi_h"] = ws[i], hs[i]
        t[i]["dst_w"], t[i]["dst_h"] = dw, dh
        t[i]["crop_x"], t[i]["crop_y"], t[i]["crop_w"], t[i]["crop_h"] = x1, y1, cw, ch
        t[i]["mirror"] = mirror[i]
    mul, add = S.normalize_tables()
    return O.resample(arena, t, 224, 224, out_dtype, T.NCHW, mul, add)


@pytest.mark.parametrize("out_dtype", [T.FP32, T.FP16])
def test_config0_pipeline(cuda, out_dtype):
    """configs[0] through the API: external source -> rocalResize(shorter=256) -> rocalCropMirrorNormalize,
    per-sample crop anchors, coin-flip mirror; three batches through a depth-2 ring, ragged feed."""
    import torch
    from rocal_b200 import types
    rng = S.rng_for(0)
    pipe, out, mirror = _classification_pipeline(64, types.FLOAT if out_dtype == T.FP32 else types.FLOAT16)
    for batch in range(3):
        arena, hs, ws, offs = S.make_images(rng, 64, (256, 512), (256, 512))
        ax, ay = rng.random(64).astype(np.float32), rng.random(64).astype(np.float32)
        pipe.set_crop_anchors(out, ax, ay)
        pipe.feed_ragged(arena, hs, ws, offs)
        pipe.run()
        m = pipe.get_int_array(mirror)
        assert len(m) == 64 and set(np.unique(m)) <= {0, 1}
        exp = _expected_classification(arena, hs, ws, offs, ax, ay, m, out_dtype)
        (t,) = pipe.get_output_tensors()
        assert t.dims() == [64, 3, 224, 224]
        got = torch.from_dlpack(t)
        assert got.is_cuda and got.data_ptr() == t.buffer()
        got = got.cpu().numpy()
        assert np.array_equal(got.view(np.uint8), exp.view(np.uint8)), "batch %d" % batch
        assert np.array_equal(t.numpy().view(np.uint8), exp.view(np.uint8))     # copy_data path
        assert (t.roi()[:, 2:] == 224).all()
    pipe.rocal_release()


def test_triangular_resize_pipeline(cuda):
    """rocalResize(interpolation_type=ROCAL_TRIANGULAR_INTERPOLATION) -> rocalCropMirrorNormalize, the filter of the
    reference's imagenet example, fused into one launch; host input goes up as footprint rectangles widened by the
    filter radius."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(22)
    n = 8
    pipe = Pipeline(batch_size=n, device_id=0, seed=5)
    with pipe:
        img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_UNCOMPRESSED, max_width=600, max_height=600)
        r = fn.resize(img, resize_shorter=128, interpolation_type=types.TRIANGULAR_INTERPOLATION)
        mirror = fn.random.coin_flip()
        out = fn.crop_mirror_normalize(r, crop=[112, 112], mean=MEAN, std=STD, mirror=mirror, output_layout=types.NCHW,
                                       output_dtype=types.FLOAT)
        pipe.set_outputs(out)
    pipe.build()
    for _ in range(2):
        arena, hs, ws, offs = S.make_images(rng, n, (150, 600), (150, 600))
        ax, ay = rng.random(n).astype(np.float32), rng.random(n).astype(np.float32)
        pipe.set_crop_anchors(out, ax, ay)
        pipe.feed_ragged(arena, hs, ws, offs)
        pipe.run()
        m = pipe.get_int_array(mirror)
        t = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
        for i in range(n):
            dw, dh = O.resize_dst_size(int(ws[i]), int(hs[i]), 128, 128, 2, cap_w=768, cap_h=768)
            x1, y1, cw, ch = O.crop_fixed(dw, dh, 112, 112, float(ax[i]), float(ay[i]))
            t[i]["src_offset"], t[i]["src_stride"] = offs[i], ws[i] * 3
            t[i]["roi_w"], t[i]["roi_h"], t[i]["dst_w"], t[i]["dst_h"] = ws[i], hs[i], dw, dh
            t[i]["crop_x"], t[i]["crop_y"], t[i]["crop_w"], t[i]["crop_h"], t[i]["mirror"] = x1, y1, cw, ch, m[i]
        mul, add = S.normalize_tables()
        exp = O.resample(arena, t, 112, 112, T.FP32, T.NCHW, mul, add, interpolation=1)
        assert np.array_equal(pipe.get_output_tensors()[0].numpy(), exp)
    pipe.rocal_release()


def _jpeg_batch(rng, n, size_range):
    """Smooth synthetic images (JPEG-friendly), their 4:4:4 quality-95 JPEG streams and the host decoder's pixels."""
    cv2 = pytest.importorskip("cv2")
    imgs, streams = [], []
    for _ in range(n):
        h, w = int(rng.integers(*size_range)), int(rng.integers(*size_range))
        yy, xx = np.mgrid[0:h, 0:w].astype(np.float32)
        chans = [127 + 100 * np.sin(xx / rng.uniform(15, 60) + rng.uniform(0, 6)) * np.cos(yy / rng.uniform(15, 60)) for _ in range(3)]
        rgb = np.clip(np.stack(chans, axis=-1) + rng.normal(0, 3, (h, w, 3)), 0, 255).astype(np.uint8)
        ok, enc = cv2.imencode(".jpg", rgb[:, :, ::-1], [cv2.IMWRITE_JPEG_QUALITY, 95, cv2.IMWRITE_JPEG_SAMPLING_FACTOR,
                                                         cv2.IMWRITE_JPEG_SAMPLING_FACTOR_444])
        assert ok
        streams.append(enc.tobytes())
        imgs.append(np.ascontiguousarray(cv2.imdecode(enc, cv2.IMREAD_COLOR)[:, :, ::-1]))
    return imgs, streams


def test_jpeg_external_source(cuda, tmp_path):
    """rocalJpegExternalFileSource in RAW_COMPRESSED and FNAME mode: JPEG streams are decoded on the GPU into the
    arena the kernels read. The decoded pixels (through an identity flip) stay within a few grey levels of the host
    decoder's (the two IDCTs differ in rounding), and Resize + CropMirrorNormalize on them matches the oracle run on
    the host-decoded pixels to the same degree."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(23)
    n = 6
    imgs, streams = _jpeg_batch(rng, n, (120, 400))
    for mode in (types.EXTSOURCE_RAW_COMPRESSED, types.EXTSOURCE_FNAME):
        pipe = Pipeline(batch_size=n, device_id=0, seed=3)
        with pipe:
            img, _ = fn.external_source(None, mode=mode, max_width=400, max_height=400)
            ident = fn.flip(img, horizontal=0, vertical=0)
            r = fn.resize(img, resize_shorter=96)
            out = fn.crop_mirror_normalize(r, crop=[80, 80], crop_pos_x=0.5, crop_pos_y=0.5, mean=MEAN, std=STD, mirror=0,
                                           output_layout=types.NCHW, output_dtype=types.FLOAT)
            pipe.set_outputs(ident, out)
        pipe.build()
        if mode == types.EXTSOURCE_FNAME:
            paths = []
            for i, sbytes in enumerate(streams):
                p = tmp_path / ("img%d.jpg" % i)
                p.write_bytes(sbytes)
                paths.append(str(p))
            pipe.feed_files(paths)
        else:
            pipe.feed_encoded(streams)
        pipe.run()
        dec, res = [t.numpy() for t in pipe.get_output_tensors()]
        hs = np.array([im.shape[0] for im in imgs])
        ws = np.array([im.shape[1] for im in imgs])
        offs = np.concatenate([[0], np.cumsum(hs * ws * 3)])[:-1]
        arena = np.concatenate([im.reshape(-1) for im in imgs])
        for i in range(n):
            d = np.abs(dec[i, :hs[i], :ws[i]].astype(np.int32) - imgs[i].astype(np.int32))
            assert d.max() <= 6 and d.mean() < 0.7, (i, d.max(), d.mean())
        # the geometry of _classification_pipeline with shorter side 96 / crop 80
        t = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
        for i in range(n):
            dw, dh = O.resize_dst_size(int(ws[i]), int(hs[i]), 96, 96, 2, cap_w=576, cap_h=576)
            x1, y1, cw, ch = O.crop_fixed(dw, dh, 80, 80, 0.5, 0.5)
            t[i]["src_offset"], t[i]["src_stride"] = offs[i], ws[i] * 3
            t[i]["roi_w"], t[i]["roi_h"], t[i]["dst_w"], t[i]["dst_h"] = ws[i], hs[i], dw, dh
            t[i]["crop_x"], t[i]["crop_y"], t[i]["crop_w"], t[i]["crop_h"] = x1, y1, cw, ch
        mul, add = S.normalize_tables()
        exp = O.resample(arena, t, 80, 80, T.FP32, T.NCHW, mul, add)
        diff = np.abs(res - exp)
        assert diff.max() <= 6.5 / 57.0 and diff.mean() < 0.02, (diff.max(), diff.mean())
        assert pipe.timing_info()["decode_time"] > 0
        pipe.rocal_release()


def test_file_source_pipeline(cuda, tmp_path):
    """A folder of JPEG files through fn.readers.file + fn.decoders.image (rocalJpegFileSourceSingleShard with the
    folder label reader): the pipeline feeds itself; labels, names, batch count and last-batch padding follow the
    folder; a second epoch after reset(); the images match the oracle on the host-decoded pixels as closely as the
    two JPEG decoders agree."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    from rocal_b200.plugin.pytorch import ROCALClassificationIterator
    rng = S.rng_for(24)
    imgs, streams = _jpeg_batch(rng, 7, (120, 300))
    classes = ["apple", "apple", "apple", "berry", "berry", "cherry", "cherry"]
    by_name = {}
    for i, (cls, sb) in enumerate(zip(classes, streams)):
        d = tmp_path / cls
        d.mkdir(exist_ok=True)
        (d / ("im%d.jpg" % i)).write_bytes(sb)
        by_name["im%d.jpg" % i] = (imgs[i], sorted(set(classes)).index(cls))
    n = 3
    pipe = Pipeline(batch_size=n, device_id=0, seed=4)
    with pipe:
        jpegs, _ = fn.readers.file(file_root=str(tmp_path))
        img = fn.decoders.image(jpegs, file_root=str(tmp_path), shard_id=0, num_shards=1, max_decoded_width=300, max_decoded_height=300,
                                last_batch_policy=types.LAST_BATCH_FILL, pad_last_batch=True)
        r = fn.resize(img, resize_shorter=96)
        out = fn.crop_mirror_normalize(r, crop=[80, 80], crop_pos_x=0.5, crop_pos_y=0.5, mean=MEAN, std=STD, mirror=0,
                                       output_layout=types.NCHW, output_dtype=types.FLOAT)
        pipe.set_outputs(out)
    pipe.build()
    assert pipe.get_remaining_images() == 9          # 7 files padded to 3 batches of 3
    mul, add = S.normalize_tables()
    for epoch in range(2):
        seen = []
        for k, (outs, labels) in enumerate(ROCALClassificationIterator(pipe)):
            names = pipe.get_image_names()
            assert labels.is_cuda and labels.cpu().tolist() == [by_name[nm][1] for nm in names]
            hot = pipe.get_one_hot_encoded_labels(3)
            for i, nm in enumerate(names):      # rocalGetOneHotImageLabels: label k > 0 -> position k-1, label 0 -> last
                lab = by_name[nm][1]
                assert hot[i].tolist() == [1 if p == (lab - 1 if lab > 0 else 2) else 0 for p in range(3)]
            assert np.array_equal(hot, pipe.get_one_hot_encoded_labels(3, device="cuda:0").cpu().numpy())
            assert pipe.get_image_sizes().tolist() == [[by_name[nm][0].shape[1], by_name[nm][0].shape[0]] for nm in names]
            res = outs[0].cpu().numpy()
            for i, nm in enumerate(names):
                im = by_name[nm][0]
                h, w = im.shape[:2]
                t = np.zeros(1, dtype=T.RESAMPLE_SAMPLE)
                dw, dh = O.resize_dst_size(w, h, 96, 96, 2, cap_w=576, cap_h=576)
                x1, y1, cw, ch = O.crop_fixed(dw, dh, 80, 80, 0.5, 0.5)
                t["src_stride"], t["roi_w"], t["roi_h"], t["dst_w"], t["dst_h"] = w * 3, w, h, dw, dh
                t["crop_x"], t["crop_y"], t["crop_w"], t["crop_h"] = x1, y1, cw, ch
                exp = O.resample(im.reshape(-1), t, 80, 80, T.FP32, T.NCHW, mul, add)[0]
                diff = np.abs(res[i] - exp)
                assert diff.max() <= 6.5 / 57.0 and diff.mean() < 0.02, (nm, diff.max(), diff.mean())
            seen += names
            assert pipe.get_last_batch_padded_size() == (2 if k == 2 else 0)
        assert seen == ["im0.jpg", "im1.jpg", "im2.jpg", "im3.jpg", "im4.jpg", "im5.jpg", "im6.jpg", "im6.jpg", "im6.jpg"]
        assert pipe.is_empty()
        with pytest.raises(Exception):
            pipe.rocal_run()
        pipe.reset()
    pipe.rocal_release()


def test_coco_source_pipeline(cuda, tmp_path):
    """A COCO-format detection dataset through fn.readers.coco + fn.decoders.image: the boxes of the annotation file
    follow the images through the flip, reach the box encoder and come back through the bounding-box getters."""
    import json
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(26)
    n = 4
    imgs, streams = _jpeg_batch(rng, n, (150, 320))
    images, anns, truth = [], [], {}
    for i, (im, sb) in enumerate(zip(imgs, streams)):
        name = "%03d.jpg" % i
        (tmp_path / name).write_bytes(sb)
        h, w = im.shape[:2]
        images.append({"id": 100 + i, "file_name": name, "width": w, "height": h})
        k = int(rng.integers(1, 6)) if i != 2 else 0          # one image without annotations
        bx = []
        for _ in range(k):
            x, y = float(rng.uniform(0, w * 0.6)), float(rng.uniform(0, h * 0.6))
            bw, bh = float(rng.uniform(w * 0.1, w * 0.4)), float(rng.uniform(h * 0.1, h * 0.4))
            cat = int(rng.choice([7, 21, 44]))
            anns.append({"id": len(anns), "image_id": 100 + i, "category_id": cat, "bbox": [x, y, bw, bh], "iscrowd": 0})
            bx.append(([x / w, y / h, (x + bw) / w, (y + bh) / h], {7: 1, 21: 2, 44: 3}[cat]))
        truth[name] = bx
    (tmp_path / "ann.json").write_text(json.dumps({"images": images, "annotations": anns,
                                                    "categories": [{"id": 7}, {"id": 21}, {"id": 44}]}))
    anchors = S.ssd300_anchors()[::4].copy()
    pipe = Pipeline(batch_size=n, device_id=0, seed=6)
    with pipe:
        jpegs, _, _ = fn.readers.coco(annotations_file=str(tmp_path / "ann.json"), ltrb=True, is_box_encoder=True)
        img = fn.decoders.image(jpegs, file_root=str(tmp_path), max_decoded_width=320, max_decoded_height=320)
        r = fn.resize(img, resize_width=128, resize_height=128, scaling_mode=types.SCALING_MODE_STRETCH)
        out = fn.crop_mirror_normalize(r, crop=[128, 128], crop_pos_x=0.0, crop_pos_y=0.0, mean=MEAN, std=STD, mirror=1,
                                       output_layout=types.NCHW, output_dtype=types.FLOAT)
        fn.box_encoder(anchors=anchors, criteria=0.5, means=[0, 0, 0, 0], stds=[0.1, 0.1, 0.2, 0.2], offset=True, scale=1.0)
        pipe.set_outputs(out)
    pipe.build()
    pipe.run()
    names = pipe.get_image_names()
    assert names == ["000.jpg", "001.jpg", "002.jpg", "003.jpg"]
    assert pipe.get_image_id().tolist() == [100, 101, 102, 103]            # rocalGetImageId: the file's image ids
    ids = np.zeros(n, dtype=np.int32)
    pipe.get_image_id(ids)
    sizes = np.zeros((n, 2), dtype=np.int32)
    pipe.get_img_sizes(sizes)
    lens = np.zeros(n, dtype=np.int32)
    assert ids.tolist() == [100, 101, 102, 103] and sizes.tolist() == pipe.get_image_sizes().tolist()
    assert pipe.get_image_name_length(lens) == 28 and lens.tolist() == [7] * 4 and pipe.get_image_name(28) == "".join(names)
    assert pipe.get_bounding_box_count() == sum(len(x) for x in pipe.get_bounding_box_labels())
    assert [len(x) for x in pipe.get_bounding_box_cords()] == [len(x) for x in pipe.get_bounding_box_labels()]
    b2, l2, c2 = pipe.get_bounding_boxes()
    at = 0
    for nm, c in zip(names, c2):
        exp = truth[nm]
        if not exp:
            # an image without annotations arrives with one empty box; CropMirrorNormalize's metadata rule drops it
            # (no area inside the window) and answers with the whole window and label 0
            # (meta_node_crop_mirror_normalize.cpp:56,84-88)
            assert c == 1 and l2[at] == 0 and b2[at].tolist() == [0.0, 0.0, 1.0, 1.0]
        else:
            assert c == len(exp)
            for k, (box, lab) in enumerate(exp):
                mirrored = [1.0 - box[2], box[1], 1.0 - box[0], box[3]]        # mirror = 1 flips the boxes with the image
                assert l2[at + k] == lab and np.allclose(b2[at + k], mirrored, atol=1e-5), (nm, k)
        at += c
    o2 = np.concatenate([[0], np.cumsum(c2)]).astype(np.int32)
    eb, el = O.box_encode(b2, l2, o2, anchors, 0.5, (0, 0, 0, 0), (0.1, 0.1, 0.2, 0.2), True, 1.0)
    gb, gl = pipe.get_encoded_boxes_and_lables()
    assert np.array_equal(gl, el) and np.allclose(gb, eb, rtol=1e-5, atol=1e-6)
    assert pipe.get_output_tensors()[0].numpy().shape == (n, 3, 128, 128)
    pipe.rocal_release()


def test_ssd_training_pipeline_from_coco_files(cuda, tmp_path):
    """The reference's SSD training graph from a COCO folder (readers.coco -> random_bbox_crop -> decoders.image_slice ->
    resize 300 x 300 -> crop_mirror_normalize(mirror) -> box_encoder), two batches. Behind random_bbox_crop the fused
    decoder cuts the box-aware windows: they are the pinned sampler's (its counter runs on across batches), the pixels
    are the oracle's resize + mirror + normalise of that window of the decoder's own pixels, the boxes follow by the
    centre rule, then the mirror, and reach the encoder. The mirror is a coin flip per sample: its values are read back per
    batch (the loader works ahead with a folder source, so the parameter object itself already holds a later batch's
    draws when this one is returned)."""
    import json
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(27)
    n, files = 4, 8
    imgs, streams = _jpeg_batch(rng, files, (150, 320))
    pixels = _decoded_by_pipeline(streams, 320)
    images, anns, truth = [], [], {}
    for i, (im, sb) in enumerate(zip(imgs, streams)):
        name = "s%02d.jpg" % i
        (tmp_path / name).write_bytes(sb)
        h, w = im.shape[:2]
        images.append({"id": 500 + i, "file_name": name, "width": w, "height": h})
        bx = []
        for _ in range(int(rng.integers(1, 5))):
            x, y = float(rng.uniform(0, w * 0.6)), float(rng.uniform(0, h * 0.6))
            bw, bh = float(rng.uniform(w * 0.15, w * 0.4)), float(rng.uniform(h * 0.15, h * 0.4))
            anns.append({"id": len(anns), "image_id": 500 + i, "category_id": 9, "bbox": [x, y, bw, bh], "iscrowd": 0})
            # the reader's arithmetic: corners summed in double, narrowed to float, divided by the float size
            bx.append([np.float32(x) / np.float32(w), np.float32(y) / np.float32(h),
                       np.float32(x + bw) / np.float32(w), np.float32(y + bh) / np.float32(h)])
        truth[name] = np.array(bx, dtype=np.float32)
    (tmp_path / "ann.json").write_text(json.dumps({"images": images, "annotations": anns, "categories": [{"id": 9}]}))
    anchors = S.ssd300_anchors()[::4].copy()
    seed = 77
    pipe = Pipeline(batch_size=n, device_id=0, seed=8)
    with pipe:
        jpegs, _, _ = fn.readers.coco(annotations_file=str(tmp_path / "ann.json"), ltrb=True, is_box_encoder=True)
        fn.random_bbox_crop(all_boxes_above_threshold=False, seed=seed)
        img = fn.decoders.image_slice(jpegs, file_root=str(tmp_path), annotations_file=str(tmp_path / "ann.json"),
                                      max_decoded_width=320, max_decoded_height=320)
        r = fn.resize(img, resize_width=300, resize_height=300, scaling_mode=types.SCALING_MODE_STRETCH)
        mirror = fn.random.coin_flip()
        out = fn.crop_mirror_normalize(r, crop=[300, 300], crop_pos_x=0.0, crop_pos_y=0.0, mean=MEAN, std=STD, mirror=mirror,
                                       output_layout=types.NCHW, output_dtype=types.FLOAT)
        fn.box_encoder(anchors=anchors, criteria=0.5, means=[0, 0, 0, 0], stds=[0.1, 0.1, 0.2, 0.2], offset=True, scale=1.0)
        pipe.set_outputs(out)
    pipe.build()
    sampler = O.BBoxCropSampler(seed, False)
    mul, add = S.normalize_tables()
    cropped, seen_flags = 0, set()
    for batch in range(2):
        got = pipe.run()[0].numpy()
        flags = pipe.get_int_array(mirror)
        seen_flags.update(int(v) for v in flags)
        names = pipe.get_image_names()
        idx = [int(nm[1:3]) for nm in names]
        assert idx == list(range(batch * n, batch * n + n))
        boxes = np.concatenate([truth[nm] for nm in names])
        offs = np.concatenate([[0], np.cumsum([len(truth[nm]) for nm in names])]).astype(np.int32)
        ws = np.array([pixels[i].shape[1] for i in idx])
        hs = np.array([pixels[i].shape[0] for i in idx])
        frac = sampler.windows(boxes, offs, ws)
        assert np.array_equal(pipe.get_bbox_crop_windows(), frac)
        win, _ = pipe.get_decoder_crop_windows()
        cropped += int((win[:, 2] < ws).sum())
        # pixels: window of the decoder's pixels -> 300 x 300 -> mirror -> normalise, one launch in the oracle too
        arena = np.concatenate([pixels[i].reshape(-1) for i in idx])
        poffs = np.concatenate([[0], np.cumsum([pixels[i].size for i in idx])])[:-1]
        t = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
        t["src_stride"] = ws * 3
        t["src_offset"] = poffs + win[:, 1].astype(np.int64) * t["src_stride"] + win[:, 0].astype(np.int64) * 3
        t["roi_w"], t["roi_h"], t["dst_w"], t["dst_h"], t["crop_w"], t["crop_h"] = win[:, 2], win[:, 3], 300, 300, 300, 300
        t["mirror"] = flags
        assert np.array_equal(got, O.resample(arena, t, 300, 300, T.FP32, T.NCHW, mul, add))
        # boxes: centre rule against the pixel window, then the whole-image CropMirrorNormalize with its mirror
        wf = win.astype(np.float32)
        nwin = np.stack([wf[:, 0] / ws, wf[:, 1] / hs, (wf[:, 0] + wf[:, 2]) / ws, (wf[:, 1] + wf[:, 3]) / hs], 1).astype(np.float32)
        b1, l1, o1 = O.box_transform(boxes, np.ones(len(boxes), np.int32), offs, nwin, 1)
        b2, l2, o2 = O.box_transform(b1, l1, o1, np.tile(np.array([[0, 0, 1, 1]], np.float32), (n, 1)), 0, mirror_h=flags)
        gb, gl, gc = pipe.get_bounding_boxes()
        assert np.array_equal(np.concatenate([[0], np.cumsum(gc)]), o2) and np.array_equal(gl, l2)
        assert np.allclose(gb, b2, atol=3e-6)
        eb, el = O.box_encode(gb, gl, o2, anchors, 0.5, (0, 0, 0, 0), (0.1, 0.1, 0.2, 0.2), True, 1.0)
        xb, xl = pipe.get_encoded_boxes_and_lables()
        assert np.array_equal(xl, el) and np.allclose(xb, eb, rtol=1e-5, atol=1e-6)
    assert cropped > 0 and seen_flags == {0, 1}
    pipe.rocal_release()


def test_resize_mirror_normalize_min_max(cuda):
    """rocalResizeMirrorNormalize with ROCAL_SCALING_MODE_MIN_MAX (the MaskRCNN resize): the shorter side becomes the
    minimum size unless the longer one would pass the maximum size; one fused launch, ragged outputs with their ROI."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(27)
    n = 8
    pipe = Pipeline(batch_size=n, device_id=0, seed=8)
    with pipe:
        img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_UNCOMPRESSED, max_width=400, max_height=400)
        mirror = fn.random.coin_flip()
        out = fn.resize_mirror_normalize(img, scaling_mode=types.SCALING_MODE_MIN_MAX, resize_shorter=64, resize_longer=96,
                                         max_size=[96, 96], mean=MEAN, std=STD, mirror=mirror, output_layout=types.NHWC,
                                         output_dtype=types.FLOAT)
        pipe.set_outputs(out)
    pipe.build()
    arena, hs, ws, offs = S.make_images(rng, n, (80, 400), (80, 400))
    hs[0], ws[0] = 90, 390              # the longer side limits this one
    pipe.feed_ragged(arena, hs, ws, offs)
    pipe.run()
    m = pipe.get_int_array(mirror)
    (t,) = pipe.get_output_tensors()
    got, roi = t.numpy(), t.roi()
    tab = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
    for i in range(n):
        dw, dh = O.resize_dst_size(int(ws[i]), int(hs[i]), 0, 0, 4, max_w=64, max_h=96, cap_w=96, cap_h=96)
        assert (roi[i, 2], roi[i, 3]) == (dw, dh) and min(dw, dh) <= 64 and max(dw, dh) <= 96
        tab[i]["src_offset"], tab[i]["src_stride"] = offs[i], ws[i] * 3
        tab[i]["roi_w"], tab[i]["roi_h"], tab[i]["dst_w"], tab[i]["dst_h"] = ws[i], hs[i], dw, dh
        tab[i]["crop_w"], tab[i]["crop_h"], tab[i]["mirror"] = dw, dh, m[i]
    mul, add = S.normalize_tables()
    exp = O.resample(arena, tab, 96, 96, T.FP32, T.NHWC, mul, add)
    assert np.array_equal(got, exp)
    assert (int(roi[0, 2]), int(roi[0, 3])) == (95, 22)          # 390 x 90: size = round(96*90/390) = 22, width = 22*390//90
    assert pipe.get_roi_image_sizes().tolist() == roi[:, 2:].tolist()     # rocalGetROIImageSizes follows ResizeMirrorNormalize
    pipe.rocal_release()


def test_upload_modes(cuda):
    """Host input reaches the kernels whole, as the rectangle the crop can read, or - pinned memory - without a
    copy (the kernel's bulk copies read the pinned buffer): the result is the same, the bytes moved are not.
    The device arenas are poisoned first (a batch of 0xFF images) so that a row the footprint missed would show."""
    import torch
    from rocal_b200 import types
    moved = {}
    for mode in (2, 1, 0):
        rng = S.rng_for(21)
        pipe, out, mirror = _classification_pipeline(16, types.FLOAT, max_side=700, seed=11)
        pipe.set_upload_mode(mode)
        arena, hs, ws, offs = S.make_images(rng, 16, (300, 700), (300, 700))
        for _ in range(2):                               # both arenas
            pipe.set_crop_anchors(out, np.full(16, 0.5, np.float32), np.full(16, 0.5, np.float32))
            pipe.feed_ragged(np.full_like(arena, 255), hs, ws, offs)
            pipe.run()
        ax, ay = rng.random(16).astype(np.float32), rng.random(16).astype(np.float32)
        ax[0], ay[0], ax[1], ay[1] = 0.0, 0.0, 1.0, 1.0   # windows at the corners
        before = pipe.h2d_bytes()
        pipe.set_crop_anchors(out, ax, ay)
        fed = torch.from_numpy(arena).pin_memory() if mode == 2 else arena
        pipe.feed_ragged(fed, hs, ws, offs)
        pipe.run()
        moved[mode] = pipe.h2d_bytes() - before
        m = pipe.get_int_array(mirror)
        got = pipe.get_output_tensors()[0].numpy()
        exp = _expected_classification(arena, hs, ws, offs, ax, ay, m, T.FP32)
        assert np.array_equal(got, exp), mode
        pipe.rocal_release()
    whole = int((hs.astype(np.int64) * ws * 3).sum())
    assert whole <= moved[0] < whole + 4096
    assert moved[1] < 0.85 * whole and moved[2] < 0.85 * whole


def test_slot_feed_and_prefetch_order(cuda):
    """The reference's feed contract (max-size slots + ROI per sample), two batches queued before the
    first run: results come back in feed order and match the ragged path's expectation."""
    from rocal_b200 import types
    rng = S.rng_for(20)
    pipe, out, mirror = _classification_pipeline(8, types.FLOAT, max_side=400, depth=3)
    batches = []
    for _ in range(2):
        arena, hs, ws, offs = S.make_images(rng, 8, (256, 400), (256, 400))
        imgs = [arena[int(offs[i]):int(offs[i]) + hs[i] * ws[i] * 3].reshape(hs[i], ws[i], 3) for i in range(8)]
        pipe.feed_input(imgs)
        batches.append((arena, hs, ws, offs))
    assert pipe.get_remaining_images() == 16
    for arena, hs, ws, offs in batches:
        pipe.run()
        got = pipe.get_output_tensors()[0].numpy()
        # the mirror draw of this batch is not observable once the next batch was prepared: accept either flag per sample
        e0 = _expected_classification(arena, hs, ws, offs, [0.5] * 8, [0.5] * 8, [0] * 8, T.FP32)
        e1 = _expected_classification(arena, hs, ws, offs, [0.5] * 8, [0.5] * 8, [1] * 8, T.FP32)
        for i in range(8):
            assert np.array_equal(got[i], e0[i]) or np.array_equal(got[i], e1[i]), "sample %d" % i
    assert pipe.is_empty()
    with pytest.raises(Exception):
        pipe.run()      # nothing fed
    pipe.rocal_release()


def test_unfused_outputs_and_to_tensor(cuda):
    """Resize marked as an output is materialised (padded max-shape uint8 tensor with per-sample ROI) and
    the CropMirrorNormalize reads it; both outputs match the oracle. rocalToTensor converts the first output."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(21)
    n = 6
    pipe = Pipeline(batch_size=n, device_id=0, seed=3)
    with pipe:
        img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_UNCOMPRESSED, max_width=300, max_height=300)
        r = fn.resize(img, resize_width=160, resize_height=120, scaling_mode=types.SCALING_MODE_STRETCH)
        out = fn.crop_mirror_normalize(r, crop=[100, 128], crop_pos_x=1.0, crop_pos_y=0.0, mean=MEAN, std=STD, mirror=1,
                                       output_layout=types.NHWC, output_dtype=types.FLOAT)
        pipe.set_outputs(r, out)
    pipe.build()
    arena, hs, ws, offs = S.make_images(rng, n, (100, 300), (100, 300))
    pipe.feed_ragged(arena, hs, ws, offs)
    pipe.run()
    t_r, t_out = pipe.get_output_tensors()
    tab = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
    tab["src_offset"], tab["src_stride"], tab["roi_w"], tab["roi_h"] = offs, ws * 3, ws, hs
    tab["dst_w"], tab["dst_h"], tab["crop_w"], tab["crop_h"] = 160, 120, 160, 120
    exp_r = O.resample(arena, tab, 160, 120, T.UINT8, T.NHWC)
    got_r = t_r.numpy()
    assert np.array_equal(got_r, exp_r)
    pw = np.zeros(n, dtype=T.POINTWISE_SAMPLE)
    pw["src_offset"] = np.arange(n) * 160 * 120 * 3
    pw["src_stride"], pw["roi_x"], pw["roi_y"], pw["roi_w"], pw["roi_h"], pw["flip_h"] = 160 * 3, 32, 0, 128, 100, 1
    mul, add = S.normalize_tables()
    exp_out = O.pointwise(exp_r.reshape(-1), pw, 128, 100, T.COLOR_NONE, T.FP32, T.NHWC, mul, add)
    assert np.array_equal(t_out.numpy(), exp_out)
    # rocalToTensor: first output (uint8 NHWC) -> fp32 NCHW with x*mult+off and channel reversal
    conv = np.zeros((n, 3, 120, 160), dtype=np.float32)
    pipe.copyToExternalTensor(conv, [0.5, 0.25, 2.0], [1.0, -1.0, 0.0], True, types.NCHW, types.FLOAT)
    src = exp_r.astype(np.float32)[..., ::-1]
    ref = np.stack([np.float32(src[..., c]) * np.float32([0.5, 0.25, 2.0][c]) + np.float32([1.0, -1.0, 0.0][c]) for c in range(3)], axis=1)
    assert np.allclose(conv, ref, rtol=1e-6, atol=1e-6)
    pipe.rocal_release()


def test_config2_color_twist_flip_pipeline(cuda):
    """configs[2] through the API: rocalColorTwist (4 uniform random parameters) -> rocalFlip (coin flip),
    fused into one launch; uint8 NHWC."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(2)
    n = 64
    pipe = Pipeline(batch_size=n, device_id=0, seed=11)
    with pipe:
        img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_UNCOMPRESSED, max_width=224, max_height=224)
        a = fn.random.uniform(range=(0.6, 1.4))
        b = fn.random.uniform(range=(0.6, 1.4))
        h = fn.random.uniform(range=(-30.0, 30.0))
        s = fn.random.uniform(range=(0.5, 1.5))
        ct = fn.color_twist(img, brightness=a, contrast=b, hue=h, saturation=s)
        hf = fn.random.coin_flip()
        out = fn.flip(ct, horizontal=hf, vertical=0)
        pipe.set_outputs(out)
    pipe.build()
    for _ in range(2):
        arena, hs, ws, offs = S.make_images(rng, n, (224, 224), (224, 224), content="noise")
        pipe.feed_ragged(arena, hs, ws, offs)
        pipe.run()
        tab = np.zeros(n, dtype=T.POINTWISE_SAMPLE)
        tab["src_offset"], tab["src_stride"], tab["roi_w"], tab["roi_h"] = offs, ws * 3, ws, hs
        tab["alpha"], tab["beta"] = pipe.get_float_array(a), pipe.get_float_array(b)
        tab["hue"], tab["sat"] = pipe.get_float_array(h), pipe.get_float_array(s)
        tab["flip_h"] = pipe.get_int_array(hf)
        assert 0.6 <= tab["alpha"].min() and tab["alpha"].max() <= 1.4 and len(np.unique(tab["hue"])) > n // 2
        exp = O.pointwise(arena, tab, 224, 224, T.COLOR_TWIST)
        got = pipe.get_output_tensors()[0].numpy()
        assert np.abs(got.astype(np.int32) - exp.astype(np.int32)).max() <= 1
        assert np.array_equal(got, exp)
    pipe.rocal_release()


def test_config3_warp_affine_and_rotate_pipeline(cuda):
    """configs[3] through the API: rocalWarpAffine with per-sample tables (extension), and rocalRotateFixed 45."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(3)
    n = 16
    pipe = Pipeline(batch_size=n, device_id=0, seed=5)
    with pipe:
        img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_UNCOMPRESSED, max_width=640, max_height=480)
        w = fn.warp_affine(img, dest_width=640, dest_height=480, matrix=[1.0, 0.0, 0.0, 1.0, 0.0, 0.0])
        r = fn.rotate(img, angle=45.0, dest_width=640, dest_height=480)
        pipe.set_outputs(w, r)
    pipe.build()
    arena, hs, ws, offs = S.make_images(rng, n, (480, 480), (640, 640))
    tab = S.warp_tables(rng, hs, ws, offs, 640, 480)
    pipe.set_affine(w, tab["m"])
    pipe.feed_ragged(arena, hs, ws, offs)
    pipe.run()
    t_w, t_r = pipe.get_output_tensors()
    assert np.array_equal(t_w.numpy(), O.warp_affine(arena, tab, 640, 480))
    rt = tab.copy()
    rt["m"][:] = S.rotate_matrix(45.0)
    assert np.array_equal(t_r.numpy(), O.warp_affine(arena, rt, 640, 480))
    # second batch without a table: the fixed parameters of the graph (identity) apply
    pipe.feed_ragged(arena, hs, ws, offs)
    pipe.run()
    it = tab.copy()
    it["m"][:] = np.array([1, 0, 0, 1, 0, 0], dtype=np.float32)
    assert np.array_equal(pipe.get_output_tensors()[0].numpy(), O.warp_affine(arena, it, 640, 480))
    pipe.rocal_release()


def test_config4_ssd_pipeline(cuda):
    """configs[4] through the API: rocalSSDRandomCrop -> rocalResize(300x300) -> rocalCropMirrorNormalize fp32 NCHW
    fused into one launch, plus rocalBoxEncoder and rocalBoxIouMatcher on the boxes that followed the crop and the mirror."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(4)
    n = 32
    anchors = S.ssd300_anchors()
    pipe = Pipeline(batch_size=n, device_id=0, seed=9)
    with pipe:
        img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_UNCOMPRESSED, max_width=800, max_height=800)
        c = fn.ssd_random_crop(img)
        r = fn.resize(c, resize_width=300, resize_height=300, scaling_mode=types.SCALING_MODE_STRETCH)
        mirror = fn.random.coin_flip()
        out = fn.crop_mirror_normalize(r, crop=[300, 300], crop_pos_x=0.0, crop_pos_y=0.0, mean=MEAN, std=STD, mirror=mirror,
                                       output_layout=types.NCHW, output_dtype=types.FLOAT)
        fn.box_encoder(anchors=anchors, criteria=0.5, means=[0, 0, 0, 0], stds=[0.1, 0.1, 0.2, 0.2], offset=True, scale=1.0)
        fn.box_iou_matcher(anchors=anchors, high_threshold=0.5, low_threshold=0.4, allow_low_quality_matches=True)
        pipe.set_outputs(out)
    pipe.build()
    for _ in range(2):
        arena, hs, ws, offs = S.make_images(rng, n, (300, 800), (300, 800))
        boxes, labels, boffs = S.random_boxes(rng, n)
        pipe.feed_boxes(boxes, labels, np.diff(boffs))
        pipe.feed_ragged(arena, hs, ws, offs)
        pipe.run()
        win = pipe.get_crop_windows(c)
        m = pipe.get_int_array(mirror)
        # window properties: inside the image, aspect ratio within [0.5, 2] (+ pixel truncation), at least 0.3 of each side
        for i in range(n):
            x, y, w, h = [int(v) for v in win[i]]
            assert x + w <= ws[i] and y + h <= hs[i] and w >= 1 and h >= 1
            if (w, h) != (ws[i], hs[i]):
                assert w >= int(0.3 * ws[i]) - 1 and h >= int(0.3 * hs[i]) - 1
        tab = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
        tab["src_offset"], tab["src_stride"] = offs, ws * 3
        tab["roi_x"], tab["roi_y"], tab["roi_w"], tab["roi_h"] = win[:, 0], win[:, 1], win[:, 2], win[:, 3]
        tab["dst_w"], tab["dst_h"], tab["crop_w"], tab["crop_h"] = 300, 300, 300, 300
        tab["mirror"] = m
        mul, add = S.normalize_tables()
        exp = O.resample(arena, tab, 300, 300, T.FP32, T.NCHW, mul, add)
        assert np.array_equal(pipe.get_output_tensors()[0].numpy(), exp)
        # boxes after crop + mirror, then the encoder on exactly those boxes
        b2, l2, c2 = pipe.get_bounding_boxes()
        assert (c2 >= 1).all() and len(l2) == c2.sum() and b2.min() >= 0.0 and b2.max() <= 1.0
        o2 = np.concatenate([[0], np.cumsum(c2)]).astype(np.int32)
        eb, el = O.box_encode(b2, l2, o2, anchors, 0.5, (0, 0, 0, 0), (0.1, 0.1, 0.2, 0.2), True, 1.0)
        gb, gl = pipe.get_encoded_boxes_and_lables()
        assert np.array_equal(gl, el)
        assert np.allclose(gb, eb, rtol=1e-5, atol=1e-6)
        # rocalBoxIouMatcher on the same boxes
        assert np.array_equal(pipe.get_matched_indices(), O.box_iou_match(b2, o2, anchors, 0.5, 0.4, True))
    pipe.rocal_release()


def test_error_convention(cuda):
    """Errors never escape as C++ exceptions: a null handle returns NULL/CONTEXT_INVALID, a bad argument is
    stored in the context and reported by rocalGetErrorMessage (reference: rocal_api.h:42-62)."""
    import rocal_b200._capi as C
    from rocal_b200 import types
    assert C.verify(None) == types.CONTEXT_INVALID
    assert C.run(None) == types.CONTEXT_INVALID
    assert not C.resize(None, None, 1, 1, 0, 1, 0, 0, 0, 0, 1, 0, 2)
    ctx = C.create(4, types.GPU, 0, 1, 2, types.FLOAT)
    assert ctx
    assert not C.create(4, types.CPU, 0, 1, 2, types.FLOAT)            # no CPU backend
    assert not C.create(4, types.GPU, 999, 1, 2, types.FLOAT)          # no such device
    assert not C.external_source(ctx, types.RGB, 0, 100, 100, 7)                        # no such mode
    assert b"external source mode" in C.get_error_message(ctx)
    assert C.get_status(ctx) == types.RUNTIME_ERROR
    src = C.external_source(ctx, types.RGB, 0, 100, 100, types.EXTSOURCE_RAW_UNCOMPRESSED)
    assert src
    assert not C.resize(ctx, src, 0, 0, 0, 1, 0, 0, 0, 0, 1, 0, 2)     # no size given
    assert b"must be specified" in C.get_error_message(ctx)
    assert not C.resize(ctx, src, 10, 10, 0, 1, 0, 0, 0, 0, 9, 0, 2)                      # no such interpolation type
    assert C.run(ctx) == types.RUNTIME_ERROR                            # not verified
    r = C.resize(ctx, src, 10, 10, 1, 1, 0, 0, 0, 0, 1, 0, 2)
    assert r and C.verify(ctx) == types.OK
    assert C.verify(ctx) == types.RUNTIME_ERROR                         # twice
    assert C.run(ctx) == types.RUNTIME_ERROR                            # nothing fed
    d = (C.ImageDesc * 4)()
    arena = np.zeros(100 * 100 * 3 * 4, dtype=np.uint8)
    assert C.feed_ragged(ctx, arena.ctypes.data, arena.nbytes, d, 4, 0) == types.RUNTIME_ERROR   # empty descriptors
    assert C.feed_ragged(ctx, arena.ctypes.data, arena.nbytes, d, 3, 0) == types.RUNTIME_ERROR   # wrong batch size
    assert C.release(ctx) == types.OK


def _decoded_by_pipeline(streams, max_side):
    """The GPU decoder's own pixels for a list of JPEG streams (identity flip of an encoded external source)."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    n = len(streams)
    pipe = Pipeline(batch_size=n, device_id=0, seed=1)
    with pipe:
        img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_COMPRESSED, max_width=max_side, max_height=max_side)
        pipe.set_outputs(fn.flip(img, horizontal=0, vertical=0))
    pipe.build()
    pipe.feed_encoded(streams)
    full = pipe.run()[0].numpy().copy()          # run() returns the output tensors
    sizes = pipe.get_image_sizes()
    pipe.rocal_release()
    return [np.ascontiguousarray(full[i, :sizes[i, 1], :sizes[i, 0]]) for i in range(n)]


def _expected_windowed_resize(pixels, windows, out_w, out_h, interpolation=0):
    """Oracle resize of window i of image i to out_w x out_h (uint8 NHWC)."""
    n = len(pixels)
    offs = np.concatenate([[0], np.cumsum([p.size for p in pixels])])[:-1]
    arena = np.concatenate([p.reshape(-1) for p in pixels])
    t = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
    for i in range(n):
        x, y, w, h = [int(v) for v in windows[i]]
        stride = pixels[i].shape[1] * 3
        t[i]["src_offset"], t[i]["src_stride"] = offs[i] + y * stride + x * 3, stride
        t[i]["roi_w"], t[i]["roi_h"], t[i]["dst_w"], t[i]["dst_h"] = w, h, out_w, out_h
        t[i]["crop_w"], t[i]["crop_h"] = out_w, out_h
    return O.resample(arena, t, out_w, out_h, T.UINT8, T.NHWC, interpolation=interpolation)


def test_fused_jpeg_crop_external_source(cuda):
    """Random-resized-crop windows on an encoded external source: the windows are the restated sampler's for the
    batch seeds that follow from the pipeline seed, the identity output is exactly that window of the decoded image,
    and Resize of the window (bilinear and triangular) equals the oracle on the decoder's pixels bit for bit."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(31)
    n = 6
    imgs, streams = _jpeg_batch(rng, n, (90, 360))
    pixels = _decoded_by_pipeline(streams, 360)
    shapes = np.array([[p.shape[0], p.shape[1]] for p in pixels])
    area, aspect, attempts = (0.08, 1.0), (0.75, 1.33333), 100
    seed = 77
    for interp, flag in ((types.LINEAR_INTERPOLATION, 0), (types.TRIANGULAR_INTERPOLATION, 1)):
        pipe = Pipeline(batch_size=n, device_id=0, seed=seed)
        with pipe:
            img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_COMPRESSED, max_width=360, max_height=360)
            pipe.set_random_crop_decoder(area, aspect, attempts)
            ident = fn.flip(img, horizontal=0, vertical=0)
            r = fn.resize(img, resize_width=64, resize_height=48, interpolation_type=interp)
            pipe.set_outputs(ident, r)
        pipe.build()
        batch_seeds = O._Mt19937(seed)
        for _ in range(3):
            pipe.feed_encoded(streams)
            pipe.run()
            win, bseed = pipe.get_decoder_crop_windows()
            assert bseed == batch_seeds()
            assert np.array_equal(win, O.random_crop_windows(bseed, shapes, aspect, area, attempts))
            assert pipe.get_image_sizes().tolist() == shapes[:, ::-1].tolist()          # the images as decoded
            assert pipe.get_roi_image_sizes().tolist() == win[:, 2:].tolist()           # what the first output holds
            cut, res = [t.numpy() for t in pipe.get_output_tensors()]
            for i in range(n):
                x, y, w, h = [int(v) for v in win[i]]
                assert x + w <= shapes[i, 1] and y + h <= shapes[i, 0]
                assert np.array_equal(cut[i, :h, :w], pixels[i][y:y + h, x:x + w])
            assert np.array_equal(res, _expected_windowed_resize(pixels, win, 64, 48, flag))
        pipe.rocal_release()


def test_fused_jpeg_crop_file_source(cuda, tmp_path):
    """fn.decoders.image_slice on a folder (rocalFusedJpegCropSingleShard), the train pipeline of the reference's
    imagenet example: image_slice -> Resize(TRIANGULAR) 224 -> CropMirrorNormalize with a coin flip, read through
    ROCALClassificationIterator. Windows follow the sampler, labels the folders, pixels the oracle."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    from rocal_b200.plugin.pytorch import ROCALClassificationIterator
    rng = S.rng_for(32)
    imgs, streams = _jpeg_batch(rng, 6, (100, 320))
    classes = ["a", "a", "b", "b", "c", "c"]
    pixels = dict(zip(["im%d.jpg" % i for i in range(6)], _decoded_by_pipeline(streams, 320)))
    for i, (cls, sb) in enumerate(zip(classes, streams)):
        d = tmp_path / cls
        d.mkdir(exist_ok=True)
        (d / ("im%d.jpg" % i)).write_bytes(sb)
    n, crop = 3, 56
    pipe = Pipeline(batch_size=n, device_id=0, seed=12)
    with pipe:
        jpegs, labels = fn.readers.file(file_root=str(tmp_path))
        dec = fn.decoders.image_slice(jpegs, output_type=types.RGB, file_root=str(tmp_path), shard_id=0, num_shards=1,
                                      random_shuffle=True, max_decoded_width=320, max_decoded_height=320)
        res = fn.resize(dec, resize_width=64, resize_height=64, output_layout=types.NHWC, output_dtype=types.UINT8,
                        interpolation_type=types.TRIANGULAR_INTERPOLATION)
        coin = fn.random.coin_flip(probability=0.5)
        out = fn.crop_mirror_normalize(res, output_layout=types.NCHW, output_dtype=types.FLOAT, crop=(crop, crop), mirror=coin,
                                       mean=MEAN, std=STD)
        pipe.set_outputs(out)
    pipe.build()
    mul, add = S.normalize_tables()
    seen = []
    for outs, labs in ROCALClassificationIterator(pipe):
        names = pipe.get_image_names()
        seen += names
        assert labs.cpu().tolist() == ["abc".index(classes[int(nm[2])]) for nm in names]
        win, bseed = pipe.get_decoder_crop_windows()
        px = [pixels[nm] for nm in names]
        shapes = np.array([[p.shape[0], p.shape[1]] for p in px])
        assert np.array_equal(win, O.random_crop_windows(bseed, shapes, (0.75, 1.33333), (0.08, 1.0), 100))
        resized = _expected_windowed_resize(px, win, 64, 64, 1)
        # the reader runs batches ahead, so the coin flips of this batch are no longer the parameter's current
        # values: every sample must equal the oracle with or without the mirror
        exp = []
        for flag in (0, 1):
            t = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
            for i in range(n):
                x1, y1, cw, ch = O.crop_fixed(64, 64, crop, crop, 0.5, 0.5)
                t[i]["src_offset"], t[i]["src_stride"] = i * 64 * 64 * 3, 64 * 3
                t[i]["roi_w"], t[i]["roi_h"], t[i]["dst_w"], t[i]["dst_h"] = 64, 64, 64, 64
                t[i]["crop_x"], t[i]["crop_y"], t[i]["crop_w"], t[i]["crop_h"], t[i]["mirror"] = x1, y1, cw, ch, flag
            exp.append(O.resample(resized.reshape(-1), t, crop, crop, T.FP32, T.NCHW, mul, add))
        got = outs[0].cpu().numpy()
        for i in range(n):
            assert np.array_equal(got[i], exp[0][i]) or np.array_equal(got[i], exp[1][i]), names[i]
    assert sorted(seen) == sorted(pixels)        # shuffled, every file once
    pipe.rocal_release()


def test_coco_source_behind_the_random_crop_decoder(cuda, tmp_path):
    """fn.decoders.image_slice behind fn.readers.coco (rocalJpegCOCOFileSourcePartialSingleShard): the pixels are cut to
    the sampler's windows, the boxes stay those of the whole image (only a box-aware crop would move them)."""
    import json
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(41)
    n = 3
    imgs, streams = _jpeg_batch(rng, n, (120, 300))
    pixels = _decoded_by_pipeline(streams, 320)
    images, anns, truth = [], [], []
    for i, (im, sb) in enumerate(zip(imgs, streams)):
        name = "c%d.jpg" % i
        (tmp_path / name).write_bytes(sb)
        h, w = im.shape[:2]
        images.append({"id": 7 + i, "file_name": name, "width": w, "height": h})
        x, y, bw, bh = w * 0.1, h * 0.2, w * 0.5, h * 0.4
        anns.append({"id": i, "image_id": 7 + i, "category_id": 5, "bbox": [x, y, bw, bh], "iscrowd": 0})
        truth.append([x / w, y / h, (x + bw) / w, (y + bh) / h])
    (tmp_path / "ann.json").write_text(json.dumps({"images": images, "annotations": anns, "categories": [{"id": 5}]}))
    pipe = Pipeline(batch_size=n, device_id=0, seed=9)
    with pipe:
        jpegs, _, _ = fn.readers.coco(annotations_file=str(tmp_path / "ann.json"), ltrb=True)
        img = fn.decoders.image_slice(jpegs, file_root=str(tmp_path), random_area=[0.2, 0.9], random_aspect_ratio=[0.5, 2.0],
                                      num_attempts=20, max_decoded_width=320, max_decoded_height=320)
        pipe.set_outputs(fn.resize(img, resize_width=64, resize_height=48, scaling_mode=types.SCALING_MODE_STRETCH))
    pipe.build()
    out = pipe.run()[0].numpy()
    assert pipe.get_image_names() == ["c0.jpg", "c1.jpg", "c2.jpg"]
    win, bseed = pipe.get_decoder_crop_windows()
    shapes = np.array([[p.shape[0], p.shape[1]] for p in pixels])
    assert np.array_equal(win, O.random_crop_windows(bseed, shapes, (0.5, 2.0), (0.2, 0.9), 20))
    assert any(int(win[i, 2]) != shapes[i, 1] or int(win[i, 3]) != shapes[i, 0] for i in range(n))
    assert np.array_equal(out, _expected_windowed_resize(pixels, win, 64, 48))
    boxes, labels, counts = pipe.get_bounding_boxes()
    assert list(counts) == [1] * n and list(labels) == [1] * n and np.allclose(boxes, truth, atol=1e-5)
    pipe.rocal_release()


def test_random_crop_crop_resize_roi_resize(cuda):
    """rocalRandomCrop, rocalCropResize, rocalROIResize and rocalNop on raw pixels. With fixed parameter values the
    windows are the restated rule's; with the default random ranges they are read back. Pixels equal the oracle:
    RandomCrop = the window copied, CropResize / ROIResize = the window stretched by the resize kernel."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(41)
    n = 8
    fixed = (0.45, 1.2, 0.3, 0.8)
    pipe = Pipeline(batch_size=n, device_id=0, seed=21)
    with pipe:
        img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_UNCOMPRESSED, max_width=400, max_height=400)
        rc = fn.random_crop(img, crop_area_factor=fixed[0], crop_aspect_ratio=fixed[1], crop_pox_x=fixed[2], crop_pox_y=fixed[3])
        cr_fixed = fn.resize_crop(img, resize_width=96, resize_height=64, crop_area_factor=fixed[0], crop_aspect_ratio=fixed[1],
                                  x_drift=fixed[2], y_drift=fixed[3])
        cr_rand = fn.resize_crop(img, resize_width=80, resize_height=80, output_layout=types.NCHW, output_dtype=types.FLOAT)
        roi = fn.roi_resize(img, resize_width=72, resize_height=56, roi_w=120, roi_h=90, roi_pos_x=17, roi_pos_y=9,
                            interpolation_type=types.CUBIC_INTERPOLATION)
        same = fn.nop(img)
        pipe.set_outputs(rc, cr_fixed, cr_rand, roi, same)
    pipe.build()
    for _ in range(2):
        arena, hs, ws, offs = S.make_images(rng, n, (130, 400), (130, 400))
        pipe.feed_ragged(arena, hs, ws, offs)
        pipe.run()
        o_rc, o_fixed, o_rand, o_roi, o_same = [t.numpy() for t in pipe.get_output_tensors()]
        wh = np.stack([ws, hs], axis=1)
        exp_win = O.random_area_windows(wh, fixed=fixed)
        for t in (rc, cr_fixed):
            assert np.array_equal(pipe.get_crop_windows(t), exp_win)
        win_rand = pipe.get_crop_windows(cr_rand)
        assert (win_rand[:, 0] + win_rand[:, 2] <= ws).all() and (win_rand[:, 1] + win_rand[:, 3] <= hs).all()
        ratio = win_rand[:, 2] / win_rand[:, 3]
        assert (ratio > 0.6).all() and (ratio < 1.6).all()
        win_roi = pipe.get_crop_windows(roi)
        assert win_roi.tolist() == [[17, 9, 120, 90]] * n

        def stretched(win, w, h, dtype, layout, interpolation=0):
            tab = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
            tab["src_offset"], tab["src_stride"] = offs, ws * 3
            tab["roi_x"], tab["roi_y"], tab["roi_w"], tab["roi_h"] = win[:, 0], win[:, 1], win[:, 2], win[:, 3]
            tab["dst_w"], tab["dst_h"], tab["crop_w"], tab["crop_h"] = w, h, w, h
            return O.resample(arena, tab, w, h, dtype, layout, interpolation=interpolation)

        assert np.array_equal(o_fixed, stretched(exp_win, 96, 64, T.UINT8, T.NHWC))
        assert np.array_equal(o_rand, stretched(win_rand, 80, 80, T.FP32, T.NCHW))
        assert np.array_equal(o_roi, stretched(win_roi, 72, 56, T.UINT8, T.NHWC, 2))      # RB200_INTERP_BICUBIC
        for i in range(n):
            ih, iw, o = int(hs[i]), int(ws[i]), int(offs[i])
            im = arena[o:o + ih * iw * 3].reshape(ih, iw, 3)
            x, y, w, h = [int(v) for v in exp_win[i]]
            assert np.array_equal(o_rc[i, :h, :w], im[y:y + h, x:x + w])
            assert np.array_equal(o_same[i, :ih, :iw], im)
        t0 = pipe.get_output_tensors()[0]
        assert t0.roi()[:, 2:].tolist() == exp_win[:, 2:].tolist()
        # the calling forms of the reference's Python binding
        buf, rois = np.empty(t0.dimensions(), dtype=np.uint8), np.zeros((n, 4), dtype=np.uint32)
        t0.copy_data(buf)
        t0.copy_roi(rois)
        assert np.array_equal(buf, o_rc) and rois[:, 2:].tolist() == exp_win[:, 2:].tolist()
        assert t0.batch_size() == n and t0.max_shape() == [n, 400, 400, 3] and t0.roi_dims_size() == 2
    pipe.rocal_release()


def test_one_hot_and_partial_last_batch_iterator(cuda, tmp_path):
    """fn.one_hot makes ROCALClassificationIterator yield one-hot labels; LAST_BATCH_PARTIAL cuts the padding off
    the last batch (plugin/pytorch.py:198-231 of the reference)."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    from rocal_b200.plugin.pytorch import ROCALClassificationIterator
    rng = S.rng_for(42)
    imgs, streams = _jpeg_batch(rng, 5, (64, 128))
    classes = ["a", "a", "b", "c", "c"]
    for i, (cls, sb) in enumerate(zip(classes, streams)):
        d = tmp_path / cls
        d.mkdir(exist_ok=True)
        (d / ("im%d.jpg" % i)).write_bytes(sb)
    pipe = Pipeline(batch_size=2, device_id=0, seed=2)
    with pipe:
        jpegs, labels = fn.readers.file(file_root=str(tmp_path))
        fn.one_hot(labels, num_classes=3)
        dec = fn.decoders.image(jpegs, file_root=str(tmp_path), max_decoded_width=128, max_decoded_height=128,
                                last_batch_policy=types.LAST_BATCH_PARTIAL, pad_last_batch=True)
        pipe.set_outputs(fn.centre_crop(dec, crop=[32, 32]))
    pipe.build()
    sizes, hots = [], []
    for outs, labs in ROCALClassificationIterator(pipe):
        sizes.append(outs[0].shape[0])
        assert labs.shape == (outs[0].shape[0], 3) and labs.is_cuda
        hots += labs.cpu().tolist()
    assert sizes == [2, 2, 1]
    # label k > 0 -> column k-1, label 0 -> last column (rocalGetOneHotImageLabels)
    assert hots == [[0, 0, 1], [0, 0, 1], [1, 0, 0], [0, 1, 0], [0, 1, 0]]
    pipe.rocal_release()


def test_file_list_source(cuda, tmp_path):
    """fn.readers.file(file_list=...): the listed files, in the list's order, with the list's labels."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    from rocal_b200.plugin.pytorch import ROCALClassificationIterator
    rng = S.rng_for(43)
    imgs, streams = _jpeg_batch(rng, 4, (64, 128))
    (tmp_path / "x").mkdir()
    for i, sb in enumerate(streams):
        (tmp_path / "x" / ("im%d.jpg" % i)).write_bytes(sb)
    lst = tmp_path / "train.txt"
    lst.write_text("x/im3.jpg 11\nx/im0.jpg 5\nx/im2.jpg 11\n")
    pipe = Pipeline(batch_size=3, device_id=0, seed=2)
    with pipe:
        jpegs, labels = fn.readers.file(file_root=str(tmp_path), file_list=str(lst))
        dec = fn.decoders.image(jpegs, file_root=str(tmp_path), max_decoded_width=128, max_decoded_height=128)
        pipe.set_outputs(fn.centre_crop(dec, crop=[32, 32]))
    pipe.build()
    got = [(pipe.get_image_names(), labs.cpu().tolist(), pipe.get_image_sizes().tolist()) for _, labs in ROCALClassificationIterator(pipe)]
    assert len(got) == 1
    assert got[0][0] == ["im3.jpg", "im0.jpg", "im2.jpg"] and got[0][1] == [11, 5, 11]
    assert got[0][2] == [[imgs[k].shape[1], imgs[k].shape[0]] for k in (3, 0, 2)]
    pipe.rocal_release()


def test_exposure_gamma_color_temp(cuda):
    """rocalExposure, rocalGamma, rocalColorTemp through the pipeline against the oracle's definitions (x * 2^e;
    255 * (x/255)^gamma; R + adjustment, B - adjustment): exposure and colour temperature are exact, gamma goes through
    powf and may differ by one level."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(44)
    n = 6
    pipe = Pipeline(batch_size=n, device_id=0, seed=5)
    with pipe:
        img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_UNCOMPRESSED, max_width=160, max_height=160)
        e = fn.exposure(img, exposure=0.7)
        g = fn.gamma_correction(img, gamma=2.2)
        c = fn.color_temp(img, adjustment_value=-37)
        cf = fn.color_temp(img, adjustment_value=25, output_layout=types.NCHW, output_dtype=types.FLOAT)
        pipe.set_outputs(e, g, c, cf)
    pipe.build()
    arena, hs, ws, offs = S.make_images(rng, n, (64, 160), (64, 160), content="noise")
    pipe.feed_ragged(arena, hs, ws, offs)
    pipe.run()
    oe, og, oc, ocf = [t.numpy() for t in pipe.get_output_tensors()]

    def expected(op, alpha=1.0, beta=0.0, hue=0.0, dtype=T.UINT8, layout=T.NHWC):
        t = np.zeros(n, dtype=T.POINTWISE_SAMPLE)
        t["src_offset"], t["src_stride"], t["roi_w"], t["roi_h"] = offs, ws * 3, ws, hs
        t["alpha"], t["beta"], t["hue"], t["sat"] = alpha, beta, hue, 1.0
        return O.pointwise(arena, t, 160, 160, color_op=op, out_dtype=dtype, out_layout=layout, fill_padding=False)

    def same_inside(got, exp, tol=0):
        for i in range(n):
            a = got[i, :hs[i], :ws[i]].astype(np.int32) if got.ndim == 4 and got.shape[-1] == 3 else got[i, :, :hs[i], :ws[i]]
            b = exp[i, :hs[i], :ws[i]].astype(np.int32) if exp.ndim == 4 and exp.shape[-1] == 3 else exp[i, :, :hs[i], :ws[i]]
            assert np.abs(a - b).max() <= tol, i

    same_inside(oe, expected(T.COLOR_BRIGHTNESS, alpha=float(np.exp2(np.float32(0.7)))))
    same_inside(oc, expected(T.COLOR_BRIGHTNESS, hue=-37.0))
    same_inside(ocf, expected(T.COLOR_BRIGHTNESS, hue=25.0, dtype=T.FP32, layout=T.NCHW))
    same_inside(og, expected(T.COLOR_GAMMA, alpha=2.2), tol=1)
    # what the definitions mean on a pixel
    i0 = arena[int(offs[0]):int(offs[0]) + 3].astype(np.int32)
    assert oc[0, 0, 0].tolist() == [max(0, i0[0] - 37), i0[1], min(255, i0[2] + 37)]
    pipe.rocal_release()


def test_blend_two_inputs(cuda):
    """rocalBlend: a node with two inputs - the source with its own flipped copy, and two colour operators of the
    source - against the oracle's blend (alpha*x + (1-alpha)*x2, rounded)."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(45)
    n = 5
    pipe = Pipeline(batch_size=n, device_id=0, seed=6)
    with pipe:
        img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_UNCOMPRESSED, max_width=120, max_height=100)
        flipped = fn.flip(img, horizontal=1, vertical=0)
        bright = fn.brightness(img, brightness=1.4, brightness_shift=10.0)
        b1 = fn.blend(img, flipped, ratio=0.3)
        b2 = fn.blend(bright, flipped, ratio=0.75, output_layout=types.NCHW, output_dtype=types.FLOAT)
        pipe.set_outputs(b1, b2, flipped, bright)
    pipe.build()
    # same-sized images: the flipped copy then covers the same window as the source
    arena, hs, ws, offs = S.make_images(rng, n, (100, 100), (120, 120), content="noise")
    pipe.feed_ragged(arena, hs, ws, offs)
    pipe.run()
    o1, o2, ofl, obr = [t.numpy() for t in pipe.get_output_tensors()]
    src = np.stack([arena[int(o):int(o) + 100 * 120 * 3].reshape(100, 120, 3) for o in offs])
    assert np.array_equal(ofl, src[:, :, ::-1])

    def blend(a, b, ratio):
        r = np.float32(ratio)
        v = r * a.astype(np.float32) + np.float32(np.float32(1.0) - r) * b.astype(np.float32)
        return np.clip(np.rint(v), 0, 255)

    assert np.array_equal(o1, blend(src, ofl, 0.3).astype(np.uint8))
    assert np.array_equal(o2, blend(obr, ofl, 0.75).transpose(0, 3, 1, 2).astype(np.float32))
    pipe.rocal_release()


def test_pipeline_stress_mixed_memory_kinds(cuda):
    """Twenty batches through one pipeline with a prefetch queue: pageable, pinned (read in place by the kernel) and
    device arenas in turn, image sizes that grow and shrink between batches (the input arenas are reallocated and
    reused), two batches in flight at a time; every result equals the oracle and comes back in feed order."""
    import torch
    from rocal_b200 import types
    rng = S.rng_for(46)
    n = 8
    pipe, out, mirror = _classification_pipeline(n, types.FLOAT, max_side=640, seed=13, depth=3)
    pending = []

    def feed(k):
        hi = int(rng.choice([300, 420, 640]))
        arena, hs, ws, offs = S.make_images(rng, n, (256, hi), (256, hi))
        ax, ay = rng.random(n).astype(np.float32), rng.random(n).astype(np.float32)
        pipe.set_crop_anchors(out, ax, ay)
        fed = [arena, torch.from_numpy(arena).pin_memory(), torch.from_numpy(arena).to(cuda)][k % 3]
        pipe.feed_ragged(fed, hs, ws, offs)
        pending.append((arena, hs, ws, offs, ax, ay, fed))

    feed(0)
    feed(1)
    for k in range(20):
        if k + 2 < 20:
            feed(k + 2)
        pipe.run()
        arena, hs, ws, offs, ax, ay, _ = pending.pop(0)
        got = pipe.get_output_tensors()[0].numpy()
        # the coin flips of this batch are no longer the parameter's current values (batches run ahead): every
        # sample must equal the oracle with or without the mirror
        e0 = _expected_classification(arena, hs, ws, offs, ax, ay, np.zeros(n, np.int32), T.FP32)
        e1 = _expected_classification(arena, hs, ws, offs, ax, ay, np.ones(n, np.int32), T.FP32)
        for i in range(n):
            assert np.array_equal(got[i], e0[i]) or np.array_equal(got[i], e1[i]), (k, i)
    assert pipe.is_empty()
    pipe.rocal_release()


def test_imagenet_style_train_and_val_pipelines(cuda, tmp_path):
    """The keyword arguments a training script written for amd.rocal passes (Pipeline(... rocal_cpu, tensor_dtype,
    tensor_layout, prefetch_queue_depth, mean, std, output_memory_type), decoders.image_slice / decoders.image with their
    sharding arguments, resize with TRIANGULAR interpolation and SCALING_MODE_NOT_SMALLER, crop_mirror_normalize with a
    coin flip, ROCALClassificationIterator(pipe, device=..., device_id=...)) are all accepted, and both loaders deliver
    every file of the folder once per epoch with the folder's labels."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    import torch
    from rocal_b200.plugin.pytorch import ROCALClassificationIterator
    rng = S.rng_for(47)
    imgs, streams = _jpeg_batch(rng, 6, (260, 420))
    for split in ("train", "val"):
        for i, sb in enumerate(streams):
            d = tmp_path / split / ("n%02d" % (i % 3))
            d.mkdir(parents=True, exist_ok=True)
            (d / ("img_%d.JPEG" % i)).write_bytes(sb)
    mean, std = [0.485 * 255, 0.456 * 255, 0.406 * 255], [0.229 * 255, 0.224 * 255, 0.225 * 255]
    common = dict(batch_size=2, num_threads=4, device_id=0, seed=10, rocal_cpu=False, tensor_dtype=types.FLOAT,
                  tensor_layout=types.NCHW, prefetch_queue_depth=6, mean=mean, std=std, output_memory_type=types.DEVICE_MEMORY)

    train = Pipeline(**common)
    with train:
        jpegs, labels = fn.readers.file(file_root=str(tmp_path / "train"))
        dec = fn.decoders.image_slice(jpegs, output_type=types.RGB, file_root=str(tmp_path / "train"), shard_id=0, num_shards=1,
                                      random_shuffle=True, max_decoded_width=500, max_decoded_height=500)
        res = fn.resize(dec, resize_width=224, resize_height=224, output_layout=types.NHWC, output_dtype=types.UINT8,
                        interpolation_type=types.TRIANGULAR_INTERPOLATION)
        out = fn.crop_mirror_normalize(res, output_layout=types.NCHW, output_dtype=types.FLOAT, crop=(224, 224),
                                       mirror=fn.random.coin_flip(probability=0.5), mean=mean, std=std)
        train.set_outputs(out)
    train.build()

    val = Pipeline(**common)
    with val:
        jpegs, labels = fn.readers.file(file_root=str(tmp_path / "val"))
        dec = fn.decoders.image(jpegs, file_root=str(tmp_path / "val"), max_decoded_width=500, max_decoded_height=500,
                                output_type=types.RGB, shard_id=0, num_shards=1, random_shuffle=False)
        res = fn.resize(dec, resize_shorter=256, scaling_mode=types.SCALING_MODE_NOT_SMALLER,
                        interpolation_type=types.TRIANGULAR_INTERPOLATION, output_layout=types.NHWC, output_dtype=types.UINT8)
        out = fn.crop_mirror_normalize(res, output_layout=types.NCHW, output_dtype=types.FLOAT, crop=(224, 224), mirror=0,
                                       mean=mean, std=std)
        val.set_outputs(out)
    val.build()

    for pipe in (train, val):
        loader = ROCALClassificationIterator(pipe, device="cuda", device_id=0)
        for epoch in range(2):
            seen = []
            for (batch,), target in loader:
                assert batch.is_cuda and batch.shape == (2, 3, 224, 224) and batch.dtype == torch.float32
                assert target.shape == (2,) and bool(torch.isfinite(batch).all())
                names = pipe.get_image_names()
                assert target.cpu().tolist() == [int(nm.split("_")[1].split(".")[0]) % 3 for nm in names]
                seen += names
            assert sorted(seen) == sorted("img_%d.JPEG" % i for i in range(6))
            loader.reset()
        pipe.rocal_release()


def test_pipeline_def_and_generic_iterator(cuda, tmp_path):
    """@pipeline_def builds a Pipeline from a graph function (decorator arguments, call-time overrides, the function's
    own arguments), and plugin.generic.ROCALClassificationIterator hands the batches out as numpy arrays."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import pipeline_def
    from rocal_b200.plugin.generic import ROCALClassificationIterator
    rng = S.rng_for(48)
    imgs, streams = _jpeg_batch(rng, 4, (100, 160))
    for i, sb in enumerate(streams):
        d = tmp_path / ("c%d" % (i // 2))
        d.mkdir(exist_ok=True)
        (d / ("f%d.jpg" % i)).write_bytes(sb)

    @pipeline_def(seed=3, batch_size=4)
    def loader(path, crop=48):
        jpegs, labels = fn.readers.file(file_root=path)
        images = fn.decoders.image(jpegs, file_root=path, max_decoded_width=160, max_decoded_height=160)
        images = fn.resize(images, resize_shorter=64, scaling_mode=types.SCALING_MODE_NOT_SMALLER)
        return fn.centre_crop(images, crop=(crop, crop))

    with pytest.raises(TypeError):
        loader(str(tmp_path), no_such_argument=1)
    pipe = loader(str(tmp_path), crop=40, batch_size=2, device_id=0)
    pipe.build()
    got = [(outs[0].shape, outs[0].dtype, labels.tolist()) for outs, labels in ROCALClassificationIterator(pipe, device="cpu")]
    assert [g[2] for g in got] == [[0, 0], [1, 1]]
    assert all(g[0] == (2, 40, 40, 3) and g[1] == np.uint8 for g in got)
    pipe.rocal_release()

"""Operators of the augmentation path through the rocAL-facing API (rocal_b200.fn over the rb200_* C-ABI) with
per-sample random parameters: ResizeCropMirror, Contrast, Hue, Saturation, Crop / CropFixed / CropCenterFixed, and
bounding boxes that follow crops, mirrors, flips and resizes. Expected tables are rebuilt here from the parameters
read back from the pipeline; pixels are compared bit for bit with the oracle, boxes with the restatements of the
reference's meta nodes."""
import numpy as np
import pytest

from oracle import pyoracle as O
import synthetic as S
from rocal_b200 import tables as T

pytestmark = pytest.mark.gpu


def _source(max_w, max_h):
    from rocal_b200 import fn, types
    img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_UNCOMPRESSED, max_width=max_w, max_height=max_h)
    return img


def _pointwise_table(hs, ws, offs):
    t = np.zeros(len(hs), dtype=T.POINTWISE_SAMPLE)
    t["src_offset"], t["src_stride"], t["roi_w"], t["roi_h"] = offs, ws * 3, ws, hs
    t["alpha"], t["sat"] = 1.0, 1.0
    return t


def _valid_equal(got, exp, ws, hs):
    for i in range(len(ws)):
        assert np.array_equal(got[i, :hs[i], :ws[i]], exp[i, :hs[i], :ws[i]]), "sample %d" % i


def test_contrast_hue_saturation_random_parameters(cuda):
    """rocalContrast / rocalHue / rocalSaturation with uniform random parameters, three outputs of one graph; ragged
    image sizes inside max-shape outputs."""
    from rocal_b200 import fn
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(30)
    n = 24
    pipe = Pipeline(batch_size=n, device_id=0, seed=13)
    with pipe:
        img = _source(300, 260)
        cf, cc = fn.random.uniform(range=(0.2, 1.9)), fn.random.uniform(range=(60.0, 90.0))
        hu = fn.random.uniform(range=(-359.0, 359.0))
        sa = fn.random.uniform(range=(0.0, 2.0))
        o_c = fn.contrast(img, contrast=cf, contrast_center=cc)
        o_h = fn.hue(img, hue=hu)
        o_s = fn.saturation(img, saturation=sa)
        pipe.set_outputs(o_c, o_h, o_s)
    pipe.build()
    for _ in range(2):
        arena, hs, ws, offs = S.make_images(rng, n, (40, 260), (40, 300))
        pipe.feed_ragged(arena, hs, ws, offs)
        pipe.run()
        t_c, t_h, t_s = pipe.get_output_tensors()
        tab = _pointwise_table(hs, ws, offs)
        tab["alpha"], tab["beta"] = pipe.get_float_array(cf), pipe.get_float_array(cc)
        assert len(np.unique(tab["alpha"])) > n // 2 and tab["beta"].min() >= 60.0
        _valid_equal(t_c.numpy(), O.pointwise(arena, tab, 300, 260, T.COLOR_CONTRAST), ws, hs)
        tab = _pointwise_table(hs, ws, offs)
        tab["hue"] = pipe.get_float_array(hu)
        assert tab["hue"].min() < -30 and tab["hue"].max() > 30
        _valid_equal(t_h.numpy(), O.pointwise(arena, tab, 300, 260, T.COLOR_TWIST), ws, hs)
        tab = _pointwise_table(hs, ws, offs)
        tab["sat"] = pipe.get_float_array(sa)
        _valid_equal(t_s.numpy(), O.pointwise(arena, tab, 300, 260, T.COLOR_TWIST), ws, hs)
        assert t_c.roi()[:, 2:].tolist() == np.stack([ws, hs], 1).tolist()
    pipe.rocal_release()


def test_resize_crop_mirror_and_crops(cuda):
    """rocalResizeCropMirrorFixed (a 200 x 160 corner stretched to 320 x 240, coin-flip mirror), rocalCropFixed at an
    absolute corner, rocalCropCenterFixed and the random rocalCrop: windows against RocalCropParam's rule, pixels
    against the oracle, output ROIs."""
    from rocal_b200 import fn
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(31)
    n = 16
    pipe = Pipeline(batch_size=n, device_id=0, seed=17)
    with pipe:
        img = _source(400, 360)
        mirror = fn.random.coin_flip()
        o_rcm = fn.resize_crop_mirror(img, resize_width=320, resize_height=240, crop_w=200, crop_h=160, mirror=mirror)
        o_fix = fn.crop(img, crop=[150, 180], crop_pos_x=37, crop_pos_y=21)
        o_ctr = fn.center_crop(img, crop=[224, 224])
        o_rnd = fn.crop(img)
        pipe.set_outputs(o_rcm, o_fix, o_ctr, o_rnd)
    pipe.build()
    for _ in range(2):
        arena, hs, ws, offs = S.make_images(rng, n, (120, 360), (140, 400))
        pipe.feed_ragged(arena, hs, ws, offs)
        pipe.run()
        wh = np.stack([ws, hs], axis=1)
        t_rcm, t_fix, t_ctr, t_rnd = pipe.get_output_tensors()
        m = pipe.get_int_array(mirror)
        assert set(np.unique(m)) == {0, 1}
        # ResizeCropMirror: window (0, 0, 200, 160) clipped to the image -> 320 x 240 -> mirror
        win = O.rocal_crop_windows(wh, 1, 200, 160, (0, 0)).astype(np.int64)
        got_win = pipe.get_crop_windows(o_rcm).astype(np.int64)
        eff = np.stack([win[:, 0], win[:, 1], win[:, 4] - win[:, 0], win[:, 5] - win[:, 1]], 1)
        assert np.array_equal(got_win, eff)
        tab = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
        tab["src_offset"], tab["src_stride"] = offs, ws * 3
        tab["roi_x"], tab["roi_y"], tab["roi_w"], tab["roi_h"] = eff[:, 0], eff[:, 1], eff[:, 2], eff[:, 3]
        tab["dst_w"], tab["dst_h"], tab["crop_w"], tab["crop_h"], tab["mirror"] = 320, 240, 320, 240, m
        assert np.array_equal(t_rcm.numpy(), O.resample(arena, tab, 320, 240, T.UINT8, T.NHWC))
        assert t_rcm.roi()[:, 2:].tolist() == [[320, 240]] * n
        # fixed corner, centre and random crops: pure indexing
        for t_out, handle, expect in ((t_fix, o_fix, O.rocal_crop_windows(wh, 1, 180, 150, (37, 21))),
                                      (t_ctr, o_ctr, O.rocal_crop_windows(wh, 0, 224, 224, (0.5, 0.5))),
                                      (t_rnd, o_rnd, None)):
            got_win = pipe.get_crop_windows(handle).astype(np.int64)
            if expect is not None:
                e = expect.astype(np.int64)
                assert np.array_equal(got_win, np.stack([e[:, 0], e[:, 1], e[:, 4] - e[:, 0], e[:, 5] - e[:, 1]], 1))
            else:   # width and height factors in 0.55 .. 0.95 of the image, inside it
                assert (got_win[:, 2] >= (0.55 * ws).astype(np.int64) - 1).all() and (got_win[:, 2] <= ws).all()
                assert (got_win[:, 0] + got_win[:, 2] <= ws).all() and (got_win[:, 1] + got_win[:, 3] <= hs).all()
            pix = t_out.numpy()
            for i in range(n):
                x, y, w, h = [int(v) for v in got_win[i]]
                im = arena[int(offs[i]):int(offs[i]) + int(hs[i]) * int(ws[i]) * 3].reshape(hs[i], ws[i], 3)
                assert np.array_equal(pix[i, :h, :w], im[y:y + h, x:x + w]), i
            assert t_out.roi()[:, 2:].tolist() == got_win[:, 2:].tolist()
    pipe.rocal_release()


def _boxes_px(boxes, boffs, wh):
    rep = np.repeat(wh, np.diff(boffs), axis=0).astype(np.float32)
    return (np.asarray(boxes, dtype=np.float32) * np.concatenate([rep, rep], 1)).astype(np.float32)


def _compare_boxes(pipe, exp_b, exp_l, exp_o, norm_wh):
    b, l, c = pipe.get_bounding_boxes()
    o = np.concatenate([[0], np.cumsum(c)]).astype(np.int32)
    assert o.tolist() == exp_o.tolist()
    assert l.tolist() == exp_l.tolist()
    rep = np.repeat(np.asarray(norm_wh, dtype=np.float32), np.diff(exp_o), axis=0)
    assert np.allclose(b, exp_b / np.concatenate([rep, rep], 1), atol=3e-6)
    return int((exp_l > 0).sum())


def test_boxes_follow_crop_mirror_flip_resize(cuda):
    """Boxes through Crop -> Flip(h, v) -> ResizeCropMirror -> Resize, against the restatements of CropMetaNode,
    FlipMetaNode, ResizeCropMirrorMetaNode and ResizeMetaNode chained in pixel coordinates (the pipeline keeps
    boxes normalised to the current image, so its output is compared after division by the final size)."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(32)
    n = 24
    pipe = Pipeline(batch_size=n, device_id=0, seed=19)
    with pipe:
        img = _source(500, 500)
        c = fn.crop(img, crop=[260, 300], crop_pos_x=40, crop_pos_y=30)
        hf, vf = fn.random.coin_flip(), fn.random.coin_flip()
        f = fn.flip(c, horizontal=hf, vertical=vf)
        mirror = fn.random.coin_flip()
        r = fn.resize_crop_mirror(f, resize_width=200, resize_height=150, crop_w=180, crop_h=170, mirror=mirror)
        out = fn.resize(r, resize_width=128, resize_height=96, scaling_mode=types.SCALING_MODE_STRETCH)
        pipe.set_outputs(out)
    pipe.build()
    kept = 0
    for _ in range(2):
        arena, hs, ws, offs = S.make_images(rng, n, (200, 500), (200, 500))
        boxes, labels, boffs = S.random_boxes(rng, n, (1, 20))
        pipe.feed_boxes(boxes, labels, np.diff(boffs))
        pipe.feed_ragged(arena, hs, ws, offs)
        pipe.run()
        wh = np.stack([ws, hs], axis=1)
        w1 = pipe.get_crop_windows(c).astype(np.int64)
        b, l, o = O.meta_crop(_boxes_px(boxes, boffs, wh), labels, boffs, w1)
        b, l, o = O.meta_flip(b, l, o, w1[:, 2:], pipe.get_int_array(hf), pipe.get_int_array(vf))
        w2 = pipe.get_crop_windows(r).astype(np.int64)
        e2 = O.rocal_crop_windows(w1[:, 2:], 1, 180, 170, (0, 0)).astype(np.int64)
        assert np.array_equal(w2, np.stack([e2[:, 0], e2[:, 1], e2[:, 4] - e2[:, 0], e2[:, 5] - e2[:, 1]], 1))
        b, l, o = O.meta_crop(b, l, o, w2, mirror=pipe.get_int_array(mirror), resize_to=(200, 150))
        b, l, o = O.meta_resize(b, l, o, [(200, 150)] * n, [(128, 96)] * n)
        kept += _compare_boxes(pipe, b, l, o, [(128, 96)] * n)
        assert pipe.get_output_tensors()[0].dims() == [n, 96, 128, 3]
    assert kept > 40
    pipe.rocal_release()


def test_boxes_follow_ssd_crop(cuda):
    """configs[4]'s metadata path: the boxes behind rocalSSDRandomCrop -> Resize(300 x 300) -> CropMirrorNormalize
    against the reference's update_random_bbox_meta_data (pinned restatement: centre strictly inside, clip, shift)
    re-normalised to the window, then the CropMirrorNormalize meta node; the encoder then runs on those boxes."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(33)
    n = 32
    anchors = S.ssd300_anchors()
    pipe = Pipeline(batch_size=n, device_id=0, seed=23)
    with pipe:
        img = _source(800, 800)
        c = fn.ssd_random_crop(img)
        r = fn.resize(c, resize_width=300, resize_height=300, scaling_mode=types.SCALING_MODE_STRETCH)
        mirror = fn.random.coin_flip()
        out = fn.crop_mirror_normalize(r, crop=[300, 300], crop_pos_x=0.0, crop_pos_y=0.0, mean=list(S.MEAN), std=list(S.STD),
                                       mirror=mirror, output_layout=types.NCHW, output_dtype=types.FLOAT)
        fn.box_encoder(anchors=anchors, criteria=0.5, means=[0, 0, 0, 0], stds=[0.1, 0.1, 0.2, 0.2], offset=True, scale=1.0)
        pipe.set_outputs(out)
    pipe.build()
    kept = 0
    for _ in range(2):
        arena, hs, ws, offs = S.make_images(rng, n, (300, 800), (300, 800))
        boxes, labels, boffs = S.random_boxes(rng, n)
        pipe.feed_boxes(boxes, labels, np.diff(boffs))
        pipe.feed_ragged(arena, hs, ws, offs)
        pipe.run()
        win = pipe.get_crop_windows(c).astype(np.float32)
        # the window as fractions of the image, a 1 x 1 "decoded size": the function then works on normalised boxes
        frac = np.stack([win[:, 0] / ws, win[:, 1] / hs, (win[:, 0] + win[:, 2]) / ws - win[:, 0] / ws,
                         (win[:, 1] + win[:, 3]) / hs - win[:, 1] / hs], 1).astype(np.float32)
        b, l, o = O.random_bbox_meta(boxes, labels, boffs, frac, np.ones((n, 2), np.uint32))
        rep = np.repeat(frac[:, 2:], np.diff(o), axis=0)
        b = (b / np.concatenate([rep, rep], 1)).astype(np.float32)          # re-normalised to the window
        # CropMirrorNormalize over the whole 300 x 300 image: every box is kept, mirrored where the flag is set
        b, l, o = O.meta_crop(b * 300.0, l, o, [(0, 0, 300, 300)] * n, mirror=pipe.get_int_array(mirror))
        kept += _compare_boxes(pipe, b, l, o, [(300, 300)] * n)
        gb, gl, gc = pipe.get_bounding_boxes()
        eb, el = O.box_encode(gb, gl, np.concatenate([[0], np.cumsum(gc)]).astype(np.int32), anchors, 0.5, (0, 0, 0, 0),
                              (0.1, 0.1, 0.2, 0.2), True, 1.0)
        xb, xl = pipe.get_encoded_boxes_and_lables()
        assert np.array_equal(xl, el) and np.allclose(xb, eb, rtol=1e-5, atol=1e-6)
    assert kept > 100
    pipe.rocal_release()


def test_boxes_follow_rotate(cuda):
    """Boxes behind rocalRotate against the restatement of RotateMetaNode (corners rotated about the image centres,
    bounding box with its left / top edge taken as min(0, .), quarter-area rule, clip to the destination)."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(38)
    n = 16
    pipe = Pipeline(batch_size=n, device_id=0, seed=41)
    with pipe:
        img = _source(400, 300)
        angle = fn.random.uniform(range=(-60.0, 60.0))
        pipe.set_outputs(fn.rotate(img, angle=angle, dest_width=320, dest_height=256))
    pipe.build()
    kept = 0
    for _ in range(3):
        arena, hs, ws, offs = S.make_images(rng, n, (120, 300), (160, 400))
        boxes, labels, boffs = S.random_boxes(rng, n, (0, 8))
        pipe.feed_boxes(boxes, labels, np.diff(boffs))
        pipe.feed_ragged(arena, hs, ws, offs)
        pipe.run()
        rep = np.repeat(np.stack([ws, hs], 1).astype(np.float32), np.diff(boffs), axis=0)
        px = (boxes * np.concatenate([rep, rep], 1)).astype(np.float32)
        b, l, o = O.meta_rotate(px, labels, boffs, np.stack([ws, hs], 1), pipe.get_float_array(angle), 320, 256)
        kept += _compare_boxes(pipe, b, l, o, [(320, 256)] * n)
    assert kept > 30
    pipe.rocal_release()


def test_random_bbox_crop_cuts_images_and_boxes(cuda):
    """rocalRandomBBoxCrop on an external source, fed three ways (packed host arena, pinned arena read in place,
    max-size slots): the sampled windows are the pinned restatement's (the sampler's counter runs on across batches),
    their pixel form is the fused decoder's rounding, the pixels behind a Resize are the oracle's resize of that
    window, and the boxes follow by the centre rule of update_random_bbox_meta_data."""
    import torch
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(36)
    n = 16
    seed = 4321
    pipe = Pipeline(batch_size=n, device_id=0, seed=31)
    with pipe:
        img = _source(640, 480)
        ret = fn.random_bbox_crop(img, all_boxes_above_threshold=False, seed=seed)
        assert ret[1:] == ([], [], [])
        pipe.set_outputs(fn.resize(img, resize_width=96, resize_height=64, scaling_mode=types.SCALING_MODE_STRETCH))
    pipe.build()
    sampler = O.BBoxCropSampler(seed, False)
    cropped = kept = 0
    for mode in ("arena", "pinned", "slots"):
        arena, hs, ws, offs = S.make_images(rng, n, (100, 480), (100, 640))
        boxes, labels, boffs = S.random_boxes(rng, n)
        pipe.feed_boxes(boxes, labels, np.diff(boffs))
        if mode == "slots":
            pipe.feed_input([arena[int(offs[i]):int(offs[i]) + int(hs[i]) * int(ws[i]) * 3].reshape(int(hs[i]), int(ws[i]), 3)
                             for i in range(n)])
        elif mode == "pinned":
            pipe.feed_ragged(torch.from_numpy(arena).pin_memory(), hs, ws, offs)
        else:
            pipe.feed_ragged(arena, hs, ws, offs)
        out = pipe.run()[0].numpy()
        frac = pipe.get_bbox_crop_windows()
        assert np.array_equal(frac, sampler.windows(boxes, boffs, ws)), mode
        win, _ = pipe.get_decoder_crop_windows()
        exp_win = np.zeros((n, 4), dtype=np.int64)
        for i in range(n):
            W, H = int(ws[i]), int(hs[i])
            x, y = min(O._lround_f32(frac[i, 0] * np.float32(W)), W - 1), min(O._lround_f32(frac[i, 1] * np.float32(H)), H - 1)
            exp_win[i] = (x, y, max(1, min(O._lround_f32(frac[i, 2] * np.float32(W)), W - x)),
                          max(1, min(O._lround_f32(frac[i, 3] * np.float32(H)), H - y)))
        assert np.array_equal(win.astype(np.int64), exp_win), mode
        assert np.array_equal(pipe.get_image_sizes(), np.stack([ws, hs], 1)), mode    # the images the windows were cut from
        cropped += int((win[:, 2] < ws).sum())
        t = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
        t["src_stride"] = ws.astype(np.int64) * 3
        t["src_offset"] = offs + win[:, 1].astype(np.int64) * t["src_stride"] + win[:, 0].astype(np.int64) * 3
        t["roi_w"], t["roi_h"], t["dst_w"], t["dst_h"], t["crop_w"], t["crop_h"] = win[:, 2], win[:, 3], 96, 64, 96, 64
        assert np.array_equal(out, O.resample(arena, t, 96, 64, T.UINT8, T.NHWC)), mode
        wf = win.astype(np.float32)
        pf = np.stack([wf[:, 0] / ws, wf[:, 1] / hs, (wf[:, 0] + wf[:, 2]) / ws - wf[:, 0] / ws,
                       (wf[:, 1] + wf[:, 3]) / hs - wf[:, 1] / hs], 1).astype(np.float32)
        b, l, o = O.random_bbox_meta(boxes, labels, boffs, pf, np.ones((n, 2), np.uint32))
        rep = np.repeat(pf[:, 2:], np.diff(o), axis=0)
        kept += _compare_boxes(pipe, (b / np.concatenate([rep, rep], 1)).astype(np.float32), l, o, [(1, 1)] * n)
    assert cropped > 20 and kept > 40
    pipe.rocal_release()


def test_per_launch_device_timing(cuda):
    """Profiling on: the upload and every launch of a batch are bracketed by CUDA events; the accumulated device times
    come back by step, in plan order, once per returned batch."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(37)
    n = 32
    pipe = Pipeline(batch_size=n, device_id=0, seed=3)
    with pipe:
        img = _source(500, 400)
        r = fn.resize(img, resize_width=224, resize_height=224, scaling_mode=types.SCALING_MODE_STRETCH)
        b = fn.brightness(r, brightness=1.1, brightness_shift=3.0)
        pipe.set_outputs(fn.rotate(b, angle=10.0))
        pipe.set_profiling(True)
    pipe.build()
    assert pipe.step_timing()[0][2] == 0
    for _ in range(6):
        arena, hs, ws, offs = S.make_images(rng, n, (200, 400), (300, 500))
        pipe.feed_ragged(arena, hs, ws, offs)
        pipe.run()
    t = pipe.step_timing()
    assert [x[0] for x in t] == ["upload", "resample", "pointwise", "warp_affine"]
    for name, us, batches in t:
        assert batches == 6 and 0.5 < us < 50000.0, t
    info = pipe.timing_info()
    assert info is not None
    pipe.rocal_release()


def test_normalize_and_transpose_through_the_api(cuda):
    """rocalNormalize with computed per-channel statistics, with given statistics, and per-image statistics behind a
    crop; rocalTranspose HWC -> CHW and the height / width swap. Four outputs of one graph against the oracle."""
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    rng = S.rng_for(34)
    n = 12
    pipe = Pipeline(batch_size=n, device_id=0, seed=29)
    with pipe:
        img = _source(200, 160)
        o_stat = fn.normalize(img, axes=[0, 1])                                             # per-channel mean / stddev, computed
        o_given = fn.normalize(img, mean=list(S.MEAN), stddev=list(S.STD), scale=2.0, shift=0.5, output_datatype=types.FLOAT16)
        c = fn.crop(img, crop=[64, 96], crop_pos_x=10, crop_pos_y=5)
        o_img = fn.normalize(c, axes=[0, 1, 2], stddev=[50.0])                              # per-image mean, given deviation
        o_chw = fn.transpose(img, perm=[2, 0, 1])
        o_swap = fn.transpose(c, perm=[1, 0, 2])
        pipe.set_outputs(o_stat, o_given, o_img, o_chw, o_swap)
    pipe.build()
    for _ in range(2):
        arena, hs, ws, offs = S.make_images(rng, n, (70, 160), (100, 200))
        pipe.feed_ragged(arena, hs, ws, offs)
        pipe.run()
        t_stat, t_given, t_img, t_chw, t_swap = pipe.get_output_tensors()
        tab = _pointwise_table(hs, ws, offs)
        assert np.array_equal(t_stat.numpy(), O.normalize(arena, tab, 200, 160, axis_mask=3))
        exp = O.normalize(arena, tab, 200, 160, mean=S.MEAN, stddev=S.STD, scale=2.0, shift=0.5, out_dtype=T.FP16)
        assert np.array_equal(t_given.numpy().view(np.uint16), exp.view(np.uint16))
        win = pipe.get_crop_windows(c).astype(np.int64)
        ctab = _pointwise_table(hs, ws, offs)
        ctab["roi_x"], ctab["roi_y"], ctab["roi_w"], ctab["roi_h"] = win[:, 0], win[:, 1], win[:, 2], win[:, 3]
        assert np.array_equal(t_img.numpy(), O.normalize(arena, ctab, 96, 64, axis_mask=7, stddev=(50.0, 50.0, 50.0)))
        assert t_chw.dims() == [n, 3, 160, 200] and t_swap.dims() == [n, 96, 64, 3]
        assert np.array_equal(t_chw.numpy(), O.transpose(arena, tab, (2, 0, 1), (3, 160, 200)))
        assert np.array_equal(t_swap.numpy(), O.transpose(arena, ctab, (1, 0, 2), (96, 64, 3)))
    pipe.rocal_release()

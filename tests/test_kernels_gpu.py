"""Parity of the CUDA kernels (called through the C-ABI) with the CPU oracle on seeded inputs.

Tolerances (stated by the task): bit-exact for indexing ops and uint8 paths computed with the
same operation order; <= 1 LSB for uint8 in general; 1e-5 relative for fp32; 1e-3 for fp16.
The kernels are written to reproduce the oracle's operation order, so most checks are exact.
"""

import numpy as np
import pytest

from oracle import pyoracle as O
import synthetic as S
from rocal_b200 import tables as T

pytestmark = pytest.mark.gpu


def _device_status():
    from rocal_b200._lib import lib
    return lib.rb200k_device_status()


def _dev(arena, cuda):
    import torch
    return torch.from_numpy(arena).to(cuda)


def _assert_fp(gpu, ref, rel, what):
    gpu = gpu.astype(np.float64)
    ref = ref.astype(np.float64)
    err = np.abs(gpu - ref)
    tol = rel * np.maximum(np.abs(ref), 1e-3)
    bad = err > tol
    assert not bad.any(), "%s: %d elements beyond rel %g (max err %g)" % (what, int(bad.sum()), rel, err.max())


@pytest.mark.parametrize("dtype,layout", [(T.FP32, T.NCHW), (T.FP16, T.NCHW), (T.FP32, T.NHWC), (T.UINT8, T.NHWC),
                                          (T.FP16, T.NHWC), (T.UINT8, T.NCHW)])
def test_resize_cmn_config0(cuda, dtype, layout):
    """configs[0]: batch 64, 256..512 px sides, resize shorter->256, crop 224, mirror, normalize."""
    from rocal_b200 import kernels as K
    rng = S.rng_for(0)
    arena, hs, ws, offs = S.make_images(rng, 64, (256, 512), (256, 512))
    t = S.classification_tables(rng, hs, ws, offs)
    mul, add = S.normalize_tables()
    ref = O.resample(arena, t, 224, 224, dtype, layout, mul, add)
    for staged, force_tile in ((True, False), (True, True), (False, False)):
        # three code paths: strip-streaming kernel, shared-memory tile kernel, direct gather
        got = K.resample(_dev(arena, cuda), t, 224, 224, dtype, layout, mul, add, staged=staged,
                         path=1 if force_tile else 0).cpu().numpy()
        assert _device_status() == 0
        if dtype == T.FP32:
            _assert_fp(got, ref, 1e-5, "fp32")
            assert np.array_equal(got, ref), "fp32 path is expected to be bit-identical"
        elif dtype == T.FP16:
            _assert_fp(got, ref, 1e-3, "fp16")
            assert np.array_equal(got.view(np.uint16), ref.view(np.uint16))
        else:
            assert np.abs(got.astype(np.int32) - ref.astype(np.int32)).max() <= 1
            assert np.array_equal(got, ref)


def test_resize_cmn_config1_shapes(cuda):
    """configs[1] shapes (300..1080 px sides, fp16 NCHW) on a 48-image slice."""
    from rocal_b200 import kernels as K
    rng = S.rng_for(1)
    arena, hs, ws, offs = S.make_images(rng, 48, (300, 1080), (300, 1080))
    t = S.classification_tables(rng, hs, ws, offs)
    mul, add = S.normalize_tables()
    ref = O.resample(arena, t, 224, 224, T.FP16, T.NCHW, mul, add)
    got = K.resample(_dev(arena, cuda), t, 224, 224, T.FP16, T.NCHW, mul, add).cpu().numpy()
    _assert_fp(got, ref, 1e-3, "fp16")
    assert np.array_equal(got.view(np.uint16), ref.view(np.uint16))


def test_resize_cmn_config1_full_batch(cuda):
    """The launch the benchmark times: all 1024 images of configs[1] (300..1080 px sides, fp16 NCHW, 32-row strips,
    the ring depth picked from the widest source span of the batch), every output bit compared with the oracle."""
    from rocal_b200 import kernels as K
    rng = S.rng_for(1)
    arena, hs, ws, offs = S.make_images(rng, 1024, (300, 1080), (300, 1080))
    t = S.classification_tables(rng, hs, ws, offs)
    mul, add = S.normalize_tables()
    ref = O.resample(arena, t, 224, 224, T.FP16, T.NCHW, mul, add)
    got = K.resample(_dev(arena, cuda), t, 224, 224, T.FP16, T.NCHW, mul, add).cpu().numpy()
    assert _device_status() == 0
    assert np.array_equal(got.view(np.uint16), ref.view(np.uint16))
    # a checksum of per-sample checksums, so that a later change of the generator or the kernel shows up as one number
    per = got.view(np.uint16).reshape(1024, -1).astype(np.uint64).sum(axis=1)
    assert int(per.sum()) == int(ref.view(np.uint16).astype(np.uint64).sum())


@pytest.mark.parametrize("n", [3, 64, 200])
def test_strip_rows_do_not_change_the_result(cuda, n):
    """The row-streaming kernel cuts the output into strips of rows per CTA; the library picks the strip height from the
    grid size and the kernel's occupancy (8, about 14, or 32 rows), `strip_rows` forces it; `path` picks the ring (2: every
    distinct source row staged once, the choice for host memory; 3: the two tap rows of each output row). Every choice - including
    heights that leave a ragged last strip and the smallest and largest allowed - gives the oracle's bits; a value
    outside 4..32 is refused."""
    from rocal_b200 import kernels as K
    from rocal_b200._lib import Rb200Error
    rng = S.rng_for(0, 7 + n)
    arena, hs, ws, offs = S.make_images(rng, n, (256, 512), (256, 512))
    t = S.classification_tables(rng, hs, ws, offs)
    mul, add = S.normalize_tables()
    ref = O.resample(arena, t, 224, 224, T.FP32, T.NCHW, mul, add)
    a = _dev(arena, cuda)
    for path in (2, 3):         # both rings of the row-streaming kernel: distinct rows once / tap-row pairs
        for rows in (0, 4, 5, 14, 15, 31, 32):
            got = K.resample(a, t, 224, 224, T.FP32, T.NCHW, mul, add, strip_rows=rows, path=path).cpu().numpy()
            assert np.array_equal(got.view(np.uint32), ref.view(np.uint32)), (path, rows)
    for rows in (3, 33, -1):
        with pytest.raises(Rb200Error):
            K.resample(a, t, 224, 224, T.FP32, T.NCHW, mul, add, strip_rows=rows)
    assert _device_status() == 0


@pytest.mark.parametrize("path", [2, 3])
def test_stream_kernel_wide_sources_take_the_short_ring(cuda, path):
    """Source spans above 12 KB per tile row leave room for only half the ring (2 stages of row pairs / 4 row slots
    instead of 4 / 8): 6000-pixel-wide images squeezed into one 512-column tile, down- and up-scaled vertically, both
    rings, against the oracle."""
    from rocal_b200 import kernels as K
    rng = S.rng_for(11, path)
    arena, hs, ws, offs = S.make_images(rng, 3, (20, 90), (5200, 6000), content="noise")
    n = len(hs)
    t = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
    t["src_offset"], t["src_stride"] = offs, ws * 3
    t["roi_w"], t["roi_h"] = ws, hs
    t["dst_w"], t["dst_h"] = [512, 400, 300], [45, 30, 64]             # 10 .. 20 source pixels per output pixel across
    t["crop_w"], t["crop_h"] = t["dst_w"], t["dst_h"]
    t["mirror"] = [0, 1, 0]
    ref = O.resample(arena, t, 512, 64, T.UINT8, T.NHWC)
    got = K.resample(_dev(arena, cuda), t, 512, 64, T.UINT8, T.NHWC, path=path).cpu().numpy()
    assert np.array_equal(got, ref)
    assert _device_status() == 0


@pytest.mark.parametrize("dtype,layout", [(T.FP16, T.NCHW), (T.UINT8, T.NHWC)])
def test_pair_ring_warp_kinds(cuda, dtype, layout):
    """The pair ring picks one of four row loops per warp. One batch holds a sample for each: a crop narrower than the tile
    (warps with no column at all and a warp whose upper lanes are idle), an odd crop width (a last column without a
    partner), a whole-image window whose first and last columns clamp their right tap onto the left one (up-scale from a
    3-pixel-wide ROI: the border variant in every warp), a one-pixel-wide source, and the common full case; up- and
    down-scaling, mirrored and not. Both rings and the automatic choice give the oracle's bits."""
    from rocal_b200 import kernels as K
    rng = S.rng_for(12, 3)
    arena, hs, ws, offs = S.make_images(rng, 8, (60, 400), (260, 900), content="noise")
    n = len(hs)
    t = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
    t["src_offset"], t["src_stride"] = offs, ws * 3
    t["roi_w"], t["roi_h"] = ws, hs
    t["dst_w"], t["dst_h"] = 256, 96
    t["crop_w"], t["crop_h"] = 256, 96
    t["mirror"] = np.arange(n) % 2
    t[1]["crop_w"] = 70                                  # warps 2, 3 idle, warp 1 half idle
    t[2]["crop_w"], t[2]["crop_x"] = 133, 40             # odd width: the last thread owns one column
    t[3]["roi_x"], t[3]["roi_w"] = 5, 3                  # 3 source columns -> 256: most columns sit on a border
    t[4]["roi_x"], t[4]["roi_w"] = 17, 1                 # one source column
    t[5]["roi_y"], t[5]["roi_h"] = 9, 2                  # two source rows
    t[6]["dst_w"], t[6]["crop_w"] = 255, 255             # odd resized width, crop = whole
    t[7]["dst_w"], t[7]["dst_h"], t[7]["crop_w"], t[7]["crop_h"] = 1024, 300, 256, 96
    t[7]["crop_x"], t[7]["crop_y"] = 768, 204            # window in the far corner of a larger resized image
    ref = O.resample(arena, t, 256, 96, dtype, layout)
    a = _dev(arena, cuda)
    for path in (0, 2, 3):
        for rows in (0, 8, 32):
            got = K.resample(a, t, 256, 96, dtype, layout, strip_rows=rows, path=path).cpu().numpy()
            assert np.array_equal(got.view(np.uint8), ref.view(np.uint8)), (path, rows)
    assert _device_status() == 0


def test_resize_only_ragged_output(cuda):
    """Plain Resize: uint8 HWC out, per-sample output sizes inside a larger max-shape tensor; only
    the ROI is defined (padding not filled), up- and down-scaling, odd sizes."""
    from rocal_b200 import kernels as K
    import torch
    rng = S.rng_for(10)
    arena, hs, ws, offs = S.make_images(rng, 12, (1, 90), (1, 130))
    n = len(hs)
    t = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
    t["src_offset"], t["src_stride"] = offs, ws * 3
    t["roi_w"], t["roi_h"] = ws, hs
    t["dst_w"] = rng.integers(1, 300, n)
    t["dst_h"] = rng.integers(1, 200, n)
    t["crop_w"], t["crop_h"] = t["dst_w"], t["dst_h"]
    ow, oh = 300, 200
    ref = O.resample(arena, t, ow, oh, T.UINT8, T.NHWC, fill_padding=False)
    canary = torch.full((n, oh, ow, 3), 77, dtype=torch.uint8, device=cuda)
    got = K.resample(_dev(arena, cuda), t, ow, oh, T.UINT8, T.NHWC, fill_padding=False, out=canary).cpu().numpy()
    for i in range(n):
        w, h = int(t[i]["dst_w"]), int(t[i]["dst_h"])
        assert np.array_equal(got[i, :h, :w], ref[i, :h, :w]), "sample %d" % i
        assert (got[i, h:, :] == 77).all() and (got[i, :, w:] == 77).all(), "padding of sample %d was written" % i


def test_resample_roi_crop_mirror_edges(cuda):
    """ResizeCropMirror-style chains: source ROI not at the origin, crop window touching every
    border of the resized image, all-mirror / no-mirror, crop larger than the image (padding
    zero-filled), batch of one, wide outputs that need more than one tile column."""
    from rocal_b200 import kernels as K
    rng = S.rng_for(11)
    arena, hs, ws, offs = S.make_images(rng, 9, (40, 120), (300, 700))
    n = len(hs)
    t = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
    t["src_offset"], t["src_stride"] = offs, ws * 3
    for i in range(n):
        rx, ry = int(rng.integers(0, 20)), int(rng.integers(0, 10))
        t[i]["roi_x"], t[i]["roi_y"] = rx, ry
        t[i]["roi_w"], t[i]["roi_h"] = ws[i] - rx - int(rng.integers(0, 20)), hs[i] - ry - int(rng.integers(0, 10))
        t[i]["dst_w"], t[i]["dst_h"] = int(rng.integers(200, 900)), int(rng.integers(30, 200))
        cw, ch = min(int(rng.integers(100, 640)), t[i]["dst_w"]), min(int(rng.integers(20, 150)), t[i]["dst_h"])
        corner = i % 4
        t[i]["crop_x"] = 0 if corner in (0, 2) else t[i]["dst_w"] - cw
        t[i]["crop_y"] = 0 if corner in (0, 1) else t[i]["dst_h"] - ch
        t[i]["crop_w"], t[i]["crop_h"] = cw, ch
        t[i]["mirror"] = i % 2
    for sl in (slice(0, n), slice(3, 4)):
        tt = np.ascontiguousarray(t[sl])
        for dtype, layout in ((T.UINT8, T.NHWC), (T.FP32, T.NCHW)):
            ref = O.resample(arena, tt, 640, 150, dtype, layout)
            for staged in (True, False):
                got = K.resample(_dev(arena, cuda), tt, 640, 150, dtype, layout, staged=staged).cpu().numpy()
                assert np.array_equal(got, ref)


def test_resample_extreme_ratios(cuda):
    """Heavy down-scaling (ratio > 2: sparse row staging) and up-scaling in one batch."""
    from rocal_b200 import kernels as K
    rng = S.rng_for(12)
    arena, hs, ws, offs = S.make_images(rng, 6, (900, 1500), (1200, 2000))
    n = len(hs)
    t = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
    t["src_offset"], t["src_stride"] = offs, ws * 3
    t["roi_w"], t["roi_h"] = ws, hs
    t["dst_w"] = [64, 100, 224, 3000, 150, 224]
    t["dst_h"] = [64, 80, 224, 40, 2500, 224]
    t["crop_w"] = np.minimum(t["dst_w"], 224)
    t["crop_h"] = np.minimum(t["dst_h"], 224)
    t["crop_x"] = (t["dst_w"] - t["crop_w"]) // 2
    t["crop_y"] = (t["dst_h"] - t["crop_h"]) // 2
    t["mirror"] = [0, 1, 0, 1, 0, 1]
    ref = O.resample(arena, t, 224, 224, T.UINT8, T.NHWC)
    got = K.resample(_dev(arena, cuda), t, 224, 224, T.UINT8, T.NHWC).cpu().numpy()
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("op", [T.COLOR_TWIST, T.COLOR_BRIGHTNESS, T.COLOR_CONTRAST, T.COLOR_NONE])
def test_color_flip_config2(cuda, op):
    """configs[2]: batch 256 of 224x224 noise, per-sample alpha/beta/hue/sat, hflip p=.5, uint8 HWC."""
    from rocal_b200 import kernels as K
    rng = S.rng_for(2)
    arena, hs, ws, offs = S.make_images(rng, 256, (224, 224), (224, 224), content="noise")
    t = S.color_twist_tables(rng, hs, ws, offs)
    if op == T.COLOR_CONTRAST:
        t["beta"] = rng.uniform(60, 200, len(t)).astype(np.float32)
    ref = O.pointwise(arena, t, 224, 224, op)
    got = K.pointwise(_dev(arena, cuda), t, 224, 224, op).cpu().numpy()
    diff = np.abs(got.astype(np.int32) - ref.astype(np.int32))
    assert diff.max() <= 1
    assert np.array_equal(got, ref)


def test_pointwise_crop_flip_normalize(cuda):
    """Crop / Flip / CropMirrorNormalize / to_tensor: pure indexing must be bit-exact; windows that
    touch the borders, vertical + horizontal flips, channel reversal, every dtype and layout."""
    from rocal_b200 import kernels as K
    rng = S.rng_for(13)
    arena, hs, ws, offs = S.make_images(rng, 10, (1, 70), (1, 300))
    n = len(hs)
    t = np.zeros(n, dtype=T.POINTWISE_SAMPLE)
    t["src_offset"], t["src_stride"] = offs, ws * 3
    for i in range(n):
        w = int(rng.integers(1, ws[i] + 1))
        h = int(rng.integers(1, hs[i] + 1))
        t[i]["roi_w"], t[i]["roi_h"] = w, h
        t[i]["roi_x"] = (ws[i] - w) if i % 2 else 0
        t[i]["roi_y"] = (hs[i] - h) if i % 3 else 0
        t[i]["flip_h"], t[i]["flip_v"] = i & 1, (i >> 1) & 1
    mul, add = S.normalize_tables()
    for dtype in (T.UINT8, T.FP32, T.FP16):
        for layout in (T.NHWC, T.NCHW):
            for rev in (False, True):
                norm = dtype != T.UINT8
                ref = O.pointwise(arena, t, 300, 70, T.COLOR_NONE, dtype, layout, mul if norm else None,
                                  add if norm else None, reverse_channels=rev)
                got = K.pointwise(_dev(arena, cuda), t, 300, 70, T.COLOR_NONE, dtype, layout, mul if norm else None,
                                  add if norm else None, reverse_channels=rev).cpu().numpy()
                assert np.array_equal(got.view(np.uint8), ref.view(np.uint8))


@pytest.mark.parametrize("op", [T.COLOR_BRIGHTNESS, T.COLOR_CONTRAST, T.COLOR_TWIST, T.COLOR_GAMMA])
def test_color_ops_ragged_windows(cuda, op):
    """Colour operators on ragged windows (widths 1..300, so the 16-pixel units, the 4-pixel items and the partial
    groups of the uint8 path all run), horizontal / vertical flips, uint8 NHWC and normalised fp32 NCHW outputs."""
    from rocal_b200 import kernels as K
    rng = S.rng_for(14)
    arena, hs, ws, offs = S.make_images(rng, 12, (1, 70), (1, 300), content="noise")
    n = len(hs)
    t = S.color_twist_tables(rng, hs, ws, offs)
    for i in range(n):
        w = int(rng.integers(1, ws[i] + 1))
        h = int(rng.integers(1, hs[i] + 1))
        t[i]["roi_w"], t[i]["roi_h"] = w, h
        t[i]["roi_x"] = (ws[i] - w) if i % 2 else 0
        t[i]["roi_y"] = (hs[i] - h) if i % 3 else 0
        t[i]["flip_h"], t[i]["flip_v"] = i & 1, (i >> 1) & 1
    if op == T.COLOR_CONTRAST:
        t["beta"] = rng.uniform(60, 200, n).astype(np.float32)
    if op == T.COLOR_GAMMA:
        t["alpha"] = rng.uniform(0.4, 3.0, n).astype(np.float32)
    mul, add = S.normalize_tables()
    for dtype, layout, m, a in ((T.UINT8, T.NHWC, None, None), (T.FP32, T.NCHW, mul, add)):
        ref = O.pointwise(arena, t, 300, 70, op, dtype, layout, m, a)
        got = K.pointwise(_dev(arena, cuda), t, 300, 70, op, dtype, layout, m, a).cpu().numpy()
        if op != T.COLOR_GAMMA:
            assert np.array_equal(got.view(np.uint8), ref.view(np.uint8))
        elif dtype == T.UINT8:
            assert np.abs(got.astype(np.int32) - ref.astype(np.int32)).max() <= 1
        else:
            assert np.abs(got - ref).max() <= float(np.max(np.abs(np.asarray(mul, dtype=np.float32)))) * 1.0001


def test_flip_twice_is_identity(cuda):
    from rocal_b200 import kernels as K
    rng = S.rng_for(14)
    arena, hs, ws, offs = S.make_images(rng, 4, (33, 33), (47, 47), content="noise")
    t = np.zeros(4, dtype=T.POINTWISE_SAMPLE)
    t["src_offset"], t["src_stride"], t["roi_w"], t["roi_h"] = offs, ws * 3, ws, hs
    t["flip_h"], t["flip_v"] = [1, 0, 1, 1], [0, 1, 1, 1]
    d = _dev(arena, cuda)
    once = K.pointwise(d, t, 47, 33)
    t2 = t.copy()
    t2["src_offset"] = np.arange(4) * 47 * 33 * 3
    twice = K.pointwise(once.reshape(-1), t2, 47, 33).cpu().numpy()
    for i in range(4):
        img = arena[int(offs[i]):int(offs[i]) + 47 * 33 * 3].reshape(33, 47, 3)
        assert np.array_equal(twice[i], img)


@pytest.mark.parametrize("dtype,layout", [(T.UINT8, T.NHWC), (T.FP32, T.NCHW), (T.FP16, T.NCHW)])
def test_resample_triangular(cuda, dtype, layout):
    """Triangular filter (ROCAL_TRIANGULAR_INTERPOLATION): down-scale ratios 1.2..4.2 with their growing tap
    counts, up-scaling (two taps per axis), a crop -> resize chain with mirror, ragged sizes; bit-exact against
    the restatement of the reference's generic resize kernel."""
    from rocal_b200 import kernels as K
    rng = S.rng_for(19)
    arena, hs, ws, offs = S.make_images(rng, 12, (60, 400), (60, 400))
    t = S.classification_tables(rng, hs, ws, offs, resize_shorter=96, crop=80)
    # samples 0..2: up-scaling; 3..5: a window of the source resized to a fixed size
    for i in range(3):
        t[i]["dst_w"], t[i]["dst_h"] = int(ws[i] * 1.7), int(hs[i] * 1.3)
        t[i]["crop_x"], t[i]["crop_y"] = 3, 2
    for i in range(3, 6):
        t[i]["roi_x"], t[i]["roi_y"] = ws[i] // 5, hs[i] // 7
        t[i]["roi_w"], t[i]["roi_h"] = ws[i] // 2, hs[i] // 2
        t[i]["dst_w"], t[i]["dst_h"], t[i]["crop_x"], t[i]["crop_y"] = 80, 80, 0, 0
    mul, add = S.normalize_tables() if dtype != T.UINT8 else (None, None)
    ref = O.resample(arena, t, 80, 80, dtype, layout, mul, add, interpolation=1)
    got = K.resample(_dev(arena, cuda), t, 80, 80, dtype, layout, mul, add, interpolation=1).cpu().numpy()
    assert np.array_equal(got.view(np.uint8), ref.view(np.uint8))
    bil = O.resample(arena, t, 80, 80, dtype, layout, mul, add)
    assert not np.array_equal(bil.view(np.uint8), ref.view(np.uint8))      # it is a different filter


@pytest.mark.parametrize("interpolation,exact", [(2, True), (5, True), (3, False), (4, False)])
def test_resample_other_filters(cuda, interpolation, exact):
    """Bicubic (2), lanczos (3), gaussian (4), nearest (5) on the generic-filter skeleton: down- and up-scaling, a
    window with mirror, ragged sizes. Bicubic and nearest are bit-exact against the restatement; lanczos and gaussian
    go through sinf / expf, so a truncated uint8 may differ by one level (tolerance 1 LSB)."""
    from rocal_b200 import kernels as K
    rng = S.rng_for(27)
    arena, hs, ws, offs = S.make_images(rng, 10, (50, 300), (50, 300))
    t = S.classification_tables(rng, hs, ws, offs, resize_shorter=72, crop=64)
    for i in range(3):
        t[i]["dst_w"], t[i]["dst_h"] = int(ws[i] * 1.6), int(hs[i] * 1.25)
        t[i]["crop_x"], t[i]["crop_y"] = 2, 1
    for i in range(3, 5):
        t[i]["roi_x"], t[i]["roi_y"] = ws[i] // 6, hs[i] // 5
        t[i]["roi_w"], t[i]["roi_h"] = ws[i] // 2, hs[i] // 2
        t[i]["dst_w"], t[i]["dst_h"], t[i]["crop_x"], t[i]["crop_y"] = 64, 64, 0, 0
    for dtype, layout in ((T.UINT8, T.NHWC), (T.FP32, T.NCHW)):
        mul, add = S.normalize_tables() if dtype != T.UINT8 else (None, None)
        ref = O.resample(arena, t, 64, 64, dtype, layout, mul, add, interpolation=interpolation)
        got = K.resample(_dev(arena, cuda), t, 64, 64, dtype, layout, mul, add, interpolation=interpolation).cpu().numpy()
        if exact:
            assert np.array_equal(got.view(np.uint8), ref.view(np.uint8))
        elif dtype == T.UINT8:
            d = np.abs(got.astype(np.int32) - ref.astype(np.int32))
            assert d.max() <= 1 and (d != 0).mean() < 1e-3
        else:
            step = float(np.max(np.abs(np.asarray(mul, dtype=np.float32)))) * 1.0001          # one uint8 level after normalisation
            d = np.abs(got - ref)
            assert d.max() <= step and (d > 1e-6).mean() < 1e-3
    tri = O.resample(arena, t, 64, 64, T.UINT8, T.NHWC, interpolation=1)
    assert not np.array_equal(tri, O.resample(arena, t, 64, 64, T.UINT8, T.NHWC, interpolation=interpolation))


def test_warp_affine_config3(cuda):
    """configs[3]: 480x640 images, rotation +-45 deg, scale 0.8..1.2, shift +-32 px, zero border (batch 32)."""
    from rocal_b200 import kernels as K
    rng = S.rng_for(3)
    arena, hs, ws, offs = S.make_images(rng, 32, (480, 480), (640, 640))
    t = S.warp_tables(rng, hs, ws, offs, 640, 480)
    ref = O.warp_affine(arena, t, 640, 480)
    got = K.warp_affine(_dev(arena, cuda), t, 640, 480).cpu().numpy()
    diff = np.abs(got.astype(np.int32) - ref.astype(np.int32))
    assert diff.max() <= 1
    assert np.array_equal(got, ref)
    assert (ref == 0).mean() > 0.01   # the border region exists in this configuration


def test_rotate_fixed_and_identity(cuda):
    """Rotate as a warp table: 0 degrees reproduces the source away from the last row/column;
    45 degrees (the reference's RotateFixed test case) matches the oracle; ragged source sizes."""
    from rocal_b200 import kernels as K
    rng = S.rng_for(15)
    arena, hs, ws, offs = S.make_images(rng, 5, (20, 90), (20, 120))
    n = len(hs)
    for angle in (0.0, 45.0, -170.0):
        t = np.zeros(n, dtype=T.WARP_SAMPLE)
        t["src_offset"], t["src_stride"], t["src_w"], t["src_h"] = offs, ws * 3, ws, hs
        t["dst_w"], t["dst_h"] = ws, hs
        t["m"][:] = S.rotate_matrix(angle)
        ref = O.warp_affine(arena, t, 120, 90)
        got = K.warp_affine(_dev(arena, cuda), t, 120, 90).cpu().numpy()
        assert np.array_equal(got, ref)
        if angle == 0.0:
            for i in range(n):
                h, w = int(hs[i]), int(ws[i])
                if h % 2 == 0 and w % 2 == 0:
                    img = arena[int(offs[i]):int(offs[i]) + h * w * 3].reshape(h, w, 3)
                    assert np.array_equal(got[i, :h - 1, :w - 1], img[:h - 1, :w - 1])


def test_warp_affine_edges(cuda):
    """Output width not a multiple of four (byte stores), strong minification (footprint too large to
    stage: global gathers), 1-pixel-wide and 1-pixel-high sources, a table holding NaN and huge entries,
    destination smaller than the output canvas with and without zero fill."""
    import torch
    from rocal_b200 import kernels as K
    rng = S.rng_for(16)
    arena, hs, ws, offs = S.make_images(rng, 8, (1, 200), (1, 300))
    hs, ws = hs.copy(), ws.copy()
    n = len(hs)
    t = np.zeros(n, dtype=T.WARP_SAMPLE)
    # sources narrower than their allocation: the stride stays that of the allocation
    t["src_offset"], t["src_stride"] = offs, ws * 3
    ws[0], hs[1] = 1, 1
    t["src_w"], t["src_h"] = ws, hs
    mats = np.stack([S.rotate_matrix(a) for a in (0.0, 10.0, 33.0, 90.0, 181.0, -45.0, 5.0, 60.0)])
    mats[2, :4] *= 6.0            # minification by 6: staged footprint exceeds the shared-memory budget
    mats[3, :4] *= 0.2            # magnification by 5
    mats[4, 4:] = (7.25, -3.5)
    mats[6, 0] = np.nan
    mats[7, 1] = 3.0e38
    t["m"][:] = mats
    for out_w, out_h, dw, dh in ((117, 93, 117, 93), (160, 96, 101, 77), (64, 64, 200, 200)):
        t["dst_w"], t["dst_h"] = dw, dh
        for fill in (True, False):
            base = np.full((n, out_h, out_w, 3), 7, dtype=np.uint8)
            ref = O.warp_affine(arena, t, out_w, out_h, fill_padding=fill, out=base.copy())
            got = K.warp_affine(_dev(arena, cuda), t, out_w, out_h, fill_padding=fill,
                                out=torch.from_numpy(base.copy()).to(cuda)).cpu().numpy()
            assert np.array_equal(got, ref), (out_w, out_h, dw, dh, fill)


@pytest.mark.parametrize("offset", [True, False])
def test_box_encoder_config4(cuda, offset):
    """configs[4]: 128 samples, 1..50 boxes, 8732 anchors, criteria 0.5; labels (matched indices)
    bit-exact, encoded boxes within 1e-5 relative (logf differs by an ulp between libm and CUDA)."""
    import torch
    from rocal_b200 import kernels as K
    rng = S.rng_for(4)
    anchors = S.ssd300_anchors()
    boxes, labels, offs = S.random_boxes(rng, 128)
    rb, rl = O.box_encode(boxes, labels, offs, anchors, 0.5, (0, 0, 0, 0), (0.1, 0.1, 0.2, 0.2), offset, 1.0)
    gb, gl = K.box_encode(torch.from_numpy(boxes).to(cuda), torch.from_numpy(labels).to(cuda),
                          torch.from_numpy(offs).to(cuda), torch.from_numpy(anchors).to(cuda), 0.5, (0, 0, 0, 0),
                          (0.1, 0.1, 0.2, 0.2), offset, 1.0, 50)
    assert np.array_equal(gl.cpu().numpy(), rl)
    _assert_fp(gb.cpu().numpy(), rb, 1e-5, "encoded boxes")


def test_box_encoder_ties_and_chunks(cuda):
    """Duplicate boxes (ties between boxes), boxes equal to anchors (IoU 1), one box per sample,
    more boxes than one shared-memory chunk, a small anchor set, non-zero means and scale != 1."""
    import torch
    from rocal_b200 import kernels as K
    rng = S.rng_for(16)
    anchors = S.ssd300_anchors()[::7][:1000].copy()
    counts = [1, 2, 33, 64, 65, 100, 3]
    per = []
    for c in counts:
        b, _, _ = S.random_boxes(rng, 1, (c, c))
        b[c // 2] = b[0]
        if c > 2:
            b[-1] = anchors[int(rng.integers(0, len(anchors)))]
        per.append(b)
    boxes = np.ascontiguousarray(np.concatenate(per))
    offs = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    labels = rng.integers(1, 81, len(boxes)).astype(np.int32)
    for offset, scale, means in ((True, 1.0, (0, 0, 0, 0)), (True, 2.0, (0.1, -0.1, 0.2, 0.05)), (False, 1.0, (0, 0, 0, 0))):
        rb, rl = O.box_encode(boxes, labels, offs, anchors, 0.45, means, (0.1, 0.1, 0.2, 0.2), offset, scale)
        gb, gl = K.box_encode(torch.from_numpy(boxes).to(cuda), torch.from_numpy(labels).to(cuda),
                              torch.from_numpy(offs).to(cuda), torch.from_numpy(anchors).to(cuda), 0.45, means,
                              (0.1, 0.1, 0.2, 0.2), offset, scale, 100)
        assert np.array_equal(gl.cpu().numpy(), rl)
        _assert_fp(gb.cpu().numpy(), rb, 1e-5, "encoded boxes")


def test_box_encoder_degenerate_and_large_tables(cuda):
    """Zero-area and inverted boxes (IoU 0/0 = NaN and negative IoU follow the CPU loop's seeding rules),
    a sample without boxes, and anchor tables large enough for the 8- and 16-anchors-per-thread kernels."""
    import torch
    from rocal_b200 import kernels as K
    rng = S.rng_for(17)
    base = S.ssd300_anchors()
    counts = [4, 0, 6, 1, 3]
    boxes, _, _ = S.random_boxes(rng, 1, (sum(counts), sum(counts)))
    boxes[0] = (0.3, 0.3, 0.3, 0.3)                 # a point: area 0
    boxes[1] = (0.6, 0.6, 0.2, 0.2)                 # inverted
    boxes[4] = (0.0, 0.0, 0.0, 0.0)                 # equals the degenerate anchor below
    boxes[10] = (0.5, 0.2, 0.5, 0.9)                # zero width
    boxes[11] = boxes[12] = (0.25, 0.25, 0.25, 0.25)
    offs = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    labels = rng.integers(1, 81, len(boxes)).astype(np.int32)
    for num in (37, 8732, 20000, 40000):
        reps = -(-num // len(base))
        jitter = rng.uniform(-0.01, 0.01, (reps * len(base), 4)).astype(np.float32)
        anchors = np.ascontiguousarray((np.tile(base, (reps, 1)) + jitter)[:num])
        anchors[0] = (0.0, 0.0, 0.0, 0.0)           # anchor 0 degenerate: its IoU with a point box is NaN
        for offset in (True, False):
            rb, rl = O.box_encode(boxes, labels, offs, anchors, 0.5, (0, 0, 0, 0), (0.1, 0.1, 0.2, 0.2), offset, 1.0)
            gb, gl = K.box_encode(torch.from_numpy(boxes).to(cuda), torch.from_numpy(labels).to(cuda),
                                  torch.from_numpy(offs).to(cuda), torch.from_numpy(anchors).to(cuda), 0.5,
                                  (0, 0, 0, 0), (0.1, 0.1, 0.2, 0.2), offset, 1.0, 50)
            assert np.array_equal(gl.cpu().numpy(), rl), (num, offset)
            got, ref = gb.cpu().numpy(), rb
            assert np.array_equal(np.isnan(got), np.isnan(ref)), (num, offset)
            assert np.array_equal(np.isinf(got), np.isinf(ref)), (num, offset)
            fin = np.isfinite(ref)
            _assert_fp(got[fin], ref[fin], 1e-5, "encoded boxes")


@pytest.mark.parametrize("allow", [True, False])
def test_box_iou_matcher(cuda, allow):
    """Matched box index per anchor with the -1 / -2 threshold codes and the low-quality rule: SSD-300 table
    with 1..50 boxes, a RetinaNet-sized table (120 087 anchors: 15 register groups per CTA), a tiny table,
    degenerate boxes, a sample without boxes, exact ties between boxes; all indices must be equal."""
    import torch
    from rocal_b200 import kernels as K
    rng = S.rng_for(18)
    base = S.ssd300_anchors()
    boxes, labels, offs = S.random_boxes(rng, 24)
    cases = [(base, boxes, offs, 0.5, 0.4)]
    reps = -(-120087 // len(base))
    big = np.ascontiguousarray((np.tile(base, (reps, 1)) + rng.uniform(-0.02, 0.02, (reps * len(base), 4)).astype(np.float32))[:120087])
    cases.append((big, boxes[:int(offs[6])], offs[:7], 0.5, 0.4))
    counts = [4, 0, 6, 1, 3]
    db, _, _ = S.random_boxes(rng, 1, (sum(counts), sum(counts)))
    db[0] = (0.3, 0.3, 0.3, 0.3)
    db[1] = (0.6, 0.6, 0.2, 0.2)
    db[5] = db[4]                                   # two identical boxes: the lower index keeps the anchors
    db[10] = (0.5, 0.2, 0.5, 0.9)
    db[12] = base[4000]                             # IoU 1 with one anchor
    doffs = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    small = base[::200][:37].copy()
    small[0] = (0.0, 0.0, 0.0, 0.0)
    cases.append((base, db, doffs, 0.7, 0.3))
    cases.append((small, db, doffs, 0.5, 0.4))
    for anchors, bx, of, hi, lo in cases:
        ref = O.box_iou_match(bx, of, anchors, hi, lo, allow)
        got = K.box_iou_match(torch.from_numpy(np.ascontiguousarray(bx)).to(cuda), torch.from_numpy(np.ascontiguousarray(of)).to(cuda),
                              torch.from_numpy(anchors).to(cuda), hi, lo, allow, 64).cpu().numpy()
        assert np.array_equal(got, ref), (len(anchors), hi, lo)
        assert (ref >= 0).sum() > 0


def test_ssd_chain_config4(cuda):
    """configs[4] image chain: SSD random crop window -> resize 300x300 -> mirror -> normalize fp32 (batch 32)."""
    from rocal_b200 import kernels as K
    rng = S.rng_for(4)
    arena, hs, ws, offs = S.make_images(rng, 32, (300, 800), (300, 800))
    boxes, labels, boffs = S.random_boxes(rng, 32)
    crops, _, _, _ = S.ssd_random_crop(rng, boxes, labels, boffs)
    t = S.ssd_resample_tables(rng, hs, ws, offs, crops)
    mul, add = S.normalize_tables()
    ref = O.resample(arena, t, 300, 300, T.FP32, T.NCHW, mul, add)
    got = K.resample(_dev(arena, cuda), t, 300, 300, T.FP32, T.NCHW, mul, add).cpu().numpy()
    _assert_fp(got, ref, 1e-5, "fp32")
    assert np.array_equal(got, ref)


def test_empty_batch_and_bad_arguments(cuda):
    import torch
    from rocal_b200 import kernels as K
    from rocal_b200._lib import Rb200Error
    arena = torch.zeros(1024, dtype=torch.uint8, device=cuda)
    t = np.zeros(0, dtype=T.RESAMPLE_SAMPLE)
    out = K.resample(arena, t, 8, 8, d_samples=arena)
    assert out.shape[0] == 0
    t = np.zeros(1, dtype=T.RESAMPLE_SAMPLE)   # dst size 0 -> rejected on the host, nothing launched
    with pytest.raises(Rb200Error):
        K.resample(arena, t, 8, 8, fill_padding=False)
    with pytest.raises(Rb200Error):
        K.resample(arena, t, 0, 8)


def test_color_twist_fast_arithmetic_within_one_level(cuda):
    """RB200_ARITH_FAST: ColorTwist (and Hue / Saturation, the same operator) with fused operations, one hardware
    reciprocal and the periodic HSV -> RGB form. Every byte lies within one level of the exact result and all but a
    few per million are equal; greys, fully saturated colours, negative and large saturation factors, hue shifts
    beyond a full turn, flips and both uint8 layouts are covered. Other operators ignore the setting."""
    from rocal_b200 import kernels as K
    rng = S.rng_for(50)
    n = 48
    arena, hs, ws, offs = S.make_images(rng, n, (96, 96), (128, 128), content="noise")
    px = arena[:96 * 128 * 3].reshape(-1, 3)
    px[:4000] = np.repeat(rng.integers(0, 256, 4000, dtype=np.uint8)[:, None], 3, 1)     # greys
    px[4000:8000, 0] = 255                                                                # red at its maximum
    px[8000:12000, 2] = 0
    t = S.color_twist_tables(rng, hs, ws, offs)
    t["alpha"] = rng.uniform(0.1, 1.95, n)
    t["beta"] = rng.uniform(0.0, 25.0, n)
    t["hue"] = rng.uniform(-400.0, 400.0, n)
    t["sat"] = rng.uniform(-0.2, 2.5, n)
    a = _dev(arena, cuda)
    for layout in (T.NHWC, T.NCHW):
        ref = O.pointwise(arena, t, 128, 96, T.COLOR_TWIST, T.UINT8, layout)
        exact = K.pointwise(a, t, 128, 96, T.COLOR_TWIST, T.UINT8, layout, arith=0).cpu().numpy()
        fast = K.pointwise(a, t, 128, 96, T.COLOR_TWIST, T.UINT8, layout, arith=1).cpu().numpy()
        assert np.array_equal(exact, ref)
        d = np.abs(fast.astype(np.int32) - ref.astype(np.int32))
        assert d.max() <= 1, "fast arithmetic left the one-level band"
        assert np.count_nonzero(d) < d.size * 1e-4, "%d of %d bytes differ" % (np.count_nonzero(d), d.size)
    # operators without a fast instantiation, and float outputs, are exact under either setting
    ref = O.pointwise(arena, t, 128, 96, T.COLOR_BRIGHTNESS)
    assert np.array_equal(K.pointwise(a, t, 128, 96, T.COLOR_BRIGHTNESS, arith=1).cpu().numpy(), ref)
    ref = O.pointwise(arena, t, 128, 96, T.COLOR_TWIST, T.FP32, T.NCHW)
    assert np.array_equal(K.pointwise(a, t, 128, 96, T.COLOR_TWIST, T.FP32, T.NCHW, arith=1).cpu().numpy(), ref)


def test_overlapped_launches_are_exact(cuda):
    """overlap = 1: independent launches enqueued back to back may run under one another's tails. Sixty launches
    rotating over three batches with their own outputs, resample / pointwise / affine interleaved, then readers that
    know nothing of the overlap (torch copies) - every output still equals the oracle."""
    import torch
    from rocal_b200 import kernels as K
    rng = S.rng_for(51)
    mul, add = S.normalize_tables()
    sets = []
    for _ in range(3):
        arena, hs, ws, offs = S.make_images(rng, 24, (256, 400), (256, 400))
        t = S.classification_tables(rng, hs, ws, offs)
        pt = S.color_twist_tables(rng, np.minimum(hs, 224), np.minimum(ws, 224), offs)
        pt["src_stride"] = ws * 3
        wt = S.warp_tables(rng, hs, ws, offs, 160, 120)
        a = _dev(arena, cuda)
        sets.append({"arena": arena, "a": a, "t": t, "pt": pt, "wt": wt,
                     "o1": torch.zeros((24, 3, 224, 224), dtype=torch.float32, device=cuda),
                     "o2": torch.zeros((24, 224, 224, 3), dtype=torch.uint8, device=cuda),
                     "o3": torch.zeros((24, 120, 160, 3), dtype=torch.uint8, device=cuda),
                     "dt": K.to_device_table(t, cuda), "dpt": K.to_device_table(pt, cuda), "dwt": K.to_device_table(wt, cuda)})
    for i in range(20):
        s = sets[i % 3]
        K.resample(s["a"], s["t"], 224, 224, T.FP32, T.NCHW, mul, add, out=s["o1"], d_samples=s["dt"], overlap=True)
        K.pointwise(s["a"], s["pt"], 224, 224, T.COLOR_BRIGHTNESS, out=s["o2"], d_samples=s["dpt"], overlap=True)
        K.warp_affine(s["a"], s["wt"], 160, 120, out=s["o3"], d_samples=s["dwt"], overlap=True)
    copies = [(s["o1"].clone(), s["o2"].clone(), s["o3"].clone()) for s in sets]      # ordinary stream-ordered readers
    torch.cuda.synchronize()
    assert _device_status() == 0
    for s, (c1, c2, c3) in zip(sets, copies):
        assert np.array_equal(c1.cpu().numpy(), O.resample(s["arena"], s["t"], 224, 224, T.FP32, T.NCHW, mul, add))
        assert np.array_equal(c2.cpu().numpy(), O.pointwise(s["arena"], s["pt"], 224, 224, T.COLOR_BRIGHTNESS))
        assert np.array_equal(c3.cpu().numpy(), O.warp_affine(s["arena"], s["wt"], 160, 120))


@pytest.mark.parametrize("rule", [0, 1])
def test_box_transform_on_the_device(cuda, rule):
    """rb200k_box_transform: boxes that live in device memory through a crop window and mirrors, bit for bit the
    float32 restatement (quarter-area rule of the crop meta nodes / centre rule of the SSD crop), samples without
    boxes and samples that lose all of theirs included; its outputs feed the encoder directly."""
    import torch
    from rocal_b200 import kernels as K
    rng = S.rng_for(4, 900 + rule)
    n = 97
    boxes, labels, offs = S.random_boxes(rng, n, (0, 40), size_range=(0.02, 0.6))
    win = np.zeros(n, dtype=T.BOX_WINDOW)
    l, t = rng.uniform(0, 0.6, n), rng.uniform(0, 0.6, n)
    win["l"], win["t"] = l, t
    win["r"], win["b"] = l + rng.uniform(0.05, 0.4, n), t + rng.uniform(0.05, 0.4, n)
    win["l"][0], win["t"][0], win["r"][0], win["b"][0] = 0, 0, 1, 1            # the whole image
    win["mirror_h"], win["mirror_v"] = rng.integers(0, 2, n), rng.integers(0, 2, n)
    if len(boxes):
        boxes[0, 2:] = boxes[0, :2]                                          # an empty box: 0 / 0 under the area rule
    windows = np.stack([win["l"], win["t"], win["r"], win["b"]], 1)
    eb, el, eo = O.box_transform(boxes, labels, offs, windows, rule, win["mirror_h"], win["mirror_v"])
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    gb, gl, go = K.box_transform(d(boxes), d(labels), d(offs), win, rule)
    go = go.cpu().numpy()
    assert np.array_equal(go, eo)
    total = int(go[-1])
    assert np.array_equal(gl.cpu().numpy()[:total], el)
    assert np.array_equal(gb.cpu().numpy()[:total].view(np.uint32), eb.view(np.uint32))
    assert int((el > 0).sum()) > 50 and int((el == 0).sum()) > 5             # both kinds of samples occurred
    # straight into the encoder
    anchors = S.ssd300_anchors()[::7].copy()
    xb, xl = K.box_encode(gb, gl, torch.from_numpy(go).to(cuda), d(anchors), 0.5, (0, 0, 0, 0), (0.1, 0.1, 0.2, 0.2), True, 1.0, 64)
    rb, rl = O.box_encode(eb, el, eo, anchors, 0.5, (0, 0, 0, 0), (0.1, 0.1, 0.2, 0.2), True, 1.0)
    assert np.array_equal(xl.cpu().numpy(), rl) and np.allclose(xb.cpu().numpy(), rb, rtol=1e-5, atol=1e-6)
    assert _device_status() == 0

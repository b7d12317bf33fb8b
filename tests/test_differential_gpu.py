"""Randomised differential test: random sample tables (sizes 1..700, windows, crops, mirrors / flips, every output
type and layout, staged and direct resample paths, the exact filters, the colour operators, affine tables with
rotations up to 180 degrees and scales 0.3..3) go through the CUDA kernels and the CPU oracle; the results must be
bit-identical. The seeds are fixed, so a failure names the case that reproduces it."""
import numpy as np
import pytest
import torch

from oracle import pyoracle as O
from rocal_b200 import kernels as K
import synthetic as S
from rocal_b200 import tables as T

pytestmark = pytest.mark.gpu


def _case(seed, cuda):
    mul, add = S.normalize_tables()
    rng = np.random.Generator(np.random.PCG64(seed))
    n = int(rng.integers(1, 9))
    hi = int(rng.choice([8, 40, 200, 700]))
    arena, hs, ws, offs = S.make_images(rng, n, (1, hi + 1), (1, hi + 1), content="noise")
    d_arena = torch.from_numpy(arena).to(cuda)
    kind = int(rng.integers(0, 3))
    dtype = int(rng.choice([T.UINT8, T.FP32, T.FP16]))
    layout = int(rng.choice([T.NHWC, T.NCHW]))
    norm = dtype != T.UINT8 or rng.random() < 0.3
    m, a = (mul, add) if norm else (None, None)
    if kind == 0:
        out_w, out_h = int(rng.integers(1, 300)), int(rng.integers(1, 200))
        interp = int(rng.choice([0, 0, 0, 1, 2, 5]))
        t = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
        for i in range(n):
            rw, rh = int(rng.integers(1, ws[i] + 1)), int(rng.integers(1, hs[i] + 1))
            rx, ry = int(rng.integers(0, ws[i] - rw + 1)), int(rng.integers(0, hs[i] - rh + 1))
            dw, dh = int(rng.integers(1, 400)), int(rng.integers(1, 300))
            if interp != 0:   # keep the tap count of the slow filters bounded
                dw, dh = max(dw, rw // 12 + 1), max(dh, rh // 12 + 1)
            cw, ch = int(rng.integers(1, dw + 1)), int(rng.integers(1, dh + 1))
            t[i]["src_offset"], t[i]["src_stride"] = offs[i], ws[i] * 3
            t[i]["roi_x"], t[i]["roi_y"], t[i]["roi_w"], t[i]["roi_h"] = rx, ry, rw, rh
            t[i]["dst_w"], t[i]["dst_h"] = dw, dh
            t[i]["crop_x"], t[i]["crop_y"] = int(rng.integers(0, dw - cw + 1)), int(rng.integers(0, dh - ch + 1))
            t[i]["crop_w"], t[i]["crop_h"] = cw, ch
            t[i]["mirror"] = int(rng.integers(0, 2))
        staged = bool(rng.integers(0, 2))
        ref = O.resample(arena, t, out_w, out_h, dtype, layout, m, a, interpolation=interp)
        path = seed % 4      # automatic choice, tile kernel, row ring, pair ring
        got = K.resample(d_arena, t, out_w, out_h, dtype, layout, m, a, staged=staged, interpolation=interp, path=path).cpu().numpy()
        assert np.array_equal(got.view(np.uint8), ref.view(np.uint8)), ("resample", seed, interp, dtype, layout, staged, path, out_w, out_h)
    elif kind == 1:
        out_w, out_h = int(rng.integers(1, 90)) * int(rng.choice([1, 4])), int(rng.integers(1, 200))
        op = int(rng.choice([T.COLOR_NONE, T.COLOR_BRIGHTNESS, T.COLOR_CONTRAST, T.COLOR_TWIST]))
        t = S.color_twist_tables(rng, hs, ws, offs)
        for i in range(n):
            w, h = int(rng.integers(1, ws[i] + 1)), int(rng.integers(1, hs[i] + 1))
            t[i]["roi_w"], t[i]["roi_h"] = w, h
            t[i]["roi_x"], t[i]["roi_y"] = int(rng.integers(0, ws[i] - w + 1)), int(rng.integers(0, hs[i] - h + 1))
            t[i]["flip_h"], t[i]["flip_v"] = int(rng.integers(0, 2)), int(rng.integers(0, 2))
        if op == T.COLOR_CONTRAST:
            t["beta"] = rng.uniform(60, 200, n).astype(np.float32)
        rev = bool(rng.integers(0, 2))
        ref = O.pointwise(arena, t, out_w, out_h, op, dtype, layout, m, a, reverse_channels=rev)
        got = K.pointwise(d_arena, t, out_w, out_h, op, dtype, layout, m, a, reverse_channels=rev).cpu().numpy()
        assert np.array_equal(got.view(np.uint8), ref.view(np.uint8)), ("pointwise", seed, op, dtype, layout, rev, out_w, out_h)
    else:
        out_w, out_h = int(rng.integers(1, 300)), int(rng.integers(1, 200))
        t = S.warp_tables(rng, hs, ws, offs, out_w, out_h, angle=(-180.0, 180.0), scale=(0.3, 3.0), shift=20.0)
        ref = O.warp_affine(arena, t, out_w, out_h)
        got = K.warp_affine(d_arena, t, out_w, out_h).cpu().numpy()
        assert np.array_equal(got, ref), ("warp", seed, out_w, out_h)


@pytest.mark.parametrize("block", [0, 1, 2, 3])
def test_random_tables_match_the_oracle(cuda, block):
    for seed in range(block * 100000, block * 100000 + 120):
        _case(seed, cuda)

"""Normalize (mean / standard deviation over a chosen set of axes, statistics computed in scratch memory or given)
and Transpose against the CPU restatement: bit-exact, every axis mask, ragged windows, both output types."""
import numpy as np
import pytest

from oracle import pyoracle as O
import synthetic as S
from rocal_b200 import tables as T

pytestmark = pytest.mark.gpu


def _windows(rng, n, h_range, w_range, content="gradient_noise"):
    arena, hs, ws, offs = S.make_images(rng, n, h_range, w_range, content=content)
    t = np.zeros(n, dtype=T.POINTWISE_SAMPLE)
    t["src_offset"], t["src_stride"] = offs, ws * 3
    t["roi_x"] = rng.integers(0, 3, n)
    t["roi_y"] = rng.integers(0, 3, n)
    t["roi_w"], t["roi_h"] = ws - t["roi_x"] - rng.integers(0, 3, n), hs - t["roi_y"] - rng.integers(0, 3, n)
    return arena, t


@pytest.mark.parametrize("mask", [1, 2, 3, 4, 5, 6, 7])
def test_normalize_computed_statistics(cuda, mask):
    import torch
    from rocal_b200 import kernels as K
    rng = S.rng_for(60 + mask)
    arena, t = _windows(rng, 12, (20, 90), (24, 120))
    t[3]["roi_w"], t[3]["roi_h"] = 1, 1                      # a one-pixel window: every standard deviation over H, W is 0
    arena[int(t[5]["src_offset"]):int(t[5]["src_offset"]) + 90 * 120 * 3] = 77     # a constant image
    a = torch.from_numpy(arena).to(cuda)
    for dtype in (T.FP32, T.FP16):
        ref = O.normalize(arena, t, 120, 90, axis_mask=mask, scale=1.5, shift=-0.25, out_dtype=dtype)
        got = K.normalize(a, t, 120, 90, axis_mask=mask, scale=1.5, shift=-0.25, out_dtype=dtype).cpu().numpy()
        bits = np.uint32 if dtype == T.FP32 else np.uint16
        assert np.array_equal(got.view(bits), ref.view(bits)), (mask, dtype)
    # mean computed, standard deviation given, and the other way round
    ref = O.normalize(arena, t, 120, 90, axis_mask=mask, stddev=(50.0, 60.0, 70.0))
    assert np.array_equal(K.normalize(a, t, 120, 90, axis_mask=mask, stddev=(50.0, 60.0, 70.0)).cpu().numpy(), ref)
    ref = O.normalize(arena, t, 120, 90, axis_mask=mask, mean=(120.0, 110.0, 100.0))
    assert np.array_equal(K.normalize(a, t, 120, 90, axis_mask=mask, mean=(120.0, 110.0, 100.0)).cpu().numpy(), ref)


def test_normalize_given_statistics_and_scratch_reuse(cuda):
    import torch
    from rocal_b200 import kernels as K
    rng = S.rng_for(70)
    arena, t = _windows(rng, 16, (100, 224), (100, 224))
    a = torch.from_numpy(arena).to(cuda)
    mean, std = S.MEAN, S.STD
    ref = O.normalize(arena, t, 224, 224, mean=mean, stddev=std)
    got = K.normalize(a, t, 224, 224, mean=mean, stddev=std).cpu().numpy()      # no scratch at all
    assert np.array_equal(got, ref)
    # one scratch buffer, filled with junk, reused by launches with different masks: the call clears what it uses
    need = max(K.normalize_scratch_bytes(16, 224, 224, m) for m in (1, 3, 7))
    scratch = torch.full((need,), 0xAB, dtype=torch.uint8, device=cuda)
    for mask in (3, 1, 7, 3):
        ref = O.normalize(arena, t, 224, 224, axis_mask=mask)
        got = K.normalize(a, t, 224, 224, axis_mask=mask, scratch=scratch).cpu().numpy()
        assert np.array_equal(got, ref), mask
    # a scratch buffer that is too small is refused
    from rocal_b200._lib import Rb200Error
    with pytest.raises(Rb200Error):
        K.normalize(a, t, 224, 224, axis_mask=1, scratch=scratch[:1024])
    # per-channel statistics of the whole window agree with numpy's
    i = 2
    q = t[i]
    o = int(q["src_offset"])
    full = arena[o:o + (q["roi_h"] + q["roi_y"] + 2) * int(q["src_stride"])]
    rows = np.stack([full[(q["roi_y"] + y) * int(q["src_stride"]) + q["roi_x"] * 3:][:q["roi_w"] * 3] for y in range(q["roi_h"])])
    im = rows.reshape(q["roi_h"], q["roi_w"], 3).astype(np.float64)
    got = K.normalize(a, t, 224, 224, axis_mask=3).cpu().numpy()[i, :q["roi_h"], :q["roi_w"]]
    assert np.allclose(got, (im - im.mean((0, 1))) / im.std((0, 1)), atol=2e-5)


@pytest.mark.parametrize("perm", [(0, 1, 2), (2, 0, 1), (1, 0, 2), (0, 2, 1), (1, 2, 0), (2, 1, 0)])
def test_transpose(cuda, perm):
    import torch
    from rocal_b200 import kernels as K
    rng = S.rng_for(80)
    arena, t = _windows(rng, 6, (10, 60), (10, 70), content="noise")
    a = torch.from_numpy(arena).to(cuda)
    dims = [(60, 70, 3)[k] for k in perm]                    # the permuted maximum shape
    got = K.transpose(a, t, perm, dims).cpu().numpy()
    assert np.array_equal(got, O.transpose(arena, t, perm, dims))
    q = t[1]
    o, st = int(q["src_offset"]), int(q["src_stride"])
    win = np.stack([arena[o + (q["roi_y"] + y) * st + q["roi_x"] * 3:][:q["roi_w"] * 3] for y in range(q["roi_h"])]).reshape(q["roi_h"], q["roi_w"], 3)
    e = win.transpose(perm)
    assert np.array_equal(got[1][:e.shape[0], :e.shape[1], :e.shape[2]], e)

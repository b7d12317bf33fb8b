"""Run with RB200_LIBRARY pointing at the bounds-checking build of the library (librocal_b200_bounds.so).

Every image kernel is launched twice on the same batch. First with the true sizes: the results equal the oracle's and
the status word stays 0. Then with an arena size that cuts the last image in half: the kernel returns normally, its
status word reads 2, the last sample's output keeps the sentinel it was filled with (nothing of that sample was read),
the other samples are still exact, and a following launch with the true sizes is exact again. Nothing here faults or
waits: an out-of-bounds sample is skipped before any of it is touched."""
import sys

import numpy as np
import torch

from oracle import pyoracle as O
from rocal_b200 import kernels as K
from rocal_b200 import tables as T
from rocal_b200._lib import Rb200Error, lib, version as library_version
import synthetic as S


def main():
    version = library_version()
    assert version.endswith("+bounds"), "not the bounds-checking build: %s" % version
    cuda = torch.device("cuda:0")
    mul, add = S.normalize_tables()
    rng = S.rng_for(77)
    n = 5
    status = torch.zeros(1, dtype=torch.int32, device=cuda)

    def run(name, arena, offs, hs, ws, launch, reference, sentinel_dtype):
        """launch(d_arena, arena_bytes, out) -> out tensor; reference: numpy array [n, ...]."""
        d = torch.from_numpy(arena).to(cuda)
        status.zero_()
        got = launch(d, None, None)
        torch.cuda.synchronize()
        assert int(status.item()) == 0, (name, "true sizes", int(status.item()))
        assert np.array_equal(got.cpu().numpy().view(np.uint8), reference.view(np.uint8)), (name, "true sizes")
        cut = int(offs[-1]) + int(hs[-1]) * int(ws[-1]) * 3 // 2          # the last image is only half there
        out = torch.full_like(got, 77)
        launch(d, cut, out)
        torch.cuda.synchronize()
        assert int(status.item()) == 2, (name, "cut arena", int(status.item()))
        res = out.cpu().numpy()
        assert np.array_equal(res[:-1].view(np.uint8), reference[:-1].view(np.uint8)), (name, "samples inside the arena")
        assert np.all(res[-1] == 77), (name, "the sample outside the arena was written")
        status.zero_()
        again = launch(d, None, None)
        torch.cuda.synchronize()
        assert int(status.item()) == 0 and np.array_equal(again.cpu().numpy().view(np.uint8), reference.view(np.uint8)), (name, "after")
        assert lib.rb200k_device_status() == 0, name
        print("ok", name)

    # resample: row-streaming kernel (wide outputs), tile kernel (forced), direct kernel (no host table), triangular
    arena, hs, ws, offs = S.make_images(rng, n, (300, 420), (340, 500))
    t = S.classification_tables(rng, hs, ws, offs)
    ref = O.resample(arena, t, 224, 224, T.FP16, T.NCHW, mul, add)
    for name, kw in (("resample stream rows", {"path": 2}), ("resample stream pairs", {"path": 3}), ("resample tile", {"path": 1}),
                     ("resample direct", {"staged": False})):
        run(name, arena, offs, hs, ws,
            lambda d, ab, out, kw=kw: K.resample(d, t, 224, 224, T.FP16, T.NCHW, mul, add, fill_padding=False, out=out, status=status,
                                                 arena_bytes=ab, **kw), ref, np.float16)
    ref = O.resample(arena, t, 224, 224, T.UINT8, T.NHWC, interpolation=1)
    run("resample triangular", arena, offs, hs, ws,
        lambda d, ab, out: K.resample(d, t, 224, 224, T.UINT8, T.NHWC, fill_padding=False, out=out, status=status, arena_bytes=ab,
                                      interpolation=1), ref, np.uint8)

    # pointwise: vector kernel (width a multiple of 4) and scalar kernel
    arena, hs, ws, offs = S.make_images(rng, n, (64, 64), (96, 96), content="noise")
    tp = S.color_twist_tables(rng, hs, ws, offs)
    ref = O.pointwise(arena, tp, 96, 64, T.COLOR_TWIST)
    run("pointwise vector", arena, offs, hs, ws,
        lambda d, ab, out: K.pointwise(d, tp, 96, 64, T.COLOR_TWIST, fill_padding=False, out=out, status=status, arena_bytes=ab), ref,
        np.uint8)
    ref = O.pointwise(arena, tp, 95, 64, T.COLOR_BRIGHTNESS, T.FP32, T.NCHW, mul, add)
    run("pointwise scalar", arena, offs, hs, ws,
        lambda d, ab, out: K.pointwise(d, tp, 95, 64, T.COLOR_BRIGHTNESS, T.FP32, T.NCHW, mul, add, fill_padding=False, out=out,
                                       status=status, arena_bytes=ab), ref, np.float32)

    # affine gather
    arena, hs, ws, offs = S.make_images(rng, n, (120, 200), (150, 240))
    tw = S.warp_tables(rng, hs, ws, offs, 160, 128)
    ref = O.warp_affine(arena, tw, 160, 128)
    run("warp affine", arena, offs, hs, ws,
        lambda d, ab, out: K.warp_affine(d, tw, 160, 128, fill_padding=False, out=out, status=status, arena_bytes=ab), ref, np.uint8)

    # an output that is too small is refused before any launch, in every build
    d = torch.from_numpy(arena).to(cuda)
    try:
        K.warp_affine(d, tw, 160, 128, out_bytes=n * 160 * 128 * 3 - 1)
    except Rb200Error as e:
        assert "do not fit" in str(e), e
        print("ok output size refused")
    else:
        raise AssertionError("an undersized output was accepted")
    print("bounds build check passed")


if __name__ == "__main__":
    sys.exit(main())

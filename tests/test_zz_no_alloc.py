"""rb200k_normalize_static: Normalize for callers that cannot allocate device memory (a host language that binds the
C ABI without a CUDA binding of its own; a loader beside a framework that has claimed the whole device). Its
statistics live in a fixed 1 MiB array inside the library instead of a caller-provided scratch buffer.

The entry point is called through the C ABI (ctypes) twice in a row, with different data and different axis masks, so
that the second call finds the first one's leftovers in the shared array; both results must equal those of the
existing entry point rb200k_normalize bit for bit. A batch beyond the array's capacity must be refused with a clear
message. This file is collected last on purpose: a run that stops at the first failure has then run every other test."""
import ctypes

import numpy as np
import pytest

import synthetic as S
from rocal_b200 import tables as T

pytestmark = pytest.mark.gpu


def _windows(rng, n, h_range, w_range):
    arena, hs, ws, offs = S.make_images(rng, n, h_range, w_range)
    t = np.zeros(n, dtype=T.POINTWISE_SAMPLE)
    t["src_offset"], t["src_stride"], t["roi_w"], t["roi_h"] = offs, ws * 3, ws, hs
    return arena, t


def _call_static(arena_d, table, out_w, out_h, axis_mask, scale, shift, out_dtype, mean=None, stddev=None):
    """One call of the new entry point through ctypes: plain device pointers and PODs, nothing else."""
    import torch
    from rocal_b200 import kernels as K
    from rocal_b200._lib import NormalizeParams, lib
    lib.rb200k_normalize_static.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                            ctypes.POINTER(NormalizeParams), ctypes.c_void_p]
    lib.rb200k_normalize_static.restype = ctypes.c_int
    n = len(table)
    out = torch.empty((n, out_h, out_w, 3), dtype=torch.float32 if out_dtype == T.FP32 else torch.float16, device=arena_d.device)
    d_table = K.to_device_table(table, arena_d.device)
    p = K._normalize_params(out, out_w, out_h, out_dtype, axis_mask, mean, stddev, scale, shift, True)
    rc = lib.rb200k_normalize_static(arena_d.data_ptr(), d_table.data_ptr(), table.ctypes.data_as(ctypes.c_void_p), n,
                                     ctypes.byref(p), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return rc, out


def test_normalize_without_allocation_matches_the_scratch_entry_point(cuda):
    import torch
    from rocal_b200 import kernels as K
    from rocal_b200._lib import lib
    rng = S.rng_for(90)
    arena_a, ta = _windows(rng, 32, (60, 224), (60, 224))
    arena_b, tb = _windows(rng, 20, (40, 100), (40, 128))
    a, b = torch.from_numpy(arena_a).to(cuda), torch.from_numpy(arena_b).to(cuda)
    # first call: per-channel statistics (3 slots per sample)
    rc, got = _call_static(a, ta, 224, 224, 3, 1.0, 0.0, T.FP32)
    assert rc == 0, lib.rb200k_last_error().decode()
    ref = K.normalize(a, ta, 224, 224, axis_mask=3)
    assert torch.equal(got, ref)
    # second call right behind it: per-column statistics (3 * 128 slots per sample) over the first call's leftovers
    rc, got = _call_static(b, tb, 128, 100, 1, 2.0, -1.0, T.FP16)
    assert rc == 0, lib.rb200k_last_error().decode()
    ref = K.normalize(b, tb, 128, 100, axis_mask=1, scale=2.0, shift=-1.0, out_dtype=T.FP16)
    assert torch.equal(got.view(torch.int16), ref.view(torch.int16))
    # and the first case once more: identical again
    rc, got = _call_static(a, ta, 224, 224, 3, 1.0, 0.0, T.FP32)
    assert rc == 0 and torch.equal(got, K.normalize(a, ta, 224, 224, axis_mask=3))
    # given statistics never touch the array and have no limit
    rc, got = _call_static(a, ta, 224, 224, 0, 1.0, 0.0, T.FP32, mean=S.MEAN, stddev=S.STD)
    assert rc == 0 and torch.equal(got, K.normalize(a, ta, 224, 224, mean=S.MEAN, stddev=S.STD))


def test_normalize_without_allocation_refuses_what_does_not_fit(cuda):
    import torch
    from rocal_b200._lib import lib
    rng = S.rng_for(91)
    arena, t = _windows(rng, 4, (200, 224), (200, 224))
    a = torch.from_numpy(arena).to(cuda)
    # per-pixel statistics: 4 x 224 x 224 = 200 704 slots, more than the 65 536 the array holds
    rc, _ = _call_static(a, t, 224, 224, 4, 1.0, 0.0, T.FP32)
    assert rc == -3                                          # RB200_E_LIMIT
    msg = lib.rb200k_last_error().decode()
    assert "200704" in msg and "65536" in msg
    # the entry point still works afterwards
    rc, _ = _call_static(a, t, 224, 224, 7, 1.0, 0.0, T.FP32)
    assert rc == 0

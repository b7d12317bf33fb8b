"""Failure handling and buffer lifetimes on the GPU, without faulting, trapping or hanging anything:
  - a bounded wait that runs out (the producer of the kernel is told not to start one row's copy, and the wait limit
    is about a millisecond): the kernel returns, the status word reads 1, the next launch is bit-exact;
  - the same through the pipeline: rocalRun reports the batch as failed and the context goes on working;
  - zero-copy outputs consumed on another stream while later batches are produced (rb200_consumer_fence through the
    DLPack `stream` argument);
  - host buffers of batches that are fed far ahead of rocalRun stay alive until their batch has been returned;
  - contexts that are built, run and released leave neither device nor host memory behind;
  - contexts driven by concurrent threads."""
import gc

import numpy as np
import pytest

from oracle import pyoracle as O
import synthetic as S
from rocal_b200 import tables as T

pytestmark = pytest.mark.gpu

WAIT_CYCLES = 2_000_000      # about a millisecond of SM clock


def _dev(arena, cuda):
    import torch
    return torch.from_numpy(arena).to(cuda)


def _library_status():
    from rocal_b200._lib import lib
    return lib.rb200k_device_status()


@pytest.mark.parametrize("path", [2, 3])
def test_stream_kernel_wait_runs_out_and_recovers(cuda, path):
    """Both rings of the row-streaming kernel (2: distinct source rows, 3: tap-row pairs)."""
    import torch
    from rocal_b200 import kernels as K
    rng = S.rng_for(40)
    arena, hs, ws, offs = S.make_images(rng, 1, (400, 400), (500, 500))
    t = S.classification_tables(rng, hs, ws, offs)
    mul, add = S.normalize_tables()
    ref = O.resample(arena, t, 224, 224, T.FP32, T.NCHW, mul, add)
    a = _dev(arena, cuda)
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    assert _library_status() == 0
    # row 3 of every strip is never copied: the compute threads wait for it, give up after the limit, raise the
    # status word and the kernel returns
    K.resample(a, t, 224, 224, T.FP32, T.NCHW, mul, add, status=status, probe=(WAIT_CYCLES, 3), path=path)
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    assert _library_status() == 0                       # the launch had its own word
    status.zero_()
    got = K.resample(a, t, 224, 224, T.FP32, T.NCHW, mul, add, status=status, path=path).cpu().numpy()
    assert int(status.item()) == 0 and np.array_equal(got, ref)
    # without a word of its own the launch reports through the library-wide one, which reads 1 once and then 0
    K.resample(a, t, 224, 224, T.FP32, T.NCHW, mul, add, probe=(WAIT_CYCLES, 0), path=path)
    torch.cuda.synchronize()
    assert _library_status() == 1 and _library_status() == 0
    # a probe that skips nothing is an ordinary launch
    got = K.resample(a, t, 224, 224, T.FP32, T.NCHW, mul, add, status=status, probe=(WAIT_CYCLES * 1000, -1), path=path).cpu().numpy()
    assert int(status.item()) == 0 and np.array_equal(got, ref)


def test_pointwise_kernel_wait_runs_out_and_recovers(cuda):
    import torch
    from rocal_b200 import kernels as K
    rng = S.rng_for(41)
    arena, hs, ws, offs = S.make_images(rng, 2, (64, 64), (96, 96), content="noise")
    t = S.color_twist_tables(rng, hs, ws, offs)
    ref = O.pointwise(arena, t, 96, 64, T.COLOR_BRIGHTNESS)
    a = _dev(arena, cuda)
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    # row 0 of every tile is never copied (small batches run one-row tiles, so only row 0 exists everywhere)
    K.pointwise(a, t, 96, 64, T.COLOR_BRIGHTNESS, status=status, probe=(WAIT_CYCLES, 0))
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    status.zero_()
    got = K.pointwise(a, t, 96, 64, T.COLOR_BRIGHTNESS, status=status).cpu().numpy()
    assert int(status.item()) == 0 and np.array_equal(got, ref)
    assert _library_status() == 0


def _small_pipeline(n, depth=2):
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    pipe = Pipeline(batch_size=n, device_id=0, seed=3, prefetch_queue_depth=depth)
    with pipe:
        img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_UNCOMPRESSED, max_width=400, max_height=400)
        r = fn.resize(img, resize_shorter=256)
        out = fn.crop_mirror_normalize(r, crop=[224, 224], crop_pos_x=0.5, crop_pos_y=0.5, mean=list(S.MEAN), std=list(S.STD), mirror=0,
                                       output_layout=types.NCHW, output_dtype=types.FLOAT)
        pipe.set_outputs(out)
    pipe.build()
    return pipe


def _expected(arena, hs, ws, offs):
    n = len(hs)
    t = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
    for i in range(n):
        dw, dh = O.resize_dst_size(int(ws[i]), int(hs[i]), 256, 256, 2, cap_w=1536, cap_h=1536)
        x1, y1, cw, ch = O.crop_fixed(dw, dh, 224, 224, 0.5, 0.5)
        t[i]["src_offset"], t[i]["src_stride"] = offs[i], ws[i] * 3
        t[i]["roi_w"], t[i]["roi_h"], t[i]["dst_w"], t[i]["dst_h"] = ws[i], hs[i], dw, dh
        t[i]["crop_x"], t[i]["crop_y"], t[i]["crop_w"], t[i]["crop_h"] = x1, y1, cw, ch
    mul, add = S.normalize_tables()
    return O.resample(arena, t, 224, 224, T.FP32, T.NCHW, mul, add)


def test_pipeline_reports_a_batch_whose_kernel_gave_up(cuda):
    from rocal_b200 import _capi as C
    from rocal_b200.pipeline import RocalError
    rng = S.rng_for(42)
    n = 4
    pipe = _small_pipeline(n)
    arena, hs, ws, offs = S.make_images(rng, n, (260, 400), (260, 400))
    assert C.set_wait_probe(pipe._handle, WAIT_CYCLES, 2) == 0
    pipe.feed_ragged(arena, hs, ws, offs)
    with pytest.raises(RocalError) as e:
        pipe.run()
    assert "gave up" in str(e.value)
    assert C.set_wait_probe(pipe._handle, 0, -1) == 0
    for _ in range(2):                                   # the context is still usable and exact
        pipe.feed_ragged(arena, hs, ws, offs)
        pipe.run()
        assert np.array_equal(pipe.get_output_tensors()[0].numpy(), _expected(arena, hs, ws, offs))
    pipe.rocal_release()


def test_zero_copy_output_survives_later_batches_on_another_stream(cuda):
    """Batch k is exported zero-copy to a side stream that is kept busy; batches k+1 and k+2 are then produced (the
    ring has two slots, so k+2 reuses k's buffer). The copy the side stream makes of batch k afterwards must still
    be batch k: the pipeline waits for the consumer's stream before it writes the buffer again."""
    import torch
    rng = S.rng_for(43)
    n = 8
    pipe = _small_pipeline(n, depth=2)
    batches = [S.make_images(rng, n, (260, 400), (260, 400)) for _ in range(3)]
    side = torch.cuda.Stream()
    pipe.feed_ragged(*batches[0])
    pipe.run()
    with torch.cuda.stream(side):
        view = torch.from_dlpack(pipe.get_output_tensors()[0])      # hands `side` to the pipeline
        torch.cuda._sleep(400_000_000)                               # ~0.2 s of GPU time ahead of the read
        kept = view.clone()
    for k in (1, 2):
        pipe.feed_ragged(*batches[k])
        pipe.run()
    last = pipe.get_output_tensors()[0].numpy()
    side.synchronize()
    assert np.array_equal(kept.cpu().numpy(), _expected(*batches[0]))
    assert np.array_equal(last, _expected(*batches[2]))
    pipe.rocal_release()


def test_batches_fed_far_ahead_keep_their_host_buffers(cuda):
    """Six batches are fed before the first rocalRun and the caller drops its own references: every batch must still
    come out exact (the feed queue holds raw pointers into those buffers)."""
    rng = S.rng_for(44)
    n = 4
    pipe = _small_pipeline(n)
    pipe.set_upload_mode(pipe.UPLOAD_FOOTPRINT)
    expected = []
    for _ in range(6):
        arena, hs, ws, offs = S.make_images(rng, n, (260, 400), (260, 400))
        expected.append(_expected(arena, hs, ws, offs))
        pipe.feed_ragged(arena, hs, ws, offs)
        del arena, hs, ws, offs
    gc.collect()
    junk = [np.full(4_000_000, 255, dtype=np.uint8) for _ in range(8)]     # reuse freed memory, if any was freed
    for k in range(6):
        pipe.run()
        assert np.array_equal(pipe.get_output_tensors()[0].numpy(), expected[k]), k
    assert len(pipe._keepalive) == 0 and len(junk) == 8
    pipe.rocal_release()


def test_contexts_and_batches_leave_no_memory_behind(cuda):
    """Twelve contexts built, run for 120 batches each from pinned ragged arenas (the zero-copy path) and released: after
    the first one has set the high-water mark, neither the free device memory nor the process's resident set moves by
    more than a few megabytes (a minute of the same loop - 270 contexts, 81 000 batches - moved them by 0 and 0.3 MB)."""
    import os
    import torch
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline

    def rss():
        with open("/proc/%d/statm" % os.getpid()) as f:
            return int(f.read().split()[1]) * os.sysconf("SC_PAGE_SIZE")

    n = 32
    rng = S.rng_for(41)
    batches = []
    for _ in range(4):
        arena, hs, ws, offs = S.make_images(rng, n, (200, 400), (200, 400))
        batches.append((torch.from_numpy(arena).pin_memory(), hs, ws, offs))
    free0 = rss0 = None
    for c in range(12):
        pipe = Pipeline(batch_size=n, device_id=0, seed=7 + c, prefetch_queue_depth=2)
        with pipe:
            img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_UNCOMPRESSED, max_width=400, max_height=400)
            r = fn.resize(img, resize_shorter=128)
            out = fn.crop_mirror_normalize(r, crop=[112, 112], mean=list(S.MEAN), std=list(S.STD), mirror=fn.random.coin_flip(),
                                           output_layout=types.NCHW, output_dtype=types.FLOAT16)
            pipe.set_outputs(out)
        pipe.build()
        for i in range(120):
            ap_, hs, ws, offs = batches[i % 4]
            pipe.feed_ragged(ap_, hs, ws, offs)
            pipe.run()
            o = torch.from_dlpack(pipe.get_output_tensors()[0])
            assert o.shape == (n, 3, 112, 112)
        del o
        pipe.rocal_release()
        torch.cuda.synchronize()
        gc.collect()
        if free0 is None:
            free0, rss0 = torch.cuda.mem_get_info()[0], rss()
    assert abs(free0 - torch.cuda.mem_get_info()[0]) <= 8 << 20
    assert rss() - rss0 <= 32 << 20


def test_contexts_in_concurrent_threads(cuda):
    """The reference's threading rule (tests/cpp_api/dataloader_multithread/dataloader_multithread.cpp:54-66: one context per
    thread, creation under a mutex): four
    contexts, created one after the other, each driven by a thread of its own for 25 batches at the same time - different
    batch sizes, output types and mirror settings, pageable and pinned arenas. Every batch of every thread equals the
    oracle's bits; no thread sees another's error text."""
    import threading
    import torch
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    mul, add = S.normalize_tables()
    jobs = []
    for k, (n, dtype, mirror, pinned) in enumerate(((16, T.FP32, 0, True), (24, T.FP16, 1, False), (8, T.FP32, 1, True),
                                                     (32, T.FP16, 0, True))):
        rng = S.rng_for(42, k)
        arena, hs, ws, offs = S.make_images(rng, n, (150, 400), (150, 400))
        t = np.zeros(n, dtype=T.RESAMPLE_SAMPLE)
        for i in range(n):
            dw, dh = O.resize_dst_size(int(ws[i]), int(hs[i]), 128, 128, 2, cap_w=768, cap_h=768)
            x1, y1, cw, ch = O.crop_fixed(dw, dh, 112, 112, 0.5, 0.5)
            t[i]["src_offset"], t[i]["src_stride"] = offs[i], ws[i] * 3
            t[i]["roi_w"], t[i]["roi_h"] = ws[i], hs[i]
            t[i]["dst_w"], t[i]["dst_h"] = dw, dh
            t[i]["crop_x"], t[i]["crop_y"], t[i]["crop_w"], t[i]["crop_h"] = x1, y1, cw, ch
            t[i]["mirror"] = mirror
        ref = O.resample(arena, t, 112, 112, dtype, T.NCHW, mul, add)
        pipe = Pipeline(batch_size=n, device_id=0, seed=3 + k, prefetch_queue_depth=2)      # created serially
        with pipe:
            img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_UNCOMPRESSED, max_width=400, max_height=400)
            r = fn.resize(img, resize_shorter=128)
            out = fn.crop_mirror_normalize(r, crop=[112, 112], mean=list(S.MEAN), std=list(S.STD), mirror=mirror,
                                           output_layout=types.NCHW, output_dtype=types.FLOAT if dtype == T.FP32 else types.FLOAT16)
            pipe.set_outputs(out)
        pipe.build()
        src = torch.from_numpy(arena).pin_memory() if pinned else arena
        jobs.append((pipe, src, hs, ws, offs, ref))
    failures = []
    start = threading.Barrier(len(jobs))

    def drive(k):
        pipe, src, hs, ws, offs, ref = jobs[k]
        try:
            start.wait()
            for batch in range(25):
                pipe.feed_ragged(src, hs, ws, offs)
                pipe.run()
                got = torch.from_dlpack(pipe.get_output_tensors()[0]).cpu().numpy()
                if not np.array_equal(got.view(np.uint8), ref.view(np.uint8)):
                    failures.append("context %d, batch %d differs from the oracle" % (k, batch))
                    return
        except Exception as e:          # noqa: BLE001 - reported through the list below
            failures.append("context %d: %r" % (k, e))

    threads = [threading.Thread(target=drive, args=(k,)) for k in range(len(jobs))]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    for pipe, *_ in jobs:
        pipe.rocal_release()
    assert not failures, failures
    assert _library_status() == 0

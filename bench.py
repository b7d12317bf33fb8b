"""Benchmark of the augmentation hot path: fused Resize(shorter->256, bilinear) + CropMirrorNormalize
(224x224, fp16 NCHW) over batches of 1024 variable-size uint8 images per GPU (BASELINE configs[1]).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 0|2|3|4] [--op NAME[,NAME...]]

One step = one pass of the path over one batch. Rank 0 prints one JSON line:
  value     images/s with the batch already resident in HBM (CUDA events, max over ranks)
  e2e       images/s through the public pipeline API (external source -> rocalResize -> rocalCropMirrorNormalize
            -> rocalRun) fed from pinned HOST memory: every feed, the host-to-device traffic of the batch and its
            tables, the kernel, and a D2H read-back of one output image lie inside the timed region (the clock
            starts before the first feed; wall clock between device syncs). One image comes back per step because
            the outputs are consumed on the device (DLPack), by design.
  roofline  algorithmic bytes of the resample kernel / its mean launch time, against the measured
            HBM copy bandwidth (MEASURED_PEAKS.json, else the 6650 GB/s fallback)
  cpu_baseline  the CPU oracle (OpenMP over samples) on whole passes over the same batch
  per_rank  every rank's own device-resident and end-to-end times, uploaded bytes, host-link rate during the e2e run and
            the rate of plain pinned-to-device copies issued by all ranks at once (the link's ceiling at this GPU count)
  other_configs (one GPU only) short runs of configs[0], [2], [3], [4]: ms per step, images/s, roofline fraction, e2e
`--impl reference` times the CPU implementation alone on rank 0's whole batch (the oracle port: the reference's own
pixel code lives in the RPP library, which is not available) and prints the same line shape; it does not load the
CUDA library.
`--config 0|2|3|4` prints the full line for one of the other benchmark configurations (one GPU, our arm only).
`--op NAME` prints one line per operator-level case (device-resident launches through the kernel C-ABI; the cases the
ncu summaries under profiles/ were captured on).
Under torchrun every rank owns one GPU and one shard of the synthetic dataset
(shard i of S = indices [floor(N*i/S), floor(N*(i+1)/S)), rocAL's reader partitioning); no
data-path collective is used.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BATCH = 1024
OUT = 224
RESIZE_SHORTER = 256
H_RANGE = (300, 1080)
W_RANGE = (300, 1080)
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one resample launch, per image, from
#   ncu --set full --clock-control none -k regex:resample_stream_pairs -s 3 -c 1 python bench.py --batch 512 --steps 3 --warmup 3 --no-cpu-baseline --no-other-configs
# (a 512-image launch: traffic grows in proportion to the images processed, so it is scaled by the batch size).
NCU_TRAFFIC_BYTES_PER_IMAGE = (337212416 + 128423936) / 512.0


def peak_hbm():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return FALLBACK_HBM_GBS, "fallback"


def algorithmic_bytes(t):
    """Per launch: source footprint 3*(ceil(224/s)+1)^2 with s = 256/min(H,W), plus the fp16 output."""
    short = np.minimum(t["roi_w"], t["roi_h"]).astype(np.float64)
    s = RESIZE_SHORTER / short
    fp = 3.0 * (np.ceil(OUT / s) + 1.0) ** 2
    return float(fp.sum() + len(t) * 3 * OUT * OUT * 2)


def shard_range(total, shard_id, num_shards):
    return (total * shard_id) // num_shards, (total * (shard_id + 1)) // num_shards


def make_shard(rank, world):
    """The global dataset has BATCH*world images; this rank builds only its own shard (seeded per index block)."""
    import synthetic as S
    lo, hi = shard_range(BATCH * world, rank, world)
    rng = np.random.Generator(np.random.PCG64([1235, lo]))
    arena, hs, ws, offs = S.make_images(rng, hi - lo, H_RANGE, W_RANGE)
    t = S.classification_tables(rng, hs, ws, offs, RESIZE_SHORTER, OUT)
    return arena, t


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            f = [x.strip() for x in s.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_baseline(arena, t, seconds_target=10.0):
    """Oracle (CPU restatement, OpenMP over samples): whole passes over this batch for about seconds_target."""
    from oracle import pyoracle as O
    import synthetic as S
    cores = os.cpu_count() or 1
    O.set_threads(cores)
    mul, add = S.normalize_tables()
    n = len(t)
    O.resample(arena, t, OUT, OUT, S.T.FP16, S.T.NCHW, mul, add)   # warm-up
    reps, elapsed = 0, 0.0
    t0 = time.perf_counter()
    while elapsed < seconds_target and reps < 200:
        O.resample(arena, t, OUT, OUT, S.T.FP16, S.T.NCHW, mul, add)
        reps += 1
        elapsed = time.perf_counter() - t0
    return {"value": n * reps / elapsed, "unit": "images/s", "cores": cores, "kind": "port",
            "sample": "the %d-image batch x %d passes, OpenMP over samples" % (n, reps)}


def run_reference(args, rank, world):
    """CPU arm: the oracle port with all host threads on rank 0's whole batch, one pass per step. Loads neither
    torch nor the CUDA library."""
    if rank != 0:
        return
    from oracle import pyoracle as O
    import synthetic as S
    cores = os.cpu_count() or 1
    O.set_threads(cores)
    arena, t = make_shard(0, world)
    n = len(t)
    mul, add = S.normalize_tables()
    for _ in range(max(1, min(args.warmup, 3))):
        O.resample(arena, t, OUT, OUT, S.T.FP16, S.T.NCHW, mul, add)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.resample(arena, t, OUT, OUT, S.T.FP16, S.T.NCHW, mul, add)
    dt = time.perf_counter() - t0
    value = n * args.steps / dt
    line = {"impl": "reference", "metric": "augmented images/sec", "value": value, "unit": "images/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(world),
            "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": "port",
                             "sample": "rank 0's whole %d-image batch per step on the host cores, OpenMP over samples; "
                                       "the reference's own pixel code (RPP) is not available" % n},
            "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def workload_config(world):
    return {"workload": "configs[1]: Resize(shorter=256, bilinear)+CropMirrorNormalize 224x224 fp16 NCHW, "
                        "batch 1024/GPU of uint8 RGB images with H,W~U[300,1080]",
            "batch_per_gpu": BATCH, "sharding": "shard_id/num_shards over %d GPU(s), no collective" % world,
            "l2": "inputs (~1.4 GB/batch) larger than L2"}


# ---------------------------------------------------------------------------------------------------------------
# The other BASELINE configurations (--config 0|2|3|4): the same three measurements on one GPU - device-resident
# kernels through the kernel C-ABI, end to end through the pipeline API from pinned host memory, and the CPU port
# on a bounded slice - printed in the same line shape. They are not part of the default run.
# ---------------------------------------------------------------------------------------------------------------

def _time_cpu(fn, images_per_call, seconds_target=4.0):
    fn()
    reps, t0, elapsed = 0, time.perf_counter(), 0.0
    while elapsed < seconds_target and reps < 50:
        fn()
        reps += 1
        elapsed = time.perf_counter() - t0
    return images_per_call * reps / elapsed, reps


def measure_config(cfg, steps, warmup, e2e_steps, with_cpu, sampler=None, fast=False):
    """Device-resident launches (CUDA events), the pipeline API from pinned host memory and, if asked, the CPU port
    for one of the configurations 0, 2, 3, 4 on cuda:0. Returns the bench line as a dict."""
    import torch
    import rocal_b200
    from oracle import pyoracle as O
    from rocal_b200 import fn, types
    from rocal_b200 import kernels as K
    import synthetic as S
    from rocal_b200 import tables as T
    from rocal_b200.pipeline import Pipeline
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream()
    mul, add = S.normalize_tables()
    cores = os.cpu_count() or 1
    O.set_threads(cores)
    peak, peak_src = peak_hbm()

    # Every configuration rotates over enough distinct batches that one pass exceeds L2 (126 MB).
    resident, feeders, extra, image_only = [], [], {}, []
    if cfg == 0:
        n, rot, name = 64, 6, "configs[0]: Resize(shorter=256)+CropMirrorNormalize 224x224 fp32 NCHW, batch 64, H,W~U[256,512]"
        kernel = "resample_stream_pairs_kernel<float,NCHW,normalize>"
        pipe = Pipeline(batch_size=n, device_id=0, seed=1234, prefetch_queue_depth=2)
        with pipe:
            img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_UNCOMPRESSED, max_width=512, max_height=512)
            r = fn.resize(img, resize_shorter=256)
            outn = fn.crop_mirror_normalize(r, crop=[224, 224], mean=list(S.MEAN), std=list(S.STD), mirror=fn.random.coin_flip(),
                                            output_layout=types.NCHW, output_dtype=types.FLOAT)
            pipe.set_outputs(outn)
        pipe.build()
        algo = 0.0
        for k in range(rot):
            rng = S.rng_for(0, 100 + k)
            arena, hs, ws, offs = S.make_images(rng, n, (256, 512), (256, 512))
            t = S.classification_tables(rng, hs, ws, offs)
            short = np.minimum(hs, ws).astype(np.float64)
            algo = float((3.0 * (np.ceil(224 / (256 / short)) + 1) ** 2).sum() + n * 3 * 224 * 224 * 4)
            a, dt = torch.from_numpy(arena).to(dev), K.to_device_table(t, dev)
            o = torch.empty((n, 3, 224, 224), dtype=torch.float32, device=dev)
            # every rotating batch has buffers of its own, so its launch may overlap the tail of the one before
            resident.append(lambda a=a, t=t, dt=dt, o=o: K.resample(a, t, 224, 224, T.FP32, T.NCHW, mul, add, fill_padding=False, out=o,
                                                                      d_samples=dt, stream=stream, overlap=True))
            ap_ = torch.from_numpy(arena).pin_memory()
            anchors = (rng.random(n).astype(np.float32), rng.random(n).astype(np.float32))
            feeders.append(lambda ap_=ap_, hs=hs, ws=ws, offs=offs, anchors=anchors: (pipe.set_crop_anchors(outn, *anchors),
                                                                                       pipe.feed_ragged(ap_, hs, ws, offs)))
            if k == 0:
                sl = np.ascontiguousarray(t[:32])
                cpu_fn, cpu_n = (lambda arena=arena, sl=sl: O.resample(arena, sl, 224, 224, T.FP32, T.NCHW, mul, add)), 32
        h2d_whole = None
    elif cfg == 2:
        n, rot, name = 256, 4, "configs[2]: ColorTwist(alpha,beta,hue,sat)+Flip u8 HWC 224x224, batch 256"
        kernel = "pointwise_vec_kernel<uint8,NHWC,twist>"
        if fast:
            name += " [RB200_ARITH_FAST: every byte within one level of the exact arithmetic]"
            kernel = "pointwise_vec_kernel<uint8,NHWC,twist_fast>"
        pipe = Pipeline(batch_size=n, device_id=0, seed=1234, prefetch_queue_depth=2)
        with pipe:
            img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_UNCOMPRESSED, max_width=224, max_height=224)
            ct = fn.color_twist(img, brightness=fn.random.uniform(range=(0.6, 1.4)), contrast=fn.random.uniform(range=(0.6, 1.4)),
                                hue=fn.random.uniform(range=(-30.0, 30.0)), saturation=fn.random.uniform(range=(0.5, 1.5)))
            outn = fn.flip(ct, horizontal=fn.random.coin_flip(), vertical=0)
            pipe.set_outputs(outn)
        pipe.build()
        pipe.set_arithmetic(1 if fast else 0)
        algo = float(n * 2 * 3 * 224 * 224)
        for k in range(rot):
            rng = S.rng_for(2, 100 + k)
            arena, hs, ws, offs = S.make_images(rng, n, (224, 224), (224, 224), content="noise")
            t = S.color_twist_tables(rng, hs, ws, offs)
            a, dt = torch.from_numpy(arena).to(dev), K.to_device_table(t, dev)
            o = torch.empty((n, 224, 224, 3), dtype=torch.uint8, device=dev)
            resident.append(lambda a=a, t=t, dt=dt, o=o: K.pointwise(a, t, 224, 224, T.COLOR_TWIST, out=o, d_samples=dt, fill_padding=False,
                                                                       stream=stream, arith=1 if fast else 0, overlap=True))
            ap_ = torch.from_numpy(arena).pin_memory()
            feeders.append(lambda ap_=ap_, hs=hs, ws=ws, offs=offs: pipe.feed_ragged(ap_, hs, ws, offs))
            if k == 0:
                sl = np.ascontiguousarray(t[:64])
                cpu_fn, cpu_n = (lambda arena=arena, sl=sl: O.pointwise(arena, sl, 224, 224, T.COLOR_TWIST)), 64
    elif cfg == 3:
        n, rot, name = 128, 2, "configs[3]: WarpAffine (rotation +-45 deg, scale 0.8-1.2, shift +-32 px) u8 480x640, batch 128"
        kernel = "warp_affine_kernel"
        pipe = Pipeline(batch_size=n, device_id=0, seed=1234, prefetch_queue_depth=2)
        with pipe:
            img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_UNCOMPRESSED, max_width=640, max_height=480)
            outn = fn.warp_affine(img, dest_width=640, dest_height=480, matrix=[1.0, 0.0, 0.0, 1.0, 0.0, 0.0])
            pipe.set_outputs(outn)
        pipe.build()
        algo = float(n * 2 * 3 * 480 * 640)
        for k in range(rot):
            rng = S.rng_for(3, 100 + k)
            arena, hs, ws, offs = S.make_images(rng, n, (480, 480), (640, 640))
            t = S.warp_tables(rng, hs, ws, offs, 640, 480)
            a, dt = torch.from_numpy(arena).to(dev), K.to_device_table(t, dev)
            o = torch.empty((n, 480, 640, 3), dtype=torch.uint8, device=dev)
            resident.append(lambda a=a, t=t, dt=dt, o=o: K.warp_affine(a, t, 640, 480, out=o, d_samples=dt, stream=stream, overlap=True))
            ap_ = torch.from_numpy(arena).pin_memory()
            feeders.append(lambda ap_=ap_, hs=hs, ws=ws, offs=offs, m=t["m"].copy(): (pipe.set_affine(outn, m), pipe.feed_ragged(ap_, hs, ws, offs)))
            if k == 0:
                sl = np.ascontiguousarray(t[:16])
                cpu_fn, cpu_n = (lambda arena=arena, sl=sl: O.warp_affine(arena, sl, 640, 480)), 16
    else:
        n, rot, name = 128, 2, ("configs[4]: SSDRandomCrop -> Resize 300x300 -> CropMirrorNormalize fp32 NCHW + BoxEncoder "
                                "(8732 anchors, criteria 0.5, offset), batch 128, H,W~U[300,800], 1-50 boxes")
        kernel = "resample_stream_pairs_kernel<float,NCHW,normalize> (+ box_encode_kernel<4>)"
        anchors_np = S.ssd300_anchors()
        anchors_d = torch.from_numpy(anchors_np).to(dev)
        meta_stream = torch.cuda.Stream()
        pipe = Pipeline(batch_size=n, device_id=0, seed=1234, prefetch_queue_depth=2)
        with pipe:
            img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_UNCOMPRESSED, max_width=800, max_height=800)
            c = fn.ssd_random_crop(img)
            r = fn.resize(c, resize_width=300, resize_height=300, scaling_mode=types.SCALING_MODE_STRETCH)
            outn = fn.crop_mirror_normalize(r, crop=[300, 300], crop_pos_x=0.0, crop_pos_y=0.0, mean=list(S.MEAN), std=list(S.STD),
                                            mirror=fn.random.coin_flip(), output_layout=types.NCHW, output_dtype=types.FLOAT)
            fn.box_encoder(anchors=anchors_np, criteria=0.5, means=[0, 0, 0, 0], stds=[0.1, 0.1, 0.2, 0.2], offset=True, scale=1.0)
            pipe.set_outputs(outn)
        pipe.build()
        algo = 0.0
        for k in range(rot):
            rng = S.rng_for(4, 100 + k)
            arena, hs, ws, offs = S.make_images(rng, n, (300, 800), (300, 800))
            boxes, labels, boffs = S.random_boxes(rng, n)
            crops, cb, cl, co = S.ssd_random_crop(rng, boxes, labels, boffs)
            t = S.ssd_resample_tables(rng, hs, ws, offs, crops)
            algo = float((3.0 * t["roi_w"].astype(np.float64) * t["roi_h"]).sum() + n * 3 * 300 * 300 * 4)
            a, dt = torch.from_numpy(arena).to(dev), K.to_device_table(t, dev)
            o = torch.empty((n, 3, 300, 300), dtype=torch.float32, device=dev)
            bd, ld, od = torch.from_numpy(cb).to(dev), torch.from_numpy(cl).to(dev), torch.from_numpy(co).to(dev)
            eb = torch.empty((n, 8732, 4), dtype=torch.float32, device=dev)
            el = torch.empty((n, 8732), dtype=torch.int32, device=dev)

            def both(a=a, t=t, dt=dt, o=o, bd=bd, ld=ld, od=od, eb=eb, el=el):
                # the two kernels are independent: the encoder runs on a second stream beside the image chain, as in
                # the pipeline; the timed stream joins the second one once, before the closing event
                K.resample(a, t, 300, 300, T.FP32, T.NCHW, mul, add, fill_padding=False, out=o, d_samples=dt, stream=stream,
                           overlap=True)
                K.box_encode(bd, ld, od, anchors_d, 0.5, (0, 0, 0, 0), (0.1, 0.1, 0.2, 0.2), True, 1.0, 50, eb, el, stream=meta_stream)
            resident.append(both)
            image_only.append(lambda a=a, t=t, dt=dt, o=o: K.resample(a, t, 300, 300, T.FP32, T.NCHW, mul, add, fill_padding=False, out=o,
                                                                        d_samples=dt, stream=stream, overlap=True))
            ap_ = torch.from_numpy(arena).pin_memory()
            feeders.append(lambda ap_=ap_, hs=hs, ws=ws, offs=offs, boxes=boxes, labels=labels, boffs=boffs:
                           (pipe.feed_boxes(boxes, labels, np.diff(boffs)), pipe.feed_ragged(ap_, hs, ws, offs)))
            if k == 0:
                sl = np.ascontiguousarray(t[:32])
                so = np.ascontiguousarray(co[:33] - co[0])

                def cpu_fn(arena=arena, sl=sl, cb=cb, cl=cl, so=so):
                    O.resample(arena, sl, 300, 300, T.FP32, T.NCHW, mul, add)
                    O.box_encode(cb[:so[-1]], cl[:so[-1]], so, anchors_np, 0.5, (0, 0, 0, 0), (0.1, 0.1, 0.2, 0.2), True, 1.0)
                cpu_n = 32
        extra["algorithmic_bytes_note"] = "image chain only; the box encoder writes 174 640 B per sample more"

    rotn = len(resident)
    own_sampler = sampler is None
    if own_sampler:
        sampler = ClockSampler(0)
        sampler.start()
    t_warm, warm = time.perf_counter(), 0
    while warm < max(warmup, 3) or time.perf_counter() - t_warm < (0.6 if own_sampler else 0.05):
        resident[warm % rotn]()
        warm += 1
        if warm % 64 == 0:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    launches0 = rocal_b200.launch_count()
    # one event on each side of the K back-to-back steps: an event between two launches would make every launch wait
    # for the record before it (no overlap of one launch's ramp-up with its predecessor's tail)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    if cfg == 4:
        meta_stream.wait_stream(stream)
    for i in range(steps):
        resident[i % rotn]()
    if cfg == 4:
        stream.wait_stream(meta_stream)
    ev1.record(stream)
    torch.cuda.synchronize()
    launches = rocal_b200.launch_count() - launches0
    total_ms = ev0.elapsed_time(ev1)
    mean_launch_ms = total_ms / steps
    if image_only:
        # configs[4]: the image chain without the encoder beside it (the batch time above is the encoder's, the longer of
        # the two concurrent kernels)
        ev0.record(stream)
        for i in range(steps):
            image_only[i % rotn]()
        ev1.record(stream)
        torch.cuda.synchronize()
        chain_ms = ev0.elapsed_time(ev1) / steps
        extra["image_chain_alone"] = {"ms_per_step": chain_ms, "achieved_gbs": algo / (chain_ms * 1e-3) / 1e9,
                                      "frac": algo / (chain_ms * 1e-3) / 1e9 / peak}

    # end to end: pinned host arena -> pipeline -> D2H of one output sample; the clock starts before the first feed
    outs0 = None
    for k in range(2):
        feeders[k % rotn]()
        pipe.run()
        if outs0 is None:       # pinned landing place of the one sample read back per step
            outs0 = torch.empty_like(torch.from_dlpack(pipe.get_output_tensors()[0])[0], device="cpu").pin_memory()
    torch.cuda.synchronize()
    h2d0 = pipe.h2d_bytes()
    te = time.perf_counter()
    feeders[0]()
    for i in range(e2e_steps):
        if i < e2e_steps - 1:
            feeders[(i + 1) % rotn]()
        pipe.run()
        outs0.copy_(torch.from_dlpack(pipe.get_output_tensors()[0])[0], non_blocking=False)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - te) * 1e3
    h2d_per_step = (pipe.h2d_bytes() - h2d0) / e2e_steps
    clocks = sampler.stop() if own_sampler else None
    pipe.rocal_release()

    achieved = algo / (mean_launch_ms * 1e-3) / 1e9
    line = {"metric": "augmented images/sec", "value": n * steps / (total_ms * 1e-3), "unit": "images/s", "n_gpus": 1, "steps": steps,
            "warmup": max(warmup, 3), "ms_per_step": mean_launch_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": dict({"workload": name, "batch_per_gpu": n,
                            "l2": "rotates over %d batches so that one pass over inputs and outputs exceeds L2" % rotn}, **extra),
            "e2e": {"value": n * e2e_steps / (e2e_ms * 1e-3), "unit": "images/s", "h2d_bytes_per_step": int(h2d_per_step),
                    "d2h_bytes_per_step": int(outs0.numel() * outs0.element_size()), "steps": e2e_steps,
                    "d2h_note": "one sample per step: outputs are consumed on the device (DLPack)"},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                         "frac": achieved / peak, "algorithmic_bytes_per_launch": algo, "launch_ms": mean_launch_ms, "traffic": None}}
    if clocks is not None:
        line["clocks"] = dict(clocks, window="warm-up + timed steps + end-to-end steps")
    if with_cpu:
        cpu_value, cpu_reps = _time_cpu(cpu_fn, cpu_n)
        line["cpu_baseline"] = {"value": cpu_value, "unit": "images/s", "cores": cores, "kind": "port",
                                "sample": "%d images x %d passes, OpenMP over samples" % (cpu_n, cpu_reps)}
    return line


def other_configs(sampler):
    """Short runs of configs[0], [2], [3], [4] on cuda:0 for the default line: what each costs and where it stands
    against the roofline."""
    out = []
    for cfg, fast in ((0, False), (2, False), (2, True), (3, False), (4, False)):
        r = measure_config(cfg, steps=400, warmup=20, e2e_steps=12, with_cpu=False, sampler=sampler, fast=fast)
        out.append({"workload": r["config"]["workload"], "ms_per_step": r["ms_per_step"], "value": r["value"], "unit": r["unit"],
                    "roofline": {"kernel": r["roofline"]["kernel"], "frac": r["roofline"]["frac"], "achieved": r["roofline"]["achieved"],
                                 "algorithmic_bytes_per_launch": r["roofline"]["algorithmic_bytes_per_launch"]},
                    "e2e": {"value": r["e2e"]["value"], "h2d_bytes_per_step": r["e2e"]["h2d_bytes_per_step"]},
                    "gpu_launches": r["gpu_launches"]})
        if "image_chain_alone" in r["config"]:
            out[-1]["image_chain_alone"] = r["config"]["image_chain_alone"]
    return out



def _time_launches(fn_list, steps, warmup=5):
    """fn_list: one launch closure per rotating batch. Returns mean ms per launch."""
    import torch
    k = len(fn_list)
    for i in range(warmup):
        fn_list[i % k]()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn_list[i % k]()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def run_ops(args):
    """Operator-level cases (--op a,b,...): cfg0, color_twist, brightness, contrast, flip, warp, ssd_chain, box_encoder,
    box_matcher, triangular, jpeg_e2e, jpeg_slice_e2e. One JSON line each: images/s, mean launch time (CUDA events on
    the launching stream), algorithmic bytes per launch and the fraction of the measured HBM copy bandwidth. Every case
    rotates through enough distinct batches that one pass over its inputs and outputs exceeds the 126 MB L2.
    --batch overrides the batch of the colour cases."""
    import torch
    from rocal_b200 import kernels as K
    import synthetic as S
    from rocal_b200 import tables as T
    dev = torch.device("cuda:0")
    peak, peak_src = peak_hbm()
    mul, add = S.normalize_tables()
    # the rotating batches are independent of one another (separate inputs and outputs): their launches may overlap
    ov = not args.no_overlap

    def report(name, n, ms, algo_bytes, extra=None):
        line = {"op": name, "images_per_launch": n, "launch_ms": ms, "images_per_s": n / (ms * 1e-3),
                "algorithmic_bytes_per_launch": algo_bytes, "achieved_gbs": algo_bytes / (ms * 1e-3) / 1e9,
                "peak_gbs": peak, "peak_source": peak_src, "frac": algo_bytes / (ms * 1e-3) / 1e9 / peak}
        if extra:
            line.update(extra)
        print(json.dumps(line), flush=True)

    for op in args.op.split(","):
        if op == "cfg0":
            n, rot = 64, 6
            fns, algo = [], 0.0
            for r in range(rot):
                rng = S.rng_for(0, 100 + r)
                arena, hs, ws, offs = S.make_images(rng, n, (256, 512), (256, 512))
                t = S.classification_tables(rng, hs, ws, offs)
                short = np.minimum(hs, ws).astype(np.float64)
                algo = float((3.0 * (np.ceil(224 / (256 / short)) + 1) ** 2).sum() + n * 3 * 224 * 224 * 4)
                a, dt = torch.from_numpy(arena).to(dev), K.to_device_table(t, dev)
                out = torch.empty((n, 3, 224, 224), dtype=torch.float32, device=dev)
                fns.append(lambda a=a, t=t, dt=dt, out=out: K.resample(a, t, 224, 224, T.FP32, T.NCHW, mul, add, fill_padding=False, out=out, d_samples=dt,
                                                                       overlap=ov, strip_rows=args.strip_rows))
            report("cfg0 resize+CMN fp32 NCHW (batch 64, 256..512 px)", n, _time_launches(fns, args.steps), algo)
        elif op in ("color_twist", "brightness", "contrast", "flip"):
            n, rot = args.batch or 256, 4
            code = {"color_twist": T.COLOR_TWIST, "brightness": T.COLOR_BRIGHTNESS, "contrast": T.COLOR_CONTRAST, "flip": T.COLOR_NONE}[op]
            fns = []
            for r in range(rot):
                rng = S.rng_for(2, 100 + r)
                arena, hs, ws, offs = S.make_images(rng, n, (224, 224), (224, 224), content="noise")
                t = S.color_twist_tables(rng, hs, ws, offs)
                a, dt = torch.from_numpy(arena).to(dev), K.to_device_table(t, dev)
                out = torch.empty((n, 224, 224, 3), dtype=torch.uint8, device=dev)
                fns.append(lambda a=a, t=t, dt=dt, out=out: K.pointwise(a, t, 224, 224, code, out=out, d_samples=dt, fill_padding=False,
                                                                        arith=1 if args.fast else 0, overlap=ov))
            report("cfg2 %s(+flip) u8 HWC 224x224 (batch %d)%s" % (op, n, " fast arithmetic" if args.fast else ""), n, _time_launches(fns, args.steps), n * 2 * 3 * 224 * 224)
        elif op == "warp":
            n, rot = 128, 2
            fns = []
            for r in range(rot):
                rng = S.rng_for(3, 100 + r)
                arena, hs, ws, offs = S.make_images(rng, n, (480, 480), (640, 640))
                t = S.warp_tables(rng, hs, ws, offs, 640, 480)
                a, dt = torch.from_numpy(arena).to(dev), K.to_device_table(t, dev)
                out = torch.empty((n, 480, 640, 3), dtype=torch.uint8, device=dev)
                fns.append(lambda a=a, t=t, dt=dt, out=out: K.warp_affine(a, t, 640, 480, out=out, d_samples=dt, overlap=ov))
            report("cfg3 warp_affine u8 480x640 (batch 128)", n, _time_launches(fns, args.steps), n * 2 * 3 * 480 * 640)
        elif op == "ssd_chain":
            n, rot = 128, 2
            fns, algo = [], 0.0
            for r in range(rot):
                rng = S.rng_for(4, 100 + r)
                arena, hs, ws, offs = S.make_images(rng, n, (300, 800), (300, 800))
                boxes, labels, boffs = S.random_boxes(rng, n)
                crops, _, _, _ = S.ssd_random_crop(rng, boxes, labels, boffs)
                t = S.ssd_resample_tables(rng, hs, ws, offs, crops)
                algo = float((3.0 * t["roi_w"].astype(np.float64) * t["roi_h"]).sum() + n * 3 * 300 * 300 * 4)
                a, dt = torch.from_numpy(arena).to(dev), K.to_device_table(t, dev)
                out = torch.empty((n, 3, 300, 300), dtype=torch.float32, device=dev)
                fns.append(lambda a=a, t=t, dt=dt, out=out: K.resample(a, t, 300, 300, T.FP32, T.NCHW, mul, add, fill_padding=False, out=out, d_samples=dt))
            report("cfg4 crop->resize 300x300->CMN fp32 NCHW (batch 128)", n, _time_launches(fns, args.steps), algo)
        elif op == "box_encoder":
            n, rot = 128, 4
            anchors = torch.from_numpy(S.ssd300_anchors()).to(dev)
            fns, nbox = [], 0
            for r in range(rot):
                rng = S.rng_for(4, 200 + r)
                boxes, labels, boffs = S.random_boxes(rng, n)
                nbox = len(labels)
                b, l, o = torch.from_numpy(boxes).to(dev), torch.from_numpy(labels).to(dev), torch.from_numpy(boffs).to(dev)
                ob = torch.empty((n, 8732, 4), dtype=torch.float32, device=dev)
                ol = torch.empty((n, 8732), dtype=torch.int32, device=dev)
                fns.append(lambda b=b, l=l, o=o, ob=ob, ol=ol: K.box_encode(b, l, o, anchors, 0.5, (0, 0, 0, 0), (0.1, 0.1, 0.2, 0.2), True, 1.0, 50, ob, ol))
            ms = _time_launches(fns, args.steps)
            report("cfg4 box_encoder 8732 anchors (batch 128)", n, ms, n * 8732 * 20 + nbox * 20 + 8732 * 16,
                   {"us_per_batch": ms * 1e3, "boxes_per_batch": nbox})
        elif op == "triangular":
            # configs[1] geometry (Resize shorter->256 + crop 224 + mirror + normalize, fp16 NCHW) with the triangular filter
            n, rot = 256, 2
            fns, algo = [], 0.0
            for r in range(rot):
                rng = S.rng_for(1, 400 + r)
                arena, hs, ws, offs = S.make_images(rng, n, (300, 1080), (300, 1080))
                t = S.classification_tables(rng, hs, ws, offs)
                short = np.minimum(hs, ws).astype(np.float64)
                algo = float((3.0 * (np.ceil(224 / (256 / short)) + 1) ** 2).sum() + n * 3 * 224 * 224 * 2)
                a, dt = torch.from_numpy(arena).to(dev), K.to_device_table(t, dev)
                out = torch.empty((n, 3, 224, 224), dtype=torch.float16, device=dev)
                fns.append(lambda a=a, t=t, dt=dt, out=out: K.resample(a, t, 224, 224, T.FP16, T.NCHW, mul, add, fill_padding=False, out=out,
                                                                       d_samples=dt, interpolation=1))
            report("cfg1 geometry, triangular filter, fp16 NCHW (batch 256, 300..1080 px)", n, _time_launches(fns, args.steps), algo)
        elif op in ("jpeg_e2e", "jpeg_slice_e2e"):
            # configs[1] pipeline fed with JPEG streams (quality 90, 4:2:0) instead of raw pixels: GPU decode (nvJPEG)
            # -> Resize shorter 256 -> CropMirrorNormalize 224 fp16 NCHW, wall clock over whole batches
            import time
            import cv2
            from rocal_b200 import fn, types
            from rocal_b200.pipeline import Pipeline
            n, batches = 256, 6
            rng = S.rng_for(1, 500)
            streams, raw_bytes = [], 0
            for _ in range(n):
                h, w = int(rng.integers(300, 1081)), int(rng.integers(300, 1081))
                yy, xx = np.mgrid[0:h, 0:w].astype(np.float32)
                ch = [127 + 100 * np.sin(xx / rng.uniform(20, 90) + rng.uniform(0, 6)) * np.cos(yy / rng.uniform(20, 90)) for _ in range(3)]
                img = np.clip(np.stack(ch, axis=-1) + rng.normal(0, 6, (h, w, 3)), 0, 255).astype(np.uint8)
                ok, enc = cv2.imencode(".jpg", img, [cv2.IMWRITE_JPEG_QUALITY, 90])
                streams.append(enc.tobytes())
                raw_bytes += h * w * 3
            pipe = Pipeline(batch_size=n, device_id=0, seed=1, prefetch_queue_depth=2)
            with pipe:
                img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_COMPRESSED, max_width=1080, max_height=1080)
                if op == "jpeg_slice_e2e":     # the training variant: random-resized-crop windows, stretched to 224 x 224
                    pipe.set_random_crop_decoder()
                    r = fn.resize(img, resize_width=224, resize_height=224)
                else:
                    r = fn.resize(img, resize_shorter=256)
                out = fn.crop_mirror_normalize(r, crop=[224, 224], mean=list(S.MEAN), std=list(S.STD), mirror=fn.random.coin_flip(),
                                               output_layout=types.NCHW, output_dtype=types.FLOAT16)
                pipe.set_outputs(out)
            pipe.build()
            pipe.feed_encoded(streams)
            for _ in range(2):
                pipe.feed_encoded(streams)
                pipe.run()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for i in range(batches):
                if i < batches - 1:
                    pipe.feed_encoded(streams)
                pipe.run()
                torch.from_dlpack(pipe.get_output_tensors()[0])[0, 0, 0, 0].item()
            torch.cuda.synchronize()
            ms = (time.perf_counter() - t0) * 1e3 / batches
            enc_bytes = sum(len(s) for s in streams)
            tinfo = pipe.timing_info()
            pipe.rocal_release()
            print(json.dumps({"op": ("cfg1 pipeline from JPEG streams (nvJPEG decode -> resize -> CMN fp16), batch 256" if op == "jpeg_e2e" else
                                     "JPEG streams -> random-resized-crop window -> resize 224 -> CMN fp16, batch 256"), "images_per_batch": n,
                              "batch_ms": ms, "images_per_s": n / (ms * 1e-3), "encoded_bytes_per_batch": enc_bytes,
                              "decoded_bytes_per_batch": raw_bytes, "backend": os.environ.get("RB200_NVJPEG_BACKEND", "gpu_hybrid"),
                              "decode_time_us_total": tinfo["decode_time"]}), flush=True)
        elif op == "box_matcher":
            # RetinaNet-sized anchor table (120 087 boxes), batch 32, 1..50 boxes per sample
            n, rot = 32, 4
            base = S.ssd300_anchors()
            reps = -(-120087 // len(base))
            rng = S.rng_for(4, 300)
            big = (np.tile(base, (reps, 1)) + rng.uniform(-0.02, 0.02, (reps * len(base), 4)).astype(np.float32))[:120087]
            anchors = torch.from_numpy(np.ascontiguousarray(big)).to(dev)
            fns, nbox = [], 0
            for r in range(rot):
                rng = S.rng_for(4, 300 + r)
                boxes, labels, boffs = S.random_boxes(rng, n)
                nbox = len(labels)
                b, o = torch.from_numpy(boxes).to(dev), torch.from_numpy(boffs).to(dev)
                om = torch.empty((n, 120087), dtype=torch.int32, device=dev)
                fns.append(lambda b=b, o=o, om=om: K.box_iou_match(b, o, anchors, 0.5, 0.4, True, 50, om))
            ms = _time_launches(fns, args.steps)
            report("box_iou_matcher 120087 anchors, low-quality matches on (batch 32)", n, ms, n * 120087 * 4 + nbox * 16 + 120087 * 16,
                   {"us_per_batch": ms * 1e3, "boxes_per_batch": nbox})
        else:
            print(json.dumps({"op": op, "error": "unknown operator"}))



def bind_to_gpu_numa(index):
    """Restricts this process to the CPUs that are local to GPU `index` (the NUMA node its PCI function reports in
    sysfs), so that the pinned arena it allocates next is placed in that node's memory and its feeding threads
    run beside it. Returns a short description; does nothing where sysfs gives no answer."""
    try:
        import torch
        props = torch.cuda.get_device_properties(index)
        bdf = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        base = "/sys/bus/pci/devices/" + bdf
        with open(base + "/numa_node") as f:
            node = int(f.read().strip())
        with open(base + "/local_cpulist") as f:
            cpulist = f.read().strip()
        cpus = set()
        for part in cpulist.split(","):
            if "-" in part:
                lo, hi = part.split("-")
                cpus.update(range(int(lo), int(hi) + 1))
            elif part:
                cpus.add(int(part))
        allowed = cpus & os.sched_getaffinity(0)
        if node >= 0 and allowed:
            os.sched_setaffinity(0, allowed)
        return {"pci": bdf, "numa_node": node, "cpus": len(allowed)}
    except (OSError, ValueError, AttributeError) as e:
        return {"numa_node": None, "note": "not bound: %s" % type(e).__name__}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=None, help="override the per-GPU batch (profiling only)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true", help="skip the short runs of configs 0, 2, 3, 4")
    ap.add_argument("--no-numa-bind", action="store_true", help="leave the process's CPU affinity as found")
    ap.add_argument("--config", type=int, default=1, choices=[0, 1, 2, 3, 4],
                    help="BASELINE configuration; 1 (default) is the headline workload, the others run on one GPU only")
    ap.add_argument("--op", default=None, help="operator-level cases, comma separated (see run_ops)")
    ap.add_argument("--no-overlap", action="store_true", help="--op cases: plain stream order between the launches")
    ap.add_argument("--strip-rows", type=int, default=0, help="--op cfg0: output rows per CTA of the row-streaming kernel (0 = the library's choice)")
    ap.add_argument("--fast", action="store_true", help="colour operators with RB200_ARITH_FAST (--config 2 and the colour --op cases)")
    args = ap.parse_args()
    if args.op:
        run_ops(args)
        return
    if args.config != 1:
        if int(os.environ.get("WORLD_SIZE", "1")) > 1 or args.impl != "ours":
            raise SystemExit("--config %d runs our arm on one GPU only" % args.config)
        print(json.dumps(measure_config(args.config, args.steps, args.warmup, max(args.steps, 20), True, fast=args.fast)), flush=True)
        return
    global BATCH
    if args.batch:
        BATCH = args.batch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    import rocal_b200
    from rocal_b200 import kernels as K
    import synthetic as S
    from rocal_b200 import tables as T

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    numa = {"numa_node": None, "note": "binding switched off"} if args.no_numa_bind else bind_to_gpu_numa(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    arena_h, t = make_shard(rank, world)
    n = len(t)
    mul, add = S.normalize_tables()
    arena_pinned = torch.from_numpy(arena_h).pin_memory()
    arena_d = arena_pinned.to(dev)
    table_d = K.to_device_table(t, dev)
    out = torch.empty((n, 3, OUT, OUT), dtype=torch.float16, device=dev)
    stream = torch.cuda.current_stream()

    def step_resident():
        K.resample(arena_d, t, OUT, OUT, T.FP16, T.NCHW, mul, add, fill_padding=False, out=out, d_samples=table_d,
                   stream=stream)      # the same output buffer every step: plain stream order, no overlap

    # ---- device-resident throughput + per-launch kernel time (kernel-level C-ABI, CUDA events) ----
    sampler = ClockSampler(local_rank)
    sampler.start()
    t_warm = time.perf_counter()
    warm = 0
    while warm < max(args.warmup, 3) or time.perf_counter() - t_warm < 0.6:   # >= 3 steps and long enough for clock samples
        step_resident()
        warm += 1
        if warm % 64 == 0:
            torch.cuda.synchronize()
    barrier()
    launches0 = rocal_b200.launch_count()
    ev = [torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)]
    ev[0].record(stream)      # one event on each side of the K back-to-back launches
    for i in range(args.steps):
        step_resident()
    ev[1].record(stream)
    barrier()
    launches = rocal_b200.launch_count() - launches0
    total_ms = ev[0].elapsed_time(ev[1])
    launch_ms = [total_ms / args.steps]     # the K launches run back to back between the two events

    # ---- end to end through the public pipeline API: pinned host arena -> rocalRun -> D2H of one image ----
    from rocal_b200 import fn, types
    from rocal_b200.pipeline import Pipeline
    pipe = Pipeline(batch_size=n, device_id=local_rank, seed=1234, prefetch_queue_depth=2)
    with pipe:
        img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_UNCOMPRESSED, max_width=W_RANGE[1], max_height=H_RANGE[1])
        r = fn.resize(img, resize_shorter=RESIZE_SHORTER)
        cmn = fn.crop_mirror_normalize(r, crop=[OUT, OUT], mean=list(S.MEAN), std=list(S.STD), mirror=fn.random.coin_flip(),
                                       output_layout=types.NCHW, output_dtype=types.FLOAT16)
        pipe.set_outputs(cmn)
    pipe.build()
    upload_mode = int(os.environ.get("RB200_BENCH_UPLOAD", Pipeline.UPLOAD_ZERO_COPY))
    pipe.set_upload_mode(upload_mode)
    hs, ws, offs = t["roi_h"].copy(), t["roi_w"].copy(), t["src_offset"].copy()
    rng = np.random.Generator(np.random.PCG64(99 + rank))
    host_back = torch.empty((3, OUT, OUT), dtype=torch.float16).pin_memory()

    def feed():
        pipe.set_crop_anchors(cmn, rng.random(n).astype(np.float32), rng.random(n).astype(np.float32))
        pipe.feed_ragged(arena_pinned, hs, ws, offs)

    def consume():
        pipe.run()
        o = torch.from_dlpack(pipe.get_output_tensors()[0])
        host_back.copy_(o[0], non_blocking=False)

    e2e_steps = max(args.steps, 20)
    for _ in range(3):          # warm-up; the queue is empty again afterwards
        feed()
        consume()
    barrier()
    h2d_before = pipe.h2d_bytes()
    te = time.perf_counter()
    feed()                      # the clock is already running: every batch's feed, upload and kernel are inside the window
    for i in range(e2e_steps):
        if i < e2e_steps - 1:
            feed()              # one batch queued ahead (prefetch depth 2)
        consume()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - te) * 1e3
    h2d_per_step = (pipe.h2d_bytes() - h2d_before) / e2e_steps
    barrier()
    pipe.rocal_release()

    # ---- what the host link gives this rank while every rank pulls at once: plain copies of the pinned arena ----
    link_reps = 6
    barrier()
    tl = time.perf_counter()
    for _ in range(link_reps):
        arena_d.copy_(arena_pinned, non_blocking=True)
    torch.cuda.synchronize()
    link_gbs = link_reps * arena_pinned.numel() / (time.perf_counter() - tl) / 1e9
    barrier()
    # ---- and what the host's memory gives its cores at the same moment: every rank streams its pinned arena ----
    read_threads = max(1, (os.cpu_count() or 1) // max(world, 1) // 2)
    torch.set_num_threads(read_threads)
    words = arena_pinned[:arena_pinned.numel() // 8 * 8].view(torch.int64)
    words.sum()
    barrier()
    tl = time.perf_counter()
    for _ in range(3):
        words.sum()
    host_read_gbs = 3 * words.numel() * 8 / (time.perf_counter() - tl) / 1e9
    barrier()

    mine = torch.tensor([total_ms, e2e_ms, float(h2d_per_step), float(np.mean(launch_ms)), link_gbs, host_read_gbs, float(read_threads)],
                        dtype=torch.float64, device=dev)
    if world > 1:
        gathered = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        numas = [None] * world
        dist.all_gather_object(numas, numa)
    else:
        gathered, numas = [mine], [numa]
    per_rank = []
    for r_, g in enumerate(gathered):
        g = [float(v) for v in g.cpu()]
        per_rank.append({"rank": r_, "device_ms_per_step": g[0] / args.steps, "kernel_ms": g[3], "e2e_ms_per_step": g[1] / e2e_steps,
                         "h2d_bytes_per_step": int(g[2]), "host_link_gbs": g[2] * e2e_steps / (g[1] * 1e-3) / 1e9,
                         "link_copy_gbs": g[4], "host_read_gbs": g[5], "host_read_threads": int(g[6]), "numa": numas[r_]})
    total_ms = max(p_["device_ms_per_step"] for p_ in per_rank) * args.steps
    e2e_ms = max(p_["e2e_ms_per_step"] for p_ in per_rank) * e2e_steps

    if rank == 0:
        peak, peak_src = peak_hbm()
        algo = algorithmic_bytes(t)
        mean_launch_ms = float(np.mean(launch_ms))
        achieved = algo / (mean_launch_ms * 1e-3) / 1e9
        line = {
            "metric": "augmented images/sec", "value": n * world * args.steps / (total_ms * 1e-3), "unit": "images/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": workload_config(world),
            "e2e": {"value": n * world * e2e_steps / (e2e_ms * 1e-3), "unit": "images/s",
                    "h2d_bytes_per_step": int(sum(p_["h2d_bytes_per_step"] for p_ in per_rank)),
                    "h2d_whole_images_bytes": int(arena_pinned.numel()) * world,
                    "h2d": {0: "whole images, one copy", 1: "one strided copy per image of the rectangle the crop can read",
                            2: "zero-copy: the kernel's bulk copies read the rows its taps touch from the pinned arena, each "
                               "row once; bytes = rows x 16-byte-rounded spans, computed from the batch's table"}[upload_mode],
                    "d2h_bytes_per_step": int(host_back.numel() * 2) * world,
                    "d2h_note": "one sample per rank and step: outputs are consumed on the device (DLPack), by design",
                    "steps": e2e_steps, "timed": "clock starts before the first feed; every batch's feed, transfer and kernel inside",
                    "host_link_gbs": sum(p_["host_link_gbs"] for p_ in per_rank),
                    "link_copy_gbs": sum(p_["link_copy_gbs"] for p_ in per_rank),
                    "host_read_gbs": sum(p_["host_read_gbs"] for p_ in per_rank),
                    "link_note": "host_link_gbs = bytes the zero-copy kernels pulled per second, all ranks; link_copy_gbs = "
                                 "plain pinned-to-device copies of the same arenas issued by all ranks at once (what the host "
                                 "and its PCIe links deliver to this many GPUs together); host_read_gbs = the same arenas summed "
                                 "by host threads of every rank at once (what the host's memory gives its own cores)"},
            "gpu_launches": int(launches),
            "per_rank": per_rank,
            "roofline": {"bound": "hbm", "kernel": "resample_stream_pairs_kernel<half,NCHW,normalize>", "achieved": achieved,
                         "peak": peak, "peak_source": peak_src, "unit": "GB/s", "frac": achieved / peak,
                         "algorithmic_bytes_per_launch": algo, "launch_ms": mean_launch_ms,
                         "traffic": NCU_TRAFFIC_BYTES_PER_IMAGE * n, "traffic_source": "ncu, 512-image launch scaled by images"},
        }
        if world == 1 and not args.no_other_configs:
            line["other_configs"] = other_configs(sampler)
        line["clocks"] = dict(sampler.stop(), window="warm-up + timed steps + end-to-end steps" +
                              (" + other configurations" if "other_configs" in line else ""))
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(arena_h, t)
        elif world > 1:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    else:
        sampler.stop()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

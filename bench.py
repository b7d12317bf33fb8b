"""Benchmark of the augmentation hot path: fused Resize(shorter->256, bilinear) + CropMirrorNormalize
(224x224, fp16 NCHW) over batches of 1024 variable-size uint8 images per GPU (BASELINE configs[1]).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 0|2|3|4]

One step = one pass of the path over one batch. Rank 0 prints one JSON line:
  value     images/s with the batch already resident in HBM (CUDA events, max over ranks)
  e2e       images/s through the public pipeline API (external source -> rocalResize -> rocalCropMirrorNormalize
            -> rocalRun) fed from pinned HOST memory: H2D of the batch and its tables, the kernel, and a D2H
            read-back of one output image, all inside the timed region (wall clock between device syncs)
  roofline  algorithmic bytes of the resample kernel / its mean launch time, against the measured
            HBM copy bandwidth (MEASURED_PEAKS.json, else the 6650 GB/s fallback)
  cpu_baseline  the CPU oracle (OpenMP over samples) on a bounded slice of the same batch
`--impl reference` times the CPU implementation alone (the oracle port: the reference's own pixel
code lives in the RPP library, which is not available) and prints the same line shape.
`--config 0|2|3|4` prints the same line for one of the other benchmark configurations (one GPU, our arm only).
Under torchrun every rank owns one GPU and one shard of the synthetic dataset
(shard i of S = indices [floor(N*i/S), floor(N*(i+1)/S)), rocAL's reader partitioning); no
data-path collective is used.
"""
import argparse
import json
import math
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
# dram__bytes_read.sum + dram__bytes_write.sum of one resample launch: measured by ncu on a 512-image
# launch (337.8 MB read + 126.9 MB written) and scaled by the images processed to the 1024-image launch
# (profiles/resample_stream_fp16_nchw_cfg1.md). Scaled again when --batch overrides the batch size.
NCU_TRAFFIC_BYTES_PER_IMAGE = (337829376 + 126903808) / 512.0


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
    from rocal_b200 import synthetic as S
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


def cpu_baseline(arena, t, seconds_target=12.0):
    """Oracle (CPU restatement, OpenMP over samples) on a bounded slice of this batch."""
    from oracle import pyoracle as O
    from rocal_b200 import synthetic as S
    from rocal_b200 import tables as T
    cores = os.cpu_count() or 1
    O.set_threads(cores)
    mul, add = S.normalize_tables()
    n = min(len(t), max(cores * 2, 32))
    sl = np.ascontiguousarray(t[:n])
    O.resample(arena, sl, OUT, OUT, T.FP16, T.NCHW, mul, add)   # warm-up
    reps, elapsed = 0, 0.0
    t0 = time.perf_counter()
    while elapsed < seconds_target and reps < 50:
        O.resample(arena, sl, OUT, OUT, T.FP16, T.NCHW, mul, add)
        reps += 1
        elapsed = time.perf_counter() - t0
    return {"value": n * reps / elapsed, "unit": "images/s", "cores": cores, "kind": "port",
            "sample": "%d images of the batch x %d passes, OpenMP over samples" % (n, reps)}, n * reps / elapsed


def run_reference(args, rank, world):
    """CPU arm: the oracle port with all host threads, each step a bounded slice of the batch."""
    if rank != 0:
        return
    from oracle import pyoracle as O
    from rocal_b200 import synthetic as S
    from rocal_b200 import tables as T
    cores = os.cpu_count() or 1
    O.set_threads(cores)
    n = 128
    lo = 0
    rng = np.random.Generator(np.random.PCG64([1235, lo]))
    arena, hs, ws, offs = S.make_images(rng, n, H_RANGE, W_RANGE)
    t = S.classification_tables(rng, hs, ws, offs, RESIZE_SHORTER, OUT)
    mul, add = S.normalize_tables()
    for _ in range(max(1, min(args.warmup, 3))):
        O.resample(arena, t, OUT, OUT, T.FP16, T.NCHW, mul, add)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.resample(arena, t, OUT, OUT, T.FP16, T.NCHW, mul, add)
    dt = time.perf_counter() - t0
    value = n * args.steps / dt
    line = {"impl": "reference", "metric": "augmented images/sec", "value": value, "unit": "images/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(world, sample=n),
            "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": "port",
                             "sample": "%d images per step (a slice of the 1024-image batch), OpenMP over samples; "
                                       "the reference's own pixel code (RPP) is not available" % n},
            "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def workload_config(world, sample=None):
    c = {"workload": "configs[1]: Resize(shorter=256, bilinear)+CropMirrorNormalize 224x224 fp16 NCHW, "
                     "batch 1024/GPU of uint8 RGB images with H,W~U[300,1080]",
         "batch_per_gpu": BATCH, "sharding": "shard_id/num_shards over %d GPU(s), no collective" % world,
         "l2": "inputs (~1.4 GB/batch) larger than L2"}
    if sample is not None:
        c["images_per_step"] = sample
    return c


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


def run_config(args, cfg):
    import torch
    import rocal_b200
    from oracle import pyoracle as O
    from rocal_b200 import fn, types
    from rocal_b200 import kernels as K
    from rocal_b200 import synthetic as S
    from rocal_b200 import tables as T
    from rocal_b200.pipeline import Pipeline
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream()
    mul, add = S.normalize_tables()
    cores = os.cpu_count() or 1
    O.set_threads(cores)
    peak, peak_src = FALLBACK_HBM_GBS, "fallback"
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak, peak_src = float(json.load(f)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        pass

    # Every configuration rotates over enough distinct batches that one pass exceeds L2 (126 MB).
    resident, feeders, extra = [], [], {}
    if cfg == 0:
        n, rot, name = 64, 6, "configs[0]: Resize(shorter=256)+CropMirrorNormalize 224x224 fp32 NCHW, batch 64, H,W~U[256,512]"
        kernel = "resample_stream_kernel<float,NCHW,normalize>"
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
            resident.append(lambda a=a, t=t, dt=dt, o=o: K.resample(a, t, 224, 224, T.FP32, T.NCHW, mul, add, fill_padding=False, out=o,
                                                                      d_samples=dt, stream=stream))
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
        pipe = Pipeline(batch_size=n, device_id=0, seed=1234, prefetch_queue_depth=2)
        with pipe:
            img, _ = fn.external_source(None, mode=types.EXTSOURCE_RAW_UNCOMPRESSED, max_width=224, max_height=224)
            ct = fn.color_twist(img, brightness=fn.random.uniform(range=(0.6, 1.4)), contrast=fn.random.uniform(range=(0.6, 1.4)),
                                hue=fn.random.uniform(range=(-30.0, 30.0)), saturation=fn.random.uniform(range=(0.5, 1.5)))
            outn = fn.flip(ct, horizontal=fn.random.coin_flip(), vertical=0)
            pipe.set_outputs(outn)
        pipe.build()
        algo = float(n * 2 * 3 * 224 * 224)
        for k in range(rot):
            rng = S.rng_for(2, 100 + k)
            arena, hs, ws, offs = S.make_images(rng, n, (224, 224), (224, 224), content="noise")
            t = S.color_twist_tables(rng, hs, ws, offs)
            a, dt = torch.from_numpy(arena).to(dev), K.to_device_table(t, dev)
            o = torch.empty((n, 224, 224, 3), dtype=torch.uint8, device=dev)
            resident.append(lambda a=a, t=t, dt=dt, o=o: K.pointwise(a, t, 224, 224, T.COLOR_TWIST, out=o, d_samples=dt, fill_padding=False,
                                                                       stream=stream))
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
            resident.append(lambda a=a, t=t, dt=dt, o=o: K.warp_affine(a, t, 640, 480, out=o, d_samples=dt, stream=stream))
            ap_ = torch.from_numpy(arena).pin_memory()
            feeders.append(lambda ap_=ap_, hs=hs, ws=ws, offs=offs, m=t["m"].copy(): (pipe.set_affine(outn, m), pipe.feed_ragged(ap_, hs, ws, offs)))
            if k == 0:
                sl = np.ascontiguousarray(t[:16])
                cpu_fn, cpu_n = (lambda arena=arena, sl=sl: O.warp_affine(arena, sl, 640, 480)), 16
    else:
        n, rot, name = 128, 2, ("configs[4]: SSDRandomCrop -> Resize 300x300 -> CropMirrorNormalize fp32 NCHW + BoxEncoder "
                                "(8732 anchors, criteria 0.5, offset), batch 128, H,W~U[300,800], 1-50 boxes")
        kernel = "resample_stream_kernel<float,NCHW,normalize> (+ box_encode_kernel<4>)"
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
                # the pipeline, and the timed stream waits for it
                meta_stream.wait_stream(stream)
                K.resample(a, t, 300, 300, T.FP32, T.NCHW, mul, add, fill_padding=False, out=o, d_samples=dt, stream=stream)
                K.box_encode(bd, ld, od, anchors_d, 0.5, (0, 0, 0, 0), (0.1, 0.1, 0.2, 0.2), True, 1.0, 50, eb, el, stream=meta_stream)
                stream.wait_stream(meta_stream)
            resident.append(both)
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
    sampler = ClockSampler(0)
    sampler.start()
    t_warm, warm = time.perf_counter(), 0
    while warm < max(args.warmup, 3) or time.perf_counter() - t_warm < 0.6:
        resident[warm % rotn]()
        warm += 1
        if warm % 64 == 0:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    steps = args.steps
    launches0 = rocal_b200.launch_count()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    ev[0].record(stream)
    for i in range(steps):
        resident[i % rotn]()
        ev[i + 1].record(stream)
    torch.cuda.synchronize()
    launches = rocal_b200.launch_count() - launches0
    total_ms = ev[0].elapsed_time(ev[-1])
    mean_launch_ms = total_ms / steps

    # end to end: pinned host arena -> pipeline -> D2H of one output sample
    outs0 = None
    e2e_steps = min(steps, 10)
    feeders[0]()
    for k in range(2):
        feeders[(k + 1) % rotn]()
        pipe.run()
    torch.cuda.synchronize()
    h2d0 = pipe.h2d_bytes()
    te = time.perf_counter()
    for i in range(e2e_steps):
        if i < e2e_steps - 1:
            feeders[(i + 3) % rotn]()
        pipe.run()
        outs0 = torch.from_dlpack(pipe.get_output_tensors()[0])[0].cpu()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - te) * 1e3
    h2d_per_step = (pipe.h2d_bytes() - h2d0) / max(e2e_steps - 1, 1)
    clocks = sampler.stop()
    pipe.rocal_release()

    cpu_value, cpu_reps = _time_cpu(cpu_fn, cpu_n)
    achieved = algo / (mean_launch_ms * 1e-3) / 1e9
    line = {"metric": "augmented images/sec", "value": n * steps / (total_ms * 1e-3), "unit": "images/s", "n_gpus": 1, "steps": steps,
            "warmup": max(args.warmup, 3), "ms_per_step": mean_launch_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": dict({"workload": name, "batch_per_gpu": n,
                            "l2": "rotates over %d batches so that one pass over inputs and outputs exceeds L2" % rotn}, **extra),
            "e2e": {"value": n * e2e_steps / (e2e_ms * 1e-3), "unit": "images/s", "h2d_bytes_per_step": int(h2d_per_step),
                    "d2h_bytes_per_step": int(outs0.numel() * outs0.element_size()), "steps": e2e_steps},
            "gpu_launches": int(launches), "clocks": dict(clocks, window="warm-up + timed steps + end-to-end steps"),
            "roofline": {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                         "frac": achieved / peak, "algorithmic_bytes_per_launch": algo, "launch_ms": mean_launch_ms, "traffic": None},
            "cpu_baseline": {"value": cpu_value, "unit": "images/s", "cores": cores, "kind": "port",
                             "sample": "%d images x %d passes, OpenMP over samples" % (cpu_n, cpu_reps)}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=None, help="override the per-GPU batch (profiling only)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--config", type=int, default=1, choices=[0, 1, 2, 3, 4],
                    help="BASELINE configuration; 1 (default) is the headline workload, the others run on one GPU only")
    args = ap.parse_args()
    if args.config != 1:
        if int(os.environ.get("WORLD_SIZE", "1")) > 1 or args.impl != "ours":
            raise SystemExit("--config %d runs our arm on one GPU only" % args.config)
        run_config(args, args.config)
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
    from rocal_b200 import synthetic as S
    from rocal_b200 import tables as T

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
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
                   stream=stream)

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
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    ev[0].record(stream)
    for i in range(args.steps):
        step_resident()
        ev[i + 1].record(stream)
    barrier()
    launches = rocal_b200.launch_count() - launches0
    total_ms = ev[0].elapsed_time(ev[-1])
    launch_ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]

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

    e2e_steps = min(args.steps, 10)
    feed()
    for _ in range(2):          # warm-up, keeps one batch queued ahead (prefetch depth 2)
        feed()
        consume()
    barrier()
    h2d_before = pipe.h2d_bytes()
    te = time.perf_counter()
    for i in range(e2e_steps):
        if i < e2e_steps - 1:
            feed()
        consume()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - te) * 1e3
    # one batch was queued ahead before the clock started and none is left at the end: the uploads of
    # e2e_steps - 1 batches lie entirely inside the window, the first one partly
    h2d_per_step = (pipe.h2d_bytes() - h2d_before) / max(e2e_steps - 1, 1)
    barrier()
    clocks = sampler.stop()
    pipe.rocal_release()

    times = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms = float(times[0]), float(times[1])

    if rank == 0:
        peak, peak_src = FALLBACK_HBM_GBS, "fallback"
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peak, peak_src = float(json.load(f)["hbm_gbs"]), "measured"
        except (OSError, KeyError, ValueError):
            pass
        algo = algorithmic_bytes(t)
        mean_launch_ms = float(np.mean(launch_ms))
        achieved = algo / (mean_launch_ms * 1e-3) / 1e9
        line = {
            "metric": "augmented images/sec", "value": n * world * args.steps / (total_ms * 1e-3), "unit": "images/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": workload_config(world),
            "e2e": {"value": n * world * e2e_steps / (e2e_ms * 1e-3), "unit": "images/s",
                    "h2d_bytes_per_step": int(h2d_per_step) * world, "h2d_whole_images_bytes": int(arena_pinned.numel()) * world,
                    "h2d_note": "rank 0's bytes x ranks",
                    "h2d": {0: "whole images, one copy", 1: "one strided copy per image of the rectangle the crop can read",
                            2: "zero-copy: the kernel's bulk copies read the tap rows from the pinned arena; bytes = "
                               "footprint rectangles, an upper bound of what crosses the link"}[upload_mode],
                    "d2h_bytes_per_step": int(host_back.numel() * 2) * world, "steps": e2e_steps},
            "gpu_launches": int(launches),
            "clocks": dict(clocks, window="warm-up + timed steps + end-to-end steps"),
            "roofline": {"bound": "hbm", "kernel": "resample_stream_kernel<half,NCHW,normalize>", "achieved": achieved,
                         "peak": peak, "peak_source": peak_src, "unit": "GB/s", "frac": achieved / peak,
                         "algorithmic_bytes_per_launch": algo, "launch_ms": mean_launch_ms,
                         "traffic": NCU_TRAFFIC_BYTES_PER_IMAGE * n, "traffic_source": "ncu, 512-image launch scaled by images"},
        }
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"], _ = cpu_baseline(arena_h, t)
        elif world > 1:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

"""Per-operator device-resident benchmark of the kernel C-ABI on the benchmark configurations.

    python -m rocal_b200.opbench [--ops color_twist,warp,box_encoder,box_matcher,triangular,ssd_chain,cfg0,brightness,flip] [--steps 50]

Prints one JSON line per operator: images/s, mean launch time (CUDA events on the launching stream),
algorithmic bytes per launch and the fraction of the measured HBM copy bandwidth. Every operator rotates
through enough distinct batches that one pass over its inputs and outputs exceeds the 126 MB L2.
"""
import argparse
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FALLBACK_HBM_GBS = 6650.0


def _peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return FALLBACK_HBM_GBS, "fallback"


def _time(fn_list, steps, warmup=5):
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", default="cfg0,color_twist,brightness,flip,warp,ssd_chain,box_encoder")
    ap.add_argument("--steps", type=int, default=50)
    args = ap.parse_args()
    import torch
    from rocal_b200 import kernels as K
    from rocal_b200 import synthetic as S
    from rocal_b200 import tables as T
    dev = torch.device("cuda:0")
    peak, peak_src = _peak()
    mul, add = S.normalize_tables()

    def report(name, n, ms, algo_bytes, extra=None):
        line = {"op": name, "images_per_launch": n, "launch_ms": ms, "images_per_s": n / (ms * 1e-3),
                "algorithmic_bytes_per_launch": algo_bytes, "achieved_gbs": algo_bytes / (ms * 1e-3) / 1e9,
                "peak_gbs": peak, "peak_source": peak_src, "frac": algo_bytes / (ms * 1e-3) / 1e9 / peak}
        if extra:
            line.update(extra)
        print(json.dumps(line), flush=True)

    for op in args.ops.split(","):
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
                fns.append(lambda a=a, t=t, dt=dt, out=out: K.resample(a, t, 224, 224, T.FP32, T.NCHW, mul, add, fill_padding=False, out=out, d_samples=dt))
            report("cfg0 resize+CMN fp32 NCHW (batch 64, 256..512 px)", n, _time(fns, args.steps), algo)
        elif op in ("color_twist", "brightness", "contrast", "flip"):
            n, rot = int(os.environ.get("RB200_OPBENCH_N", "256")), 4
            code = {"color_twist": T.COLOR_TWIST, "brightness": T.COLOR_BRIGHTNESS, "contrast": T.COLOR_CONTRAST, "flip": T.COLOR_NONE}[op]
            fns = []
            for r in range(rot):
                rng = S.rng_for(2, 100 + r)
                arena, hs, ws, offs = S.make_images(rng, n, (224, 224), (224, 224), content="noise")
                t = S.color_twist_tables(rng, hs, ws, offs)
                a, dt = torch.from_numpy(arena).to(dev), K.to_device_table(t, dev)
                out = torch.empty((n, 224, 224, 3), dtype=torch.uint8, device=dev)
                fns.append(lambda a=a, t=t, dt=dt, out=out: K.pointwise(a, t, 224, 224, code, out=out, d_samples=dt, fill_padding=False))
            report("cfg2 %s(+flip) u8 HWC 224x224 (batch %d)" % (op, n), n, _time(fns, args.steps), n * 2 * 3 * 224 * 224)
        elif op == "warp":
            n, rot = 128, 2
            fns = []
            for r in range(rot):
                rng = S.rng_for(3, 100 + r)
                arena, hs, ws, offs = S.make_images(rng, n, (480, 480), (640, 640))
                t = S.warp_tables(rng, hs, ws, offs, 640, 480)
                a, dt = torch.from_numpy(arena).to(dev), K.to_device_table(t, dev)
                out = torch.empty((n, 480, 640, 3), dtype=torch.uint8, device=dev)
                fns.append(lambda a=a, t=t, dt=dt, out=out: K.warp_affine(a, t, 640, 480, out=out, d_samples=dt))
            report("cfg3 warp_affine u8 480x640 (batch 128)", n, _time(fns, args.steps), n * 2 * 3 * 480 * 640)
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
            report("cfg4 crop->resize 300x300->CMN fp32 NCHW (batch 128)", n, _time(fns, args.steps), algo)
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
            ms = _time(fns, args.steps)
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
            report("cfg1 geometry, triangular filter, fp16 NCHW (batch 256, 300..1080 px)", n, _time(fns, args.steps), algo)
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
            ms = _time(fns, args.steps)
            report("box_iou_matcher 120087 anchors, low-quality matches on (batch 32)", n, ms, n * 120087 * 4 + nbox * 16 + 120087 * 16,
                   {"us_per_batch": ms * 1e3, "boxes_per_batch": nbox})
        else:
            print(json.dumps({"op": op, "error": "unknown operator"}))


if __name__ == "__main__":
    sys.path.insert(0, ROOT)
    main()

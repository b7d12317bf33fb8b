"""Thin Python front of the kernel-level C-ABI (include/rb200_kernels.h).

torch is used only to own device memory and streams; every computation is a call into
librocal_b200.so. Inputs: a uint8 CUDA tensor holding the packed source images (the arena) and
a numpy structured array with one row per sample (dtypes in rocal_b200.tables).
"""
import ctypes

import numpy as np
import torch

from . import tables as T
from ._lib import (BoxEncoderParams, BoxMatcherParams, NormalizeParams, PointwiseParams, ResampleParams, WarpParams, check, lib)

_TORCH_DTYPE = {T.FP32: torch.float32, T.FP16: torch.float16, T.UINT8: torch.uint8}


def _stream_ptr(stream):
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


def to_device_table(samples, device):
    """Uploads a structured numpy table as raw bytes."""
    raw = torch.from_numpy(np.ascontiguousarray(samples).view(np.uint8).reshape(-1))
    return raw.to(device, non_blocking=False)


def _alloc_out(n, out_w, out_h, dtype, layout, device, out):
    shape = (n, 3, out_h, out_w) if layout == T.NCHW else (n, out_h, out_w, 3)
    if out is None:
        out = torch.empty(shape, dtype=_TORCH_DTYPE[dtype], device=device)
    else:
        assert tuple(out.shape) == shape and out.dtype == _TORCH_DTYPE[dtype] and out.is_contiguous()
    return out


def _sizes(p, arena, out, arena_bytes, out_bytes):
    """The sizes a launch states to the library: the tensors' own unless the caller overrides them."""
    p.arena_bytes = int(arena.numel() * arena.element_size() if arena_bytes is None else arena_bytes)
    p.out_bytes = int(out.numel() * out.element_size() if out_bytes is None else out_bytes)


def resample(arena, samples, out_w, out_h, out_dtype=T.FP32, out_layout=T.NCHW, mul=None, add=None,
             fill_padding=True, out=None, d_samples=None, stream=None, staged=True, interpolation=0, path=0,
             status=None, probe=None, overlap=False, arena_bytes=None, out_bytes=None, strip_rows=0):
    """rb200k_resample. strip_rows: rows per CTA of the row-streaming kernel (0 = the library chooses). arena_bytes / out_bytes: the sizes stated to the library (None: those of the tensors). overlap=True states that the launch is independent of the kernel enqueued just before it. `samples`: numpy RESAMPLE_SAMPLE table (host); `d_samples`: the same table
    already on the device (uploaded here when None). staged=False withholds the host table from
    the launch so that the kernel gathers straight from global memory; path=1 (RB200_RESAMPLE_PATH_TILE)
    forces the shared-memory tile kernel. status: an int32 CUDA tensor that receives 1 when a bounded wait gives up
    (None: the library-wide word); probe=(wait_cycles, skip_row) launches through rb200k_resample_probe."""
    n = len(samples)
    out = _alloc_out(n, out_w, out_h, out_dtype, out_layout, arena.device, out)
    if d_samples is None:
        d_samples = to_device_table(samples, arena.device)
    p = ResampleParams()
    p.out = out.data_ptr()
    p.out_w, p.out_h, p.out_dtype, p.out_layout = out_w, out_h, out_dtype, out_layout
    p.normalize = 1 if mul is not None else 0
    p.fill_padding = 1 if fill_padding else 0
    p.interpolation = int(interpolation)
    p.path = int(path)
    p.strip_rows = int(strip_rows)
    for c in range(3):
        p.mul[c] = float(mul[c]) if mul is not None else 1.0
        p.add[c] = float(add[c]) if add is not None else 0.0
    p.status = status.data_ptr() if status is not None else None
    p.overlap = 1 if overlap else 0
    _sizes(p, arena, out, arena_bytes, out_bytes)
    h_ptr = samples.ctypes.data_as(ctypes.c_void_p) if staged else None
    if probe is not None:
        check(lib.rb200k_resample_probe(arena.data_ptr(), d_samples.data_ptr(), h_ptr, n, ctypes.byref(p),
                                        _stream_ptr(stream), int(probe[0]), int(probe[1])), "rb200k_resample_probe")
    else:
        check(lib.rb200k_resample(arena.data_ptr(), d_samples.data_ptr(), h_ptr, n, ctypes.byref(p),
                                  _stream_ptr(stream)), "rb200k_resample")
    return out


def pointwise(arena, samples, out_w, out_h, color_op=T.COLOR_NONE, out_dtype=T.UINT8, out_layout=T.NHWC,
              mul=None, add=None, reverse_channels=False, fill_padding=True, out=None, d_samples=None,
              stream=None, arith=0, status=None, probe=None, overlap=False, arena_bytes=None, out_bytes=None):
    """rb200k_pointwise. arena_bytes / out_bytes as for resample. arith: 0 exact, 1 fast colour arithmetic; status / probe as for resample."""
    n = len(samples)
    out = _alloc_out(n, out_w, out_h, out_dtype, out_layout, arena.device, out)
    if d_samples is None:
        d_samples = to_device_table(samples, arena.device)
    p = PointwiseParams()
    p.out = out.data_ptr()
    p.out_w, p.out_h, p.out_dtype, p.out_layout = out_w, out_h, out_dtype, out_layout
    p.color_op = color_op
    p.normalize = 1 if mul is not None else 0
    p.fill_padding = 1 if fill_padding else 0
    p.reverse_channels = 1 if reverse_channels else 0
    for c in range(3):
        p.mul[c] = float(mul[c]) if mul is not None else 1.0
        p.add[c] = float(add[c]) if add is not None else 0.0
    p.arith = int(arith)
    p.overlap = 1 if overlap else 0
    p.status = status.data_ptr() if status is not None else None
    _sizes(p, arena, out, arena_bytes, out_bytes)
    if probe is not None:
        check(lib.rb200k_pointwise_probe(arena.data_ptr(), d_samples.data_ptr(), samples.ctypes.data_as(ctypes.c_void_p), n,
                                         ctypes.byref(p), _stream_ptr(stream), int(probe[0]), int(probe[1])),
              "rb200k_pointwise_probe")
    else:
        check(lib.rb200k_pointwise(arena.data_ptr(), d_samples.data_ptr(), samples.ctypes.data_as(ctypes.c_void_p), n,
                                   ctypes.byref(p), _stream_ptr(stream)), "rb200k_pointwise")
    return out


def warp_affine(arena, samples, out_w, out_h, fill_padding=True, out=None, d_samples=None, stream=None, overlap=False,
                status=None, arena_bytes=None, out_bytes=None):
    """rb200k_warp_affine: uint8 NHWC output. status / arena_bytes / out_bytes as for resample."""
    n = len(samples)
    out = _alloc_out(n, out_w, out_h, T.UINT8, T.NHWC, arena.device, out)
    if d_samples is None:
        d_samples = to_device_table(samples, arena.device)
    p = WarpParams()
    p.out = out.data_ptr()
    p.out_w, p.out_h = out_w, out_h
    p.fill_padding = 1 if fill_padding else 0
    p.overlap = 1 if overlap else 0
    p.status = status.data_ptr() if status is not None else None
    _sizes(p, arena, out, arena_bytes, out_bytes)
    check(lib.rb200k_warp_affine(arena.data_ptr(), d_samples.data_ptr(), n, ctypes.byref(p), _stream_ptr(stream)),
          "rb200k_warp_affine")
    return out


def box_encode(boxes, labels, box_offsets, anchors, criteria, means, stds, offset, scale, max_boxes,
               out_boxes=None, out_labels=None, stream=None):
    """rb200k_box_encode. boxes [total,4] f32, labels [total] i32, box_offsets [n+1] i32, anchors
    [A,4] f32 — all CUDA tensors."""
    n = box_offsets.numel() - 1
    a = anchors.shape[0]
    if out_boxes is None:
        out_boxes = torch.empty((n, a, 4), dtype=torch.float32, device=boxes.device)
    if out_labels is None:
        out_labels = torch.empty((n, a), dtype=torch.int32, device=boxes.device)
    p = BoxEncoderParams()
    p.anchors = anchors.data_ptr()
    p.num_anchors = a
    p.criteria = float(criteria)
    for k in range(4):
        p.means[k] = float(means[k])
        p.inv_stds[k] = float(np.float32(1.0 / float(np.float32(stds[k]))))
    p.offset = 1 if offset else 0
    p.scale = float(scale)
    check(lib.rb200k_box_encode(boxes.data_ptr(), labels.data_ptr(), box_offsets.data_ptr(), n, int(max_boxes),
                                ctypes.byref(p), out_boxes.data_ptr(), out_labels.data_ptr(), _stream_ptr(stream)),
          "rb200k_box_encode")
    return out_boxes, out_labels


def box_iou_match(boxes, box_offsets, anchors, high_threshold, low_threshold, allow_low_quality_matches, max_boxes,
                  out=None, stream=None):
    """rb200k_box_iou_match. boxes [total,4] f32, box_offsets [n+1] i32, anchors [A,4] f32 - CUDA tensors.
    Returns int32 [n, A]: matched box index per anchor, -1 / -2 below the low / high threshold."""
    n = box_offsets.numel() - 1
    a = anchors.shape[0]
    if out is None:
        out = torch.empty((n, a), dtype=torch.int32, device=boxes.device)
    p = BoxMatcherParams()
    p.anchors = anchors.data_ptr()
    p.num_anchors = a
    p.high_threshold, p.low_threshold = float(high_threshold), float(low_threshold)
    p.allow_low_quality_matches = 1 if allow_low_quality_matches else 0
    check(lib.rb200k_box_iou_match(boxes.data_ptr(), box_offsets.data_ptr(), n, int(max_boxes), ctypes.byref(p),
                                   out.data_ptr(), _stream_ptr(stream)), "rb200k_box_iou_match")
    return out


def box_transform(boxes, labels, box_offsets, windows, rule, stream=None):
    """rb200k_box_transform. boxes [total,4] f32, labels [total] i32, box_offsets [n+1] i32 - CUDA tensors; windows: numpy
    BOX_WINDOW table (uploaded here) or a CUDA uint8 tensor holding one. Returns (out_boxes, out_labels, out_offsets) with
    capacity total + n; out_offsets[n] is the number of valid entries."""
    n = box_offsets.numel() - 1
    total = boxes.shape[0]
    d_win = to_device_table(windows, boxes.device) if isinstance(windows, np.ndarray) else windows
    out_boxes = torch.empty((total + n, 4), dtype=torch.float32, device=boxes.device)
    out_labels = torch.empty((total + n,), dtype=torch.int32, device=boxes.device)
    out_offsets = torch.empty((n + 1,), dtype=torch.int32, device=boxes.device)
    check(lib.rb200k_box_transform(boxes.data_ptr(), labels.data_ptr(), box_offsets.data_ptr(), n, d_win.data_ptr(), int(rule),
                                   out_boxes.data_ptr(), out_labels.data_ptr(), out_offsets.data_ptr(), _stream_ptr(stream)),
          "rb200k_box_transform")
    return out_boxes, out_labels, out_offsets


def normalize_scratch_bytes(n, max_w, max_h, axis_mask):
    return int(lib.rb200k_normalize_scratch_bytes(int(n), int(max_w), int(max_h), int(axis_mask)))


def _normalize_params(out, out_w, out_h, out_dtype, axis_mask, mean, stddev, scale, shift, fill_padding):
    p = NormalizeParams()
    p.out = out.data_ptr()
    p.out_w, p.out_h, p.out_dtype, p.axis_mask = out_w, out_h, out_dtype, int(axis_mask)
    p.compute_mean, p.compute_stddev = int(mean is None), int(stddev is None)
    p.fill_padding = 1 if fill_padding else 0
    for c in range(3):
        p.mean[c] = float(mean[c]) if mean is not None else 0.0
        p.stddev[c] = float(stddev[c]) if stddev is not None else 1.0
    p.scale, p.shift = float(scale), float(shift)
    return p


def normalize(arena, samples, out_w, out_h, axis_mask=3, mean=None, stddev=None, scale=1.0, shift=0.0, out_dtype=T.FP32,
              fill_padding=True, out=None, d_samples=None, scratch=None, stream=None):
    """rb200k_normalize: uint8 HWC windows (POINTWISE_SAMPLE table) -> [n][out_h][out_w][3] float32 / float16.
    mean / stddev None = computed over the axes of axis_mask (bit 0 height, 1 width, 2 channel). `scratch`: a uint8
    CUDA tensor of at least normalize_scratch_bytes(...) bytes (allocated here when None and needed)."""
    n = len(samples)
    out = _alloc_out(n, out_w, out_h, out_dtype, T.NHWC, arena.device, out)
    if d_samples is None:
        d_samples = to_device_table(samples, arena.device)
    p = _normalize_params(out, out_w, out_h, out_dtype, axis_mask, mean, stddev, scale, shift, fill_padding)
    _sizes(p, arena, out, None, None)
    need = normalize_scratch_bytes(n, out_w, out_h, axis_mask) if (mean is None or stddev is None) else 0
    if scratch is None and need:
        scratch = torch.empty(need, dtype=torch.uint8, device=arena.device)
    check(lib.rb200k_normalize(arena.data_ptr(), d_samples.data_ptr(), samples.ctypes.data_as(ctypes.c_void_p), n, ctypes.byref(p),
                               scratch.data_ptr() if scratch is not None else None, scratch.numel() if scratch is not None else 0,
                               _stream_ptr(stream)), "rb200k_normalize")
    return out


def transpose(arena, samples, perm, out_dims, out=None, d_samples=None, stream=None):
    """rb200k_transpose: uint8 [n][out_dims...], every sample's permuted window at the origin of its slot."""
    n = len(samples)
    if out is None:
        out = torch.zeros((n,) + tuple(int(v) for v in out_dims), dtype=torch.uint8, device=arena.device)
    if d_samples is None:
        d_samples = to_device_table(samples, arena.device)
    pm = (ctypes.c_int32 * 3)(*[int(v) for v in perm])
    od = (ctypes.c_int32 * 3)(*[int(v) for v in out_dims])
    check(lib.rb200k_transpose(arena.data_ptr(), d_samples.data_ptr(), n, pm, out.data_ptr(), od, _stream_ptr(stream)),
          "rb200k_transpose")
    return out

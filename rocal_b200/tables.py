"""numpy views of the per-sample tables of include/rb200_kernels.h (same field order and sizes)."""
import numpy as np

FP32, FP16, UINT8 = 0, 1, 2
NHWC, NCHW = 0, 1
COLOR_NONE, COLOR_BRIGHTNESS, COLOR_CONTRAST, COLOR_TWIST, COLOR_GAMMA, COLOR_BLEND = 0, 1, 2, 3, 4, 5

RESAMPLE_SAMPLE = np.dtype([
    ("src_offset", "<u8"), ("src_stride", "<u4"),
    ("roi_x", "<i4"), ("roi_y", "<i4"), ("roi_w", "<i4"), ("roi_h", "<i4"),
    ("dst_w", "<i4"), ("dst_h", "<i4"),
    ("crop_x", "<i4"), ("crop_y", "<i4"), ("crop_w", "<i4"), ("crop_h", "<i4"),
    ("mirror", "<i4"), ("reserved", "<i4", (2,))], align=True)

POINTWISE_SAMPLE = np.dtype([
    ("src_offset", "<u8"), ("src_stride", "<u4"),
    ("roi_x", "<i4"), ("roi_y", "<i4"), ("roi_w", "<i4"), ("roi_h", "<i4"),
    ("flip_h", "<i4"), ("flip_v", "<i4"),
    ("alpha", "<f4"), ("beta", "<f4"), ("hue", "<f4"), ("sat", "<f4"),
    ("src2_offset_lo", "<u4"), ("src2_offset_hi", "<u4"), ("src2_stride", "<u4")], align=True)

WARP_SAMPLE = np.dtype([
    ("src_offset", "<u8"), ("src_stride", "<u4"),
    ("src_w", "<i4"), ("src_h", "<i4"),
    ("m", "<f4", (6,)),
    ("dst_w", "<i4"), ("dst_h", "<i4"),
    ("reserved", "<i4", (3,))], align=True)

BOX_WINDOW = np.dtype([("l", "<f4"), ("t", "<f4"), ("r", "<f4"), ("b", "<f4"), ("mirror_h", "<i4"), ("mirror_v", "<i4"),
                       ("reserved", "<i4", (2,))], align=True)
BOX_RULE_QUARTER_AREA, BOX_RULE_CENTRE = 0, 1

assert RESAMPLE_SAMPLE.itemsize == 64 and POINTWISE_SAMPLE.itemsize == 64 and WARP_SAMPLE.itemsize == 64
assert BOX_WINDOW.itemsize == 32

NP_DTYPE = {FP32: np.float32, FP16: np.float16, UINT8: np.uint8}

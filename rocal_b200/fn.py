"""Graph-building functions with the names and keyword arguments of amd.rocal.fn
(rocAL_pybind/amd/rocal/fn.py) for the supported operators. Each returns the output tensor handle."""
import ctypes

from . import _capi as C
from . import decoders  # noqa: F401  (fn.decoders.image)
from . import random  # noqa: F401  (fn.random.coin_flip)
from . import readers  # noqa: F401  (fn.readers.file)
from . import types
from .pipeline import Pipeline, RocalError


def _pipe():
    p = Pipeline._current_pipeline
    if p is None:
        raise RocalError("fn.* must be called inside `with pipeline:`")
    return p


def _ret(p, handle):
    if not handle:
        raise RocalError(p.error_message())
    return handle


def _fparam(v):
    """float -> fixed parameter; Param -> itself; None -> the operator's default random range."""
    if v is None or isinstance(v, C.Param):
        return v
    return C.Param(C.create_float_parameter(float(v)), False)


def _iparam(v):
    if v is None or isinstance(v, C.Param):
        return v
    return C.Param(C.create_int_parameter(int(v)), True)


def _farr(v):
    return (ctypes.c_float * len(v))(*[float(x) for x in v])


def external_source(source, device=None, color_format=types.RGB, random_shuffle=False, mode=types.EXTSOURCE_FNAME,
                    max_width=2000, max_height=2000, last_batch_policy=types.LAST_BATCH_FILL,
                    pad_last_batch_repeated=False, stick_to_shard=True, shard_size=-1):
    """fn.py:1091. mode=EXTSOURCE_RAW_UNCOMPRESSED takes decoded pixels (Pipeline.feed_input / feed_ragged);
    EXTSOURCE_RAW_COMPRESSED and EXTSOURCE_FNAME take JPEG streams / files (Pipeline.feed_encoded / feed_files),
    decoded on the GPU. Returns (images, labels) like the reference (labels is empty)."""
    p = _pipe()
    p._external_source_mode = mode
    p._max_w, p._max_h = max_width, max_height
    return _ret(p, C.external_source(p._handle, color_format, 0, max_width, max_height, mode)), []


def resize(*inputs, max_size=[], resize_longer=0, resize_shorter=0, resize_width=0, resize_height=0,
           scaling_mode=types.SCALING_MODE_DEFAULT, interpolation_type=types.LINEAR_INTERPOLATION, antialias=True,
           device=None, output_layout=types.NHWC, output_dtype=types.UINT8):
    p = _pipe()
    ms = [max_size] if isinstance(max_size, int) else list(max_size)
    mw = ms[0] if ms else 0
    mh = ms[1] if len(ms) > 1 else mw
    return _ret(p, C.resize(p._handle, inputs[0], resize_width, resize_height, 0, scaling_mode, mw, mh, resize_shorter,
                            resize_longer, interpolation_type, output_layout, output_dtype))


def resize_mirror_normalize(*inputs, max_size=[], resize_longer=0, resize_shorter=0, resize_width=0, resize_height=0,
                            scaling_mode=types.SCALING_MODE_DEFAULT, interpolation_type=types.LINEAR_INTERPOLATION,
                            mean=[0.0], std=[1.0], mirror=1, device=None, output_layout=types.NHWC, output_dtype=types.UINT8):
    p = _pipe()
    ms = [max_size] if isinstance(max_size, int) else list(max_size)
    mw = ms[0] if ms else 0
    mh = ms[1] if len(ms) > 1 else mw
    return _ret(p, C.resize_mirror_normalize(p._handle, inputs[0], resize_width, resize_height, _farr(mean), _farr(std),
                                             min(len(mean), len(std)), 0, scaling_mode, mw, mh, resize_shorter,
                                             resize_longer, interpolation_type, _iparam(mirror), output_layout, output_dtype))


def crop_mirror_normalize(*inputs, crop=[0, 0], crop_pos_x=0.5, crop_pos_y=0.5, crop_w=0, crop_h=0, mean=[0.0], std=[1.0],
                          mirror=1, device=None, output_layout=types.NHWC, output_dtype=types.UINT8, image_type=None):
    p = _pipe()
    if len(crop) == 2 and (crop[0] or crop[1]):
        crop_h, crop_w = crop[0], crop[1]
    elif len(crop) == 3:
        crop_h, crop_w = crop[1], crop[2]
    return _ret(p, C.crop_mirror_normalize(p._handle, inputs[0], crop_h, crop_w, crop_pos_x, crop_pos_y, _farr(mean),
                                           _farr(std), min(len(mean), len(std)), 0, _iparam(mirror), output_layout,
                                           output_dtype))


def crop(*inputs, crop=[0, 0], crop_pos_x=0.5, crop_pos_y=0.5, crop_pos_z=0.5, crop_w=0, crop_h=0, crop_d=1, device=None,
         output_layout=types.NHWC, output_dtype=types.UINT8):
    """Fixed-size crop at an absolute position (rocalCropFixed) when a size is given, else the random crop (rocalCrop)."""
    p = _pipe()
    if len(crop) == 2 and (crop[0] or crop[1]):
        crop_h, crop_w = crop[0], crop[1]
    if crop_w and crop_h:
        return _ret(p, C.crop_fixed(p._handle, inputs[0], crop_w, crop_h, 0, crop_pos_x, crop_pos_y, output_layout, output_dtype))
    return _ret(p, C.crop(p._handle, inputs[0], 0, None, None, None, None, output_layout, output_dtype))


def center_crop(*inputs, crop=[0, 0], crop_h=0, crop_w=0, crop_d=1, device=None, output_layout=types.NHWC,
                output_dtype=types.UINT8):
    p = _pipe()
    if len(crop) == 2 and (crop[0] or crop[1]):
        crop_h, crop_w = crop[0], crop[1]
    return _ret(p, C.crop_center_fixed(p._handle, inputs[0], crop_w, crop_h, 0, output_layout, output_dtype))


def centre_crop(*inputs, **kwargs):
    """fn.py: the British spelling the reference also exports."""
    return center_crop(*inputs, **kwargs)


def random_crop(*inputs, crop_area_factor=None, crop_aspect_ratio=None, crop_pox_x=None, crop_pox_y=None, num_attempts=20,
                device=None, all_boxes_above_threshold=True, allow_no_crop=True, ltrb=True, output_layout=types.NHWC,
                output_dtype=types.UINT8):
    """rocalRandomCrop: a window of random area and aspect ratio (floats, fn.random.uniform parameters, or None for
    the reference's default ranges 0.08..0.99 and 0.75..1.333)."""
    p = _pipe()
    return _ret(p, C.random_crop(p._handle, inputs[0], 0, _fparam(crop_area_factor), _fparam(crop_aspect_ratio),
                                 _fparam(crop_pox_x), _fparam(crop_pox_y), num_attempts, output_layout, output_dtype))


def resize_crop(*inputs, resize_width=0, resize_height=0, crop_area_factor=None, crop_aspect_ratio=None, x_drift=None,
                y_drift=None, device=None, max_size=[], resize_longer=0, resize_shorter=0,
                scaling_mode=types.SCALING_MODE_DEFAULT, interpolation_type=types.LINEAR_INTERPOLATION,
                output_layout=types.NHWC, output_dtype=types.UINT8):
    """rocalCropResize: the random window of random_crop stretched to resize_width x resize_height (one launch)."""
    p = _pipe()
    return _ret(p, C.crop_resize(p._handle, inputs[0], resize_width, resize_height, 0, _fparam(crop_area_factor),
                                 _fparam(crop_aspect_ratio), _fparam(x_drift), _fparam(y_drift), output_layout, output_dtype))


def roi_resize(*inputs, resize_width=0, resize_height=0, roi_w=None, roi_h=None, roi_pos_x=None, roi_pos_y=None, device=None,
               interpolation_type=types.LINEAR_INTERPOLATION, output_layout=types.NHWC, output_dtype=types.UINT8):
    """rocalROIResize: the window roi_w x roi_h at pixel (roi_pos_x, roi_pos_y) stretched to resize_width x resize_height."""
    p = _pipe()
    return _ret(p, C.roi_resize(p._handle, inputs[0], resize_width, resize_height, 0, int(roi_h or 0), int(roi_w or 0),
                                float(roi_pos_x or 0), float(roi_pos_y or 0), interpolation_type, output_layout, output_dtype))


def one_hot(*inputs, num_classes=0, device=None):
    """fn.py:943: asks the classification iterator for one-hot labels with num_classes columns."""
    p = _pipe()
    p._num_classes = num_classes
    p._one_hot_encoding = True
    return []


def uniform(*inputs, range=(-1.0, 1.0), device=None):
    """fn.py:888: per-sample float, uniform in range (the same parameter as fn.random.uniform)."""
    return random.uniform(*inputs, range=range, device=device)


def nop(*inputs, device=None, output_layout=types.NHWC, output_dtype=types.UINT8):
    """rocalNop / rocalCopy: the input unchanged (a copy into the operator's own output tensor)."""
    p = _pipe()
    return _ret(p, C.flip(p._handle, inputs[0], 0, _iparam(0), _iparam(0), output_layout, output_dtype))


copy = nop


def resize_crop_mirror(*inputs, resize_width=0, resize_height=0, crop_w=0, crop_h=0, mirror=1, device=None, max_size=[],
                       resize_longer=0, resize_shorter=0, scaling_mode=types.SCALING_MODE_DEFAULT,
                       interpolation_type=types.LINEAR_INTERPOLATION, output_layout=types.NHWC, output_dtype=types.UINT8):
    p = _pipe()
    return _ret(p, C.resize_crop_mirror_fixed(p._handle, inputs[0], resize_width, resize_height, 0, crop_h, crop_w,
                                              _iparam(mirror), output_layout, output_dtype))


def ssd_random_crop(*inputs, p_threshold=None, crop_area_factor=None, crop_aspect_ratio=None, crop_pos_x=None,
                    crop_pos_y=None, num_attempts=20, device=None, all_boxes_above_threshold=True, allow_no_crop=True, ltrb=True,
                    output_layout=types.NHWC, output_dtype=types.UINT8):
    p = _pipe()
    return _ret(p, C.ssd_random_crop(p._handle, inputs[0], 0, num_attempts, output_layout, output_dtype))


def random_bbox_crop(*inputs, all_boxes_above_threshold=True, allow_no_crop=True, aspect_ratio=None, bbox_layout="",
                     threshold_type="iou", thresholds=None, crop_shape=None, num_attempts=1, scaling=None, seed=1,
                     shape_layout="", input_shape=None, total_num_attempts=0, device=None, ltrb=True, labels=None):
    """rocalRandomBBoxCrop (amd/rocal/fn.py:901-940): the source images of every batch reach the graph cut to a window
    sampled around their boxes. Returns the reference's 4-tuple; its first element is None here (the reference returns
    the metadata reader's handle, which nothing consumes)."""
    p = _pipe()
    p._check(C.random_bbox_crop(p._handle, int(bool(all_boxes_above_threshold)), int(bool(crop_shape)), int(seed) & 0xFFFFFFFF))
    return (None, [], [], [])


def flip(*inputs, horizontal=0, vertical=0, device=None, output_layout=types.NHWC, output_dtype=types.UINT8):
    p = _pipe()
    return _ret(p, C.flip(p._handle, inputs[0], 0, _iparam(horizontal), _iparam(vertical), output_layout, output_dtype))


def brightness(*inputs, brightness=None, brightness_shift=None, device=None, output_layout=types.NHWC, output_dtype=types.UINT8):
    p = _pipe()
    return _ret(p, C.brightness(p._handle, inputs[0], 0, _fparam(brightness), _fparam(brightness_shift), output_layout, output_dtype))


def brightness_fixed(*inputs, brightness=1.0, brightness_shift=0.0, device=None, output_layout=types.NHWC, output_dtype=types.UINT8):
    p = _pipe()
    return _ret(p, C.brightness(p._handle, inputs[0], 0, _fparam(brightness), _fparam(brightness_shift),
                                output_layout, output_dtype))


def contrast(*inputs, contrast=None, contrast_center=None, device=None, output_layout=types.NHWC, output_dtype=types.UINT8):
    p = _pipe()
    return _ret(p, C.contrast(p._handle, inputs[0], 0, _fparam(contrast), _fparam(contrast_center), output_layout, output_dtype))


def blend(*inputs, ratio=None, device=None, output_layout=types.NHWC, output_dtype=types.UINT8):
    """rocalBlend (fn.py:37): inputs[0]*ratio + inputs[1]*(1 - ratio); ratio a float, a random parameter, or None for the
    reference's default range 0.1 .. 0.9."""
    p = _pipe()
    return _ret(p, C.blend(p._handle, inputs[0], inputs[1], 0, _fparam(ratio), output_layout, output_dtype))


def exposure(*inputs, exposure=0.5, device=None, output_layout=types.NHWC, output_dtype=types.UINT8):
    """rocalExposure (fn.py:78): x * 2^exposure; a float, a random parameter, or None for the reference's default range
    0.15 .. 0.95."""
    p = _pipe()
    return _ret(p, C.exposure(p._handle, inputs[0], 0, _fparam(exposure), output_layout, output_dtype))


def gamma_correction(*inputs, gamma=0.5, device=None, output_layout=types.NHWC, output_dtype=types.UINT8):
    """rocalGamma: 255 * (x / 255)^gamma (None: the reference's default range 0.3 .. 7)."""
    p = _pipe()
    return _ret(p, C.gamma(p._handle, inputs[0], 0, _fparam(gamma), output_layout, output_dtype))


def color_temp(*inputs, adjustment_value=50, device=None, output_layout=types.NHWC, output_dtype=types.UINT8):
    """rocalColorTemp: R + adjustment, B - adjustment (an integer; None: the reference's default range -99 .. 99)."""
    p = _pipe()
    return _ret(p, C.color_temp(p._handle, inputs[0], 0, _iparam(adjustment_value), output_layout, output_dtype))


def normalize(*inputs, axes=[], mean=[], stddev=[], scale=1.0, shift=0.0, output_datatype=types.FLOAT):
    """fn.py:1216: out = scale * (in - mean) / stddev + shift. axes (0 height, 1 width, 2 channel) name what a computed
    mean / stddev is taken over; an empty mean / stddev list asks for it to be computed per sample."""
    p = _pipe()
    ax = (ctypes.c_uint * max(len(axes), 1))(*[int(a) for a in axes])
    return _ret(p, C.normalize(p._handle, inputs[0], ax, len(axes), _farr(mean) if len(mean) else None, len(mean),
                               _farr(stddev) if len(stddev) else None, len(stddev), 0, float(scale), float(shift), output_datatype))


def transpose(*inputs, perm=[], output_layout=types.NHWC, output_dtype=types.UINT8):
    """fn.py:1239: reorders the per-sample axes (height, width, channel) by perm."""
    p = _pipe()
    pm = (ctypes.c_uint * max(len(perm), 1))(*[int(a) for a in perm])
    return _ret(p, C.transpose(p._handle, inputs[0], pm, len(perm), 0, output_layout))


def hue(*inputs, hue=None, device=None, seed=0, output_layout=types.NHWC, output_dtype=types.UINT8):
    p = _pipe()
    return _ret(p, C.hue(p._handle, inputs[0], 0, _fparam(hue), output_layout, output_dtype))


def saturation(*inputs, saturation=1.0, device=None, output_layout=types.NHWC, output_dtype=types.UINT8):
    p = _pipe()
    return _ret(p, C.saturation(p._handle, inputs[0], 0, _fparam(saturation), output_layout, output_dtype))


def color_twist(*inputs, brightness=1.0, contrast=1.0, hue=0.0, saturation=1.0, device=None, output_layout=types.NHWC,
                output_dtype=types.UINT8):
    p = _pipe()
    return _ret(p, C.color_twist(p._handle, inputs[0], 0, _fparam(brightness), _fparam(contrast), _fparam(hue),
                                 _fparam(saturation), output_layout, output_dtype))


def warp_affine(*inputs, dest_width=0, dest_height=0, matrix=[0, 0, 0, 0, 0, 0], interpolation_type=types.LINEAR_INTERPOLATION,
                device=None, output_layout=types.NHWC, output_dtype=types.UINT8):
    """matrix = [x0, x1, y0, y1, o0, o1] (fn.py:686-708); per-sample tables go through Pipeline.set_affine."""
    p = _pipe()
    x0, x1, y0, y1, o0, o1 = [_fparam(v) for v in matrix]
    return _ret(p, C.warp_affine(p._handle, inputs[0], 0, dest_height, dest_width, x0, x1, y0, y1, o0, o1,
                                 interpolation_type, output_layout, output_dtype))


def rotate(*inputs, angle=None, dest_width=0, dest_height=0, interpolation_type=types.LINEAR_INTERPOLATION, device=None,
           fill_value=None, output_layout=types.NHWC, output_dtype=types.UINT8):
    """fill_value is accepted and unused, as in the reference's wrapper (the border is zero)."""
    p = _pipe()
    return _ret(p, C.rotate(p._handle, inputs[0], 0, _fparam(angle), dest_width, dest_height, interpolation_type,
                            output_layout, output_dtype))


def box_iou_matcher(*inputs, anchors, high_threshold=0.5, low_threshold=0.4, allow_low_quality_matches=True, device=None):
    """amd.rocal.fn.box_iou_matcher: enables the matcher; read the result with Pipeline.get_matched_indices()."""
    p = _pipe()
    flat = [float(v) for v in (anchors.reshape(-1) if hasattr(anchors, "reshape") else anchors)]
    p._check(C.box_iou_matcher(p._handle, _farr(flat), len(flat) // 4, high_threshold, low_threshold,
                               1 if allow_low_quality_matches else 0))
    return None, []


def box_encoder(*inputs, anchors, criteria=0.5, means=None, offset=False, scale=1.0, stds=None, device=None):
    p = _pipe()
    means = means if means else [0.0, 0.0, 0.0, 0.0]
    stds = stds if stds else [1.0, 1.0, 1.0, 1.0]
    flat = [float(v) for v in (anchors.reshape(-1) if hasattr(anchors, "reshape") else anchors)]
    p._check(C.box_encoder(p._handle, _farr(flat), len(flat) // 4, criteria, _farr(means), _farr(stds), 1 if offset else 0, scale))
    p._box_encoder = True
    p._num_anchors = len(flat) // 4
    return None, []

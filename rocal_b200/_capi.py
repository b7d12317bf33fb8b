"""ctypes prototypes of the pipeline C ABI (include/rb200.h)."""
import ctypes
from ctypes import POINTER, c_char_p, c_double, c_float, c_int, c_size_t, c_uint, c_uint32, c_uint64, c_void_p

from ._lib import lib


class ImageDesc(ctypes.Structure):
    _fields_ = [("offset", c_uint64), ("stride", c_uint32), ("width", c_uint32), ("height", c_uint32)]


MEM_HOST, MEM_HOST_PINNED, MEM_DEVICE = 0, 1, 2


class Param:
    """Opaque RocalIntParam / RocalFloatParam handle (so that it is never mistaken for a number)."""

    def __init__(self, handle, is_int):
        if not handle:
            raise RuntimeError("parameter creation failed")
        self.handle, self.is_int = handle, is_int
        self._as_parameter_ = ctypes.c_void_p(handle)


_P = c_void_p


def _proto(name, restype, *argtypes):
    f = getattr(lib, name)
    f.restype = restype
    f.argtypes = list(argtypes)
    return f


create = _proto("rb200_create", _P, c_size_t, c_int, c_int, c_size_t, c_size_t, c_int)
verify = _proto("rb200_verify", c_int, _P)
run = _proto("rb200_run", c_int, _P)
release = _proto("rb200_release", c_int, _P)
get_status = _proto("rb200_get_status", c_int, _P)
get_error_message = _proto("rb200_get_error_message", c_char_p, _P)
get_timing = _proto("rb200_get_timing", None, _P, POINTER(ctypes.c_ulonglong))
feed_encoded = _proto("rb200_feed_encoded", c_int, _P, POINTER(c_void_p), POINTER(c_size_t), c_size_t)
feed_files = _proto("rb200_feed_files", c_int, _P, POINTER(ctypes.c_char_p), c_size_t)
set_file_list = _proto("rb200_set_file_list", c_int, _P, c_char_p)
jpeg_file_source = _proto("rb200_jpeg_file_source", _P, _P, c_char_p, c_int, c_uint, c_uint, c_int, c_int, c_int, c_uint, c_uint, c_int, c_int)
coco_file_source = _proto("rb200_coco_file_source", _P, _P, c_char_p, c_char_p, c_int, c_uint, c_uint, c_int, c_int, c_int, c_uint, c_uint, c_int, c_int, c_int)
reset_loaders = _proto("rb200_reset_loaders", c_int, _P)
get_image_labels = _proto("rb200_get_image_labels", c_int, _P, POINTER(c_int))
get_image_name_len = _proto("rb200_get_image_name_len", c_uint, _P, POINTER(c_int))
get_image_name = _proto("rb200_get_image_name", c_int, _P, c_char_p)
get_one_hot_image_labels = _proto("rb200_get_one_hot_image_labels", c_int, _P, c_void_p, c_int, c_int)
fused_jpeg_crop_file_source = _proto("rb200_fused_jpeg_crop_file_source", _P, _P, c_char_p, c_int, c_uint, c_uint, c_int,
                                     POINTER(c_float), POINTER(c_float), c_uint, c_int, c_int, c_uint, c_uint, c_int, c_int)
set_random_crop_decoder = _proto("rb200_set_random_crop_decoder", c_int, _P, POINTER(c_float), POINTER(c_float), c_uint)
get_decoder_crop_windows = _proto("rb200_get_decoder_crop_windows", c_int, _P, POINTER(c_uint), POINTER(c_uint))
class StepTiming(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char * 32), ("gpu_us", ctypes.c_double), ("batches", ctypes.c_ulonglong)]


set_profiling = _proto("rb200_set_profiling", c_int, _P, c_int)
get_step_timing = _proto("rb200_get_step_timing", c_size_t, _P, POINTER(StepTiming), c_size_t)
random_bbox_crop = _proto("rb200_random_bbox_crop", c_int, _P, c_int, c_int, c_uint)
get_bbox_crop_windows = _proto("rb200_get_bbox_crop_windows", c_int, _P, POINTER(c_float))
bbox_crop_windows = _proto("rb200_bbox_crop_windows", c_int, c_uint, c_int, c_int, POINTER(c_float), POINTER(c_int), c_size_t,
                           POINTER(c_int), POINTER(c_float))
random_crop_windows = _proto("rb200_random_crop_windows", c_int, c_uint, POINTER(c_int), c_size_t, POINTER(c_float),
                             POINTER(c_float), c_uint, POINTER(c_uint))
get_image_sizes = _proto("rb200_get_image_sizes", c_int, _P, POINTER(c_int))
get_image_ids = _proto("rb200_get_image_ids", c_int, _P, POINTER(c_int))
get_roi_image_sizes = _proto("rb200_get_roi_image_sizes", c_int, _P, POINTER(c_int))
get_last_batch_padded_size = _proto("rb200_get_last_batch_padded_size", c_size_t, _P)
get_h2d_bytes = _proto("rb200_get_h2d_bytes", ctypes.c_ulonglong, _P)
set_upload_mode = _proto("rb200_set_upload_mode", ctypes.c_int, _P, ctypes.c_int)
set_arithmetic = _proto("rb200_set_arithmetic", ctypes.c_int, _P, ctypes.c_int)
consumer_fence = _proto("rb200_consumer_fence", ctypes.c_int, _P, ctypes.c_void_p)
set_wait_probe = _proto("rb200_set_wait_probe", ctypes.c_int, _P, ctypes.c_ulonglong, ctypes.c_int)
get_remaining_images = _proto("rb200_get_remaining_images", c_size_t, _P)
set_seed = _proto("rb200_set_seed", None, c_uint)
get_seed = _proto("rb200_get_seed", c_uint)
create_int_uniform_rand = _proto("rb200_create_int_uniform_rand", _P, c_int, c_int)
create_float_uniform_rand = _proto("rb200_create_float_uniform_rand", _P, c_float, c_float)
create_int_rand = _proto("rb200_create_int_rand", _P, POINTER(c_int), POINTER(c_double), c_uint)
create_float_rand = _proto("rb200_create_float_rand", _P, POINTER(c_float), POINTER(c_double), c_uint)
create_int_parameter = _proto("rb200_create_int_parameter", _P, c_int)
create_float_parameter = _proto("rb200_create_float_parameter", _P, c_float)
update_int_parameter = _proto("rb200_update_int_parameter", c_int, c_int, _P)
update_float_parameter = _proto("rb200_update_float_parameter", c_int, c_float, _P)
update_int_uniform_rand = _proto("rb200_update_int_uniform_rand", c_int, c_int, c_int, _P)
update_float_uniform_rand = _proto("rb200_update_float_uniform_rand", c_int, c_float, c_float, _P)
get_int_value = _proto("rb200_get_int_value", c_int, _P)
get_float_value = _proto("rb200_get_float_value", c_float, _P)
external_source = _proto("rb200_external_source", _P, _P, c_int, c_int, c_uint, c_uint, c_int)
feed_input = _proto("rb200_feed_input", c_int, _P, POINTER(c_void_p), POINTER(c_uint), c_size_t, c_uint, c_uint, c_uint,
                    c_int, c_int, c_int)
feed_ragged = _proto("rb200_feed_ragged", c_int, _P, c_void_p, c_size_t, POINTER(ImageDesc), c_size_t, c_int)
feed_boxes = _proto("rb200_feed_boxes", c_int, _P, POINTER(c_float), POINTER(c_int), POINTER(c_int), c_size_t)
set_crop_anchors = _proto("rb200_set_crop_anchors", c_int, _P, _P, POINTER(c_float), POINTER(c_float), c_size_t)
set_affine = _proto("rb200_set_affine", c_int, _P, _P, POINTER(c_float), c_size_t)
resize = _proto("rb200_resize", _P, _P, _P, c_uint, c_uint, c_int, c_int, c_uint, c_uint, c_uint, c_uint, c_int, c_int, c_int)
resize_mirror_normalize = _proto("rb200_resize_mirror_normalize", _P, _P, _P, c_uint, c_uint, POINTER(c_float),
                                 POINTER(c_float), c_size_t, c_int, c_int, c_uint, c_uint, c_uint, c_uint, c_int, _P,
                                 c_int, c_int)
crop_mirror_normalize = _proto("rb200_crop_mirror_normalize", _P, _P, _P, c_uint, c_uint, c_float, c_float,
                               POINTER(c_float), POINTER(c_float), c_size_t, c_int, _P, c_int, c_int)
crop = _proto("rb200_crop", _P, _P, _P, c_int, _P, _P, _P, _P, c_int, c_int)
crop_fixed = _proto("rb200_crop_fixed", _P, _P, _P, c_uint, c_uint, c_int, c_float, c_float, c_int, c_int)
crop_center_fixed = _proto("rb200_crop_center_fixed", _P, _P, _P, c_uint, c_uint, c_int, c_int, c_int)
resize_crop_mirror_fixed = _proto("rb200_resize_crop_mirror_fixed", _P, _P, _P, c_uint, c_uint, c_int, c_uint, c_uint,
                                  _P, c_int, c_int)
resize_crop_mirror = _proto("rb200_resize_crop_mirror", _P, _P, _P, c_uint, c_uint, c_int, _P, _P, _P, c_int, c_int)
random_area_windows = _proto("rb200_random_area_windows", c_int, POINTER(c_uint), c_size_t, _P, _P, _P, _P, POINTER(c_uint))
random_crop = _proto("rb200_random_crop", _P, _P, _P, c_int, _P, _P, _P, _P, c_int, c_int, c_int)
crop_resize = _proto("rb200_crop_resize", _P, _P, _P, c_uint, c_uint, c_int, _P, _P, _P, _P, c_int, c_int)
roi_resize = _proto("rb200_roi_resize", _P, _P, _P, c_uint, c_uint, c_int, c_uint, c_uint, c_float, c_float, c_int, c_int, c_int)
ssd_random_crop = _proto("rb200_ssd_random_crop", _P, _P, _P, c_int, c_int, c_int, c_int)
flip = _proto("rb200_flip", _P, _P, _P, c_int, _P, _P, c_int, c_int)
brightness = _proto("rb200_brightness", _P, _P, _P, c_int, _P, _P, c_int, c_int)
contrast = _proto("rb200_contrast", _P, _P, _P, c_int, _P, _P, c_int, c_int)
normalize = _proto("rb200_normalize", _P, _P, _P, ctypes.POINTER(ctypes.c_uint), ctypes.c_uint, ctypes.POINTER(ctypes.c_float), ctypes.c_uint,
                   ctypes.POINTER(ctypes.c_float), ctypes.c_uint, c_int, ctypes.c_float, ctypes.c_float, c_int)
transpose = _proto("rb200_transpose", _P, _P, _P, ctypes.POINTER(ctypes.c_uint), ctypes.c_uint, c_int, c_int)
hue = _proto("rb200_hue", _P, _P, _P, c_int, _P, c_int, c_int)
blend = _proto("rb200_blend", _P, _P, _P, _P, c_int, _P, c_int, c_int)
exposure = _proto("rb200_exposure", _P, _P, _P, c_int, _P, c_int, c_int)
gamma = _proto("rb200_gamma", _P, _P, _P, c_int, _P, c_int, c_int)
color_temp = _proto("rb200_color_temp", _P, _P, _P, c_int, _P, c_int, c_int)
saturation = _proto("rb200_saturation", _P, _P, _P, c_int, _P, c_int, c_int)
color_twist = _proto("rb200_color_twist", _P, _P, _P, c_int, _P, _P, _P, _P, c_int, c_int)
warp_affine = _proto("rb200_warp_affine", _P, _P, _P, c_int, c_uint, c_uint, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int)
rotate = _proto("rb200_rotate", _P, _P, _P, c_int, _P, c_uint, c_uint, c_int, c_int, c_int)
set_outputs = _proto("rb200_set_outputs", c_int, _P, POINTER(c_void_p), c_size_t)
output_count = _proto("rb200_output_count", c_size_t, _P)
output = _proto("rb200_output", _P, _P, c_size_t)
tensor_buffer = _proto("rb200_tensor_buffer", _P, _P)
tensor_num_dims = _proto("rb200_tensor_num_dims", c_uint, _P)
tensor_dims = _proto("rb200_tensor_dims", None, _P, POINTER(c_size_t))
tensor_strides = _proto("rb200_tensor_strides", None, _P, POINTER(c_size_t))
tensor_layout = _proto("rb200_tensor_layout", c_int, _P)
tensor_dtype = _proto("rb200_tensor_dtype", c_int, _P)
tensor_data_size = _proto("rb200_tensor_data_size", c_size_t, _P)
tensor_copy_data = _proto("rb200_tensor_copy_data", c_uint, _P, c_void_p, c_int)
tensor_copy_roi = _proto("rb200_tensor_copy_roi", None, _P, c_void_p)
tensor_dlpack = _proto("rb200_tensor_dlpack", _P, _P)
device_id = _proto("rb200_device_id", c_int, _P)
stream = _proto("rb200_stream", _P, _P)
to_tensor = _proto("rb200_to_tensor", c_int, _P, c_void_p, c_int, c_int, POINTER(c_float), POINTER(c_float), c_int, c_int)
box_encoder = _proto("rb200_box_encoder", c_int, _P, POINTER(c_float), c_size_t, c_float, POINTER(c_float),
                     POINTER(c_float), c_int, c_float)
box_iou_matcher = _proto("rb200_box_iou_matcher", c_int, _P, POINTER(c_float), c_size_t, c_float, c_float, c_int)
get_matched_indices = _proto("rb200_get_matched_indices", c_int, _P, POINTER(c_void_p), POINTER(c_size_t))
copy_matched_indices = _proto("rb200_copy_matched_indices", c_int, _P, POINTER(c_int))
copy_encoded_boxes_and_labels = _proto("rb200_copy_encoded_boxes_and_labels", c_int, _P, POINTER(c_float), POINTER(c_int))
get_encoded_boxes_and_labels = _proto("rb200_get_encoded_boxes_and_labels", c_int, _P, POINTER(c_void_p), POINTER(c_void_p),
                                      POINTER(c_size_t))
get_bounding_boxes = _proto("rb200_get_bounding_boxes", c_size_t, _P, POINTER(c_float), POINTER(c_int), POINTER(c_int))
get_crop_windows = _proto("rb200_get_crop_windows", c_int, _P, _P, POINTER(c_uint))
get_int_array = _proto("rb200_get_int_array", c_size_t, _P, POINTER(c_int), c_size_t)
get_float_array = _proto("rb200_get_float_array", c_size_t, _P, POINTER(c_float), c_size_t)
get_batch_int_array = _proto("rb200_get_batch_int_array", c_size_t, _P, _P, POINTER(c_int), c_size_t)
get_batch_float_array = _proto("rb200_get_batch_float_array", c_size_t, _P, _P, POINTER(c_float), c_size_t)

"""Python face of the pipeline, shaped like amd.rocal.pipeline.Pipeline
(rocAL_pybind/amd/rocal/pipeline.py:34-273) for the supported subset.

    pipe = Pipeline(batch_size=64, device_id=0, seed=0)
    with pipe:
        img = fn.external_source(None, mode=types.EXTSOURCE_RAW_UNCOMPRESSED, max_width=512, max_height=512)[0]
        r = fn.resize(img, resize_shorter=256)
        out = fn.crop_mirror_normalize(r, crop=[224, 224], mean=..., std=..., mirror=fn.random.coin_flip(),
                                       output_layout=types.NCHW, output_dtype=types.FLOAT)
        pipe.set_outputs(out)
    pipe.build()
    pipe.feed_ragged(arena, heights, widths, offsets)      # or pipe.feed_input(list_of_hwc_arrays)
    pipe.run()
    tensors = pipe.get_output_tensors()                     # list of RocalTensor (DLPack capable)
"""
import collections
import ctypes

import numpy as np

from . import _capi as C
from . import types


_IMAGE_DESC = np.dtype({"names": ["offset", "stride", "width", "height"], "formats": [np.uint64, np.uint32, np.uint32, np.uint32],
                        "offsets": [0, 8, 12, 16], "itemsize": ctypes.sizeof(C.ImageDesc)})


class RocalError(RuntimeError):
    pass


class RocalTensor:
    """Output tensor handle: device memory owned by the pipeline, valid until the next run()."""

    def __init__(self, pipe, handle):
        self._pipe, self._h = pipe, handle

    def dims(self):
        n = C.tensor_num_dims(self._h)
        buf = (ctypes.c_size_t * n)()
        C.tensor_dims(self._h, buf)
        return list(buf)

    def strides(self):
        n = C.tensor_num_dims(self._h)
        buf = (ctypes.c_size_t * n)()
        C.tensor_strides(self._h, buf)
        return list(buf)

    def layout(self):
        return C.tensor_layout(self._h)

    def dtype(self):
        return C.tensor_dtype(self._h)

    def data_size(self):
        return C.tensor_data_size(self._h)

    def buffer(self):
        return C.tensor_buffer(self._h)

    def roi(self):
        n = self.dims()[0]
        out = np.zeros((n, 4), dtype=np.uint32)
        C.tensor_copy_roi(self._h, out.ctypes.data_as(ctypes.c_void_p))
        return out

    def copy_data(self, dst, mem_type=types.HOST_MEMORY):
        """dst: a numpy array (filled in place), an integer address or a ctypes pointer of a buffer of data_size() bytes
        (the calling forms of the reference's binding, rocal_pybind.cpp:532-557)."""
        if isinstance(dst, np.ndarray):
            ptr = dst.ctypes.data
        else:
            ptr = dst if isinstance(dst, int) else ctypes.cast(dst, ctypes.c_void_p).value
        if C.tensor_copy_data(self._h, ctypes.c_void_p(ptr), mem_type):
            raise RocalError(self._pipe.error_message())

    # names of the reference's binding (rocal_pybind.cpp:478-531)
    def max_shape(self):
        return self.dims()

    def dimensions(self):
        return self.dims()

    def batch_size(self):
        return self.dims()[0]

    def roi_dims_size(self):
        return 2

    def copy_roi(self, array):
        """Fills a uint32 numpy array with x, y, w, h per sample."""
        np.asarray(array).reshape(-1)[:4 * self.dims()[0]] = self.roi().reshape(-1)

    def numpy(self):
        np_dt = {types.FLOAT: np.float32, types.FLOAT16: np.float16, types.UINT8: np.uint8, types.INT32: np.int32}[self.dtype()]
        out = np.empty(self.dims(), dtype=np_dt)
        self.copy_data(out.ctypes.data)
        return out

    def __dlpack_device__(self):
        return (2, C.device_id(self._pipe._handle))   # kDLCUDA

    def __dlpack__(self, stream=None, **_):
        """Zero-copy export. The batch is complete when run() returns, so the consumer never waits for the pipeline;
        the other direction is what `stream` is for: the pipeline remembers the consumer's stream (DLPack's
        convention: None or 1 = the legacy default stream, 2 = the per-thread default stream, -1 = no ordering
        wanted, anything else a cudaStream_t) and, at the next run(), orders the reuse of this batch's buffers behind
        whatever the consumer has queued there by then (rb200_consumer_fence)."""
        if stream != -1:
            self._pipe._consumer_streams.add(0 if stream in (None, 1) else int(stream))
        m = C.tensor_dlpack(self._h)
        if not m:
            raise RocalError("no batch is available yet (call run() first)")
        ctypes.pythonapi.PyCapsule_New.restype = ctypes.py_object
        ctypes.pythonapi.PyCapsule_New.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p]
        return ctypes.pythonapi.PyCapsule_New(m, b"dltensor", None)


class Pipeline(object):
    _current_pipeline = None

    def __init__(self, batch_size=-1, num_threads=0, device_id=0, seed=1, exec_pipelined=True, prefetch_queue_depth=2,
                 exec_async=True, bytes_per_sample=0, rocal_cpu=False, max_streams=-1, default_cuda_stream_priority=0,
                 tensor_layout=types.NCHW, reverse_channels=False, mean=None, std=None, tensor_dtype=types.FLOAT,
                 output_memory_type=None):
        if rocal_cpu:
            raise RocalError("this library has no CPU backend (rocal_cpu must be False)")
        self._handle = C.create(batch_size, types.GPU, device_id, max(1, num_threads), prefetch_queue_depth, tensor_dtype)
        if not self._handle:
            raise RocalError("Failed creating the pipeline")
        self._batch_size = batch_size
        self._device_id = device_id
        self._tensor_layout = tensor_layout
        self._tensor_dtype = tensor_dtype
        self._multiplier = [1.0 / x for x in std] if std else [1.0, 1.0, 1.0]
        self._offset = [-(m / s) for m, s in zip(mean, std)] if mean and std else [0.0, 0.0, 0.0]
        self._reverse_channels = reverse_channels
        self._outputs = []
        self._keepalive = collections.deque()    # one entry per fed batch that rocal_run has not returned yet
        self._consumer_streams = set()           # streams the held batch was exported to through DLPack
        self._box_encoder = False
        self._num_anchors = 0
        self._external_source_mode = None
        self._max_w = self._max_h = 0
        self.set_seed(seed)

    # ---- graph ----
    def __enter__(self):
        Pipeline._current_pipeline = self
        return self

    def __exit__(self, *exc):
        Pipeline._current_pipeline = None

    def get_handle(self):
        return self._handle

    def set_seed(self, seed=0):
        C.set_seed(seed)

    def set_outputs(self, *output_list):
        self._outputs = list(output_list)

    def build(self):
        if self._outputs:
            arr = (ctypes.c_void_p * len(self._outputs))(*self._outputs)
            self._check(C.set_outputs(self._handle, arr, len(self._outputs)))
        self._check(C.verify(self._handle))
        return self

    # ---- parameters (Pipeline.create_int_param ... pipeline.py:173-193) ----
    def create_int_param(self, value=1):
        return C.Param(C.create_int_parameter(value), True)

    def create_float_param(self, value=1):
        return C.Param(C.create_float_parameter(value), False)

    def update_int_param(self, value=1, param=1):
        return C.update_int_parameter(value, param)

    def update_float_param(self, value=1, param=1):
        return C.update_float_parameter(value, param)

    def get_int_value(self, param):
        return C.get_int_value(param)

    def get_float_value(self, param):
        return C.get_float_value(param)

    # ---- input ----
    def feed_input(self, images):
        """The reference's external-source contract: a list of HWC uint8 arrays, each copied into a
        max_height x max_width slot (Pipeline/external source mode RAW_UNCOMPRESSED)."""
        n = len(images)
        slots = np.zeros((n, self._max_h, self._max_w, 3), dtype=np.uint8)
        roi = np.zeros((n, 4), dtype=np.uint32)
        for i, im in enumerate(images):
            h, w = im.shape[:2]
            slots[i, :h, :w] = im
            roi[i] = (0, 0, w, h)
        ptrs = (ctypes.c_void_p * n)(*[slots[i].ctypes.data for i in range(n)])
        self._keepalive.append((slots, roi, ptrs))
        self._check(C.feed_input(self._handle, ptrs, roi.ctypes.data_as(ctypes.POINTER(ctypes.c_uint)), n, self._max_w,
                                 self._max_h, 3, types.EXTSOURCE_RAW_UNCOMPRESSED, types.NHWC, 0))

    def feed_ragged(self, arena, heights, widths, offsets, strides=None, mem_kind=None):
        """[extension] One packed arena (numpy array, torch tensor — host, pinned or CUDA) + per-image sizes."""
        n = len(heights)
        # rb200_image_desc rows built in one go (a per-image Python loop costs ~1 us per image)
        d = np.zeros(n, dtype=_IMAGE_DESC)
        d["offset"] = offsets
        d["width"] = widths
        d["height"] = heights
        d["stride"] = strides if strides is not None else np.asarray(widths, dtype=np.int64) * 3
        descs = d.ctypes.data_as(ctypes.POINTER(C.ImageDesc))
        if isinstance(arena, np.ndarray):
            ptr, nbytes, kind = arena.ctypes.data, arena.nbytes, C.MEM_HOST
        else:   # torch tensor
            ptr, nbytes = arena.data_ptr(), arena.numel() * arena.element_size()
            kind = C.MEM_DEVICE if arena.is_cuda else (C.MEM_HOST_PINNED if arena.is_pinned() else C.MEM_HOST)
        if mem_kind is not None:
            kind = mem_kind
        self._keepalive.append((arena, d))
        self._check(C.feed_ragged(self._handle, ctypes.c_void_p(ptr), nbytes, descs, n, kind))

    def feed_encoded(self, streams):
        """JPEG streams (bytes objects or uint8 numpy arrays), one per sample: decoded on the GPU (nvJPEG) into the
        arena the kernels read. The source must have been created with mode=EXTSOURCE_RAW_COMPRESSED."""
        n = len(streams)
        arrs = [np.frombuffer(s, dtype=np.uint8) if isinstance(s, (bytes, bytearray, memoryview)) else np.ascontiguousarray(s, dtype=np.uint8)
                for s in streams]
        ptrs = (ctypes.c_void_p * n)(*[a.ctypes.data for a in arrs])
        sizes = (ctypes.c_size_t * n)(*[a.nbytes for a in arrs])
        self._keepalive.append((arrs, ptrs, sizes))
        self._check(C.feed_encoded(self._handle, ptrs, sizes, n))

    def feed_files(self, paths):
        """JPEG files by name (the FNAME mode of rocalExternalSourceFeedInput)."""
        n = len(paths)
        arr = (ctypes.c_char_p * n)(*[str(p).encode() for p in paths])
        self._keepalive.append(None)       # keeps the one-entry-per-fed-batch order of the queue
        self._check(C.feed_files(self._handle, arr, n))

    def feed_boxes(self, boxes, labels, counts):
        """[extension] Normalized ltrb boxes, labels and per-sample counts of the next fed batch."""
        b = np.ascontiguousarray(boxes, dtype=np.float32)
        lab = np.ascontiguousarray(labels, dtype=np.int32)
        c = np.ascontiguousarray(counts, dtype=np.int32)
        self._check(C.feed_boxes(self._handle, b.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
                                 lab.ctypes.data_as(ctypes.POINTER(ctypes.c_int)),
                                 c.ctypes.data_as(ctypes.POINTER(ctypes.c_int)), len(c)))

    def set_crop_anchors(self, cmn_output, anchor_x, anchor_y):
        ax = np.ascontiguousarray(anchor_x, dtype=np.float32)
        ay = np.ascontiguousarray(anchor_y, dtype=np.float32)
        self._check(C.set_crop_anchors(self._handle, cmn_output, ax.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
                                       ay.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), len(ax)))

    def set_affine(self, warp_output, matrices):
        m = np.ascontiguousarray(matrices, dtype=np.float32).reshape(-1, 6)
        self._check(C.set_affine(self._handle, warp_output, m.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), len(m)))

    # ---- run / outputs ----
    def rocal_run(self):
        for stream in self._consumer_streams:      # consumers of the batch that is about to go back to the ring
            C.consumer_fence(self._handle, ctypes.c_void_p(stream))
        self._consumer_streams.clear()
        self._check(C.run(self._handle))
        # the batch just returned has been consumed: its host buffers (oldest entry) may go. Every other entry
        # belongs to a batch that is still queued, whatever their number.
        if self._keepalive:
            self._keepalive.popleft()
        return types.OK

    def set_arithmetic(self, mode):
        """[extension] 0 = exact (bit-identical to the CPU restatement), 1 = fast colour arithmetic (every uint8
        output within one level of exact)."""
        if C.set_arithmetic(self._handle, int(mode)) != 0:
            raise ValueError("arithmetic mode must be 0 or 1")

    def run(self):
        """pipeline.py:262-275 of the reference: runs the next batch and returns its output tensors; StopIteration when
        a pipeline that reads files itself has reached the end of its data."""
        if getattr(self, "_has_file_source", False) and self.is_empty():
            raise StopIteration
        self.rocal_run()
        return self.get_output_tensors()

    def get_output_tensors(self):
        return [RocalTensor(self, C.output(self._handle, i)) for i in range(C.output_count(self._handle))]

    def copyToExternalTensor(self, array, multiplier, offset, reverse_channels, tensor_format, tensor_dtype,
                             max_roi_height=0, max_roi_width=0):
        """rocalToTensor into a numpy array (host) or a CUDA torch tensor."""
        mul = (ctypes.c_float * 3)(*multiplier)
        off = (ctypes.c_float * 3)(*offset)
        if isinstance(array, np.ndarray):
            ptr, mem = array.ctypes.data, types.HOST_MEMORY
        else:
            ptr, mem = array.data_ptr(), (types.DEVICE_MEMORY if array.is_cuda else types.HOST_MEMORY)
        self._check(C.to_tensor(self._handle, ctypes.c_void_p(ptr), tensor_format, tensor_dtype, mul, off,
                                1 if reverse_channels else 0, mem))

    def copy_encoded_boxes_and_lables(self, bbox_array, label_array):
        self._check(C.copy_encoded_boxes_and_labels(self._handle, bbox_array.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
                                                    label_array.ctypes.data_as(ctypes.POINTER(ctypes.c_int))))

    def get_encoded_boxes_and_lables(self, batch_size=None, num_anchors=None):
        """Returns (boxes [N, A, 4] float32, labels [N, A] int32) as numpy arrays."""
        bp, lp, na = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_size_t()
        self._check(C.get_encoded_boxes_and_labels(self._handle, ctypes.byref(bp), ctypes.byref(lp), ctypes.byref(na)))
        boxes = np.empty((self._batch_size, na.value, 4), dtype=np.float32)
        labels = np.empty((self._batch_size, na.value), dtype=np.int32)
        self.copy_encoded_boxes_and_lables(boxes, labels)
        return boxes, labels

    def get_image_labels(self):
        """rocalGetImageLabels: class label of every sample of the current batch (file source), int32 numpy array."""
        out = np.empty(self._batch_size, dtype=np.int32)
        self._check(C.get_image_labels(self._handle, out.ctypes.data_as(ctypes.POINTER(ctypes.c_int))))
        return out

    def get_one_hot_encoded_labels(self, num_classes, device=None):
        """rocalGetOneHotImageLabels: int32 [N, num_classes]; a numpy array, or a CUDA torch tensor when device is given."""
        if device is None:
            out = np.zeros((self._batch_size, num_classes), dtype=np.int32)
            self._check(C.get_one_hot_image_labels(self._handle, ctypes.c_void_p(out.ctypes.data), num_classes, types.HOST_MEMORY))
            return out
        import torch
        out = torch.zeros((self._batch_size, num_classes), dtype=torch.int32, device=device)
        self._check(C.get_one_hot_image_labels(self._handle, ctypes.c_void_p(out.data_ptr()), num_classes, types.DEVICE_MEMORY))
        return out

    def get_image_sizes(self):
        """rocalGetImageSizes: (width, height) of every source image of the batch as it was read, int32 [N, 2]."""
        out = np.zeros((self._batch_size, 2), dtype=np.int32)
        self._check(C.get_image_sizes(self._handle, out.ctypes.data_as(ctypes.POINTER(ctypes.c_int))))
        return out

    def get_image_id(self, array=None):
        """rocalGetImageId: the annotation file's id of every image of the batch (COCO reader), int32 [N]; written into
        `array` too when one is given (the reference's calling form)."""
        out = np.zeros(self._batch_size, dtype=np.int32)
        self._check(C.get_image_ids(self._handle, out.ctypes.data_as(ctypes.POINTER(ctypes.c_int))))
        if array is not None:
            np.asarray(array).reshape(-1)[:self._batch_size] = out
        return out

    def get_roi_image_sizes(self):
        """rocalGetROIImageSizes: (width, height) of the valid region of every sample after ResizeMirrorNormalize (of the
        first output when the graph has none), int32 [N, 2]."""
        out = np.zeros((self._batch_size, 2), dtype=np.int32)
        self._check(C.get_roi_image_sizes(self._handle, out.ctypes.data_as(ctypes.POINTER(ctypes.c_int))))
        return out

    def set_random_crop_decoder(self, random_area=(0.08, 1.0), random_aspect_ratio=(3.0 / 4, 4.0 / 3), num_attempts=10):
        """[extension] Random-resized-crop windows on an external source fed with encoded JPEG (what
        decoders.image_slice does for a folder reader). Call inside `with pipeline:` before build()."""
        area = (ctypes.c_float * 2)(*random_area)
        aspect = (ctypes.c_float * 2)(*random_aspect_ratio)
        self._check(C.set_random_crop_decoder(self._handle, area, aspect, int(num_attempts)))

    def get_decoder_crop_windows(self):
        """[extension] The crop windows (x, y, w, h) of the current batch inside the decoded images, uint32 [N, 4],
        and the batch seed they were drawn from."""
        out = np.zeros((self._batch_size, 4), dtype=np.uint32)
        seed = ctypes.c_uint(0)
        self._check(C.get_decoder_crop_windows(self._handle, out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint)), ctypes.byref(seed)))
        return out, int(seed.value)

    def set_profiling(self, on=True):
        """[extension] Per-launch device timing with CUDA events; call before build()."""
        self._check(C.set_profiling(self._handle, int(bool(on))))

    def step_timing(self):
        """[extension] [(name, device microseconds per batch, batches measured)]: the upload, then every launch of the
        plan in order. Empty unless profiling is on."""
        buf = (C.StepTiming * 64)()
        k = min(int(C.get_step_timing(self._handle, buf, 64)), 64)
        return [(buf[i].name.decode(), buf[i].gpu_us / max(1, buf[i].batches), int(buf[i].batches)) for i in range(k)]

    def get_bbox_crop_windows(self):
        """[extension] The windows rocalRandomBBoxCrop sampled for the current batch, float32 [N, 4] = (x, y, w, h) as
        fractions of the image; get_decoder_crop_windows() gives the same windows in pixels."""
        out = np.zeros((self._batch_size, 4), dtype=np.float32)
        self._check(C.get_bbox_crop_windows(self._handle, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float))))
        return out

    def get_image_names(self):
        """rocalGetImageNameLen + rocalGetImageName: file names of the current batch."""
        lens = (ctypes.c_int * self._batch_size)()
        total = C.get_image_name_len(self._handle, lens)
        buf = ctypes.create_string_buffer(total + 1)
        self._check(C.get_image_name(self._handle, buf))
        raw, names, pos = buf.raw[:total], [], 0
        for k in lens:
            names.append(raw[pos:pos + k].decode())
            pos += k
        return names

    def reset(self):
        """rocalResetLoaders: the file source starts its next epoch."""
        self._check(C.reset_loaders(self._handle))

    def get_last_batch_padded_size(self):
        return int(C.get_last_batch_padded_size(self._handle))

    def get_matched_indices(self):
        """rocalGetMatchedIndices: matched box index per anchor, [N, A] int32 (numpy)."""
        mp, na = ctypes.c_void_p(), ctypes.c_size_t()
        self._check(C.get_matched_indices(self._handle, ctypes.byref(mp), ctypes.byref(na)))
        out = np.empty((self._batch_size, na.value), dtype=np.int32)
        self._check(C.copy_matched_indices(self._handle, out.ctypes.data_as(ctypes.POINTER(ctypes.c_int))))
        return out

    def get_bounding_boxes(self):
        """Boxes of the current batch after the graph's crops and mirrors: (ltrb [T,4], labels [T], counts [N])."""
        total = C.get_bounding_boxes(self._handle, None, None, None)
        b = np.zeros((total, 4), dtype=np.float32)
        lab = np.zeros(total, dtype=np.int32)
        c = np.zeros(self._batch_size, dtype=np.int32)
        if total:
            C.get_bounding_boxes(self._handle, b.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
                                 lab.ctypes.data_as(ctypes.POINTER(ctypes.c_int)), c.ctypes.data_as(ctypes.POINTER(ctypes.c_int)))
        return b, lab, c

    # ---- the reference's method names (rocAL_pybind/amd/rocal/pipeline.py:149-245) ----
    def get_handle(self):
        return self._handle

    def get_bounding_box_count(self):
        """rocalGetBoundingBoxCount: boxes in the whole batch."""
        return int(self.get_bounding_boxes()[2].sum())

    def get_bounding_box_cords(self):
        """rocalGetBoundingBoxCords: one float32 [count_i, 4] array (normalized ltrb) per sample."""
        b, _, c = self.get_bounding_boxes()
        ends = np.cumsum(c)
        return [b[e - k:e] for e, k in zip(ends, c)]

    def get_bounding_box_labels(self):
        """rocalGetBoundingBoxLabel: one int32 [count_i] array per sample."""
        _, lab, c = self.get_bounding_boxes()
        ends = np.cumsum(c)
        return [lab[e - k:e] for e, k in zip(ends, c)]

    def get_image_name_length(self, idx):
        """rocalGetImageNameLen: fills idx (int32 [N]) with the name lengths, returns their sum."""
        names = self.get_image_names()
        for i, nm in enumerate(names):
            idx[i] = len(nm.encode())
        return sum(len(nm.encode()) for nm in names)

    def get_image_name(self, array_len=0):
        """rocalGetImageName: the names of the batch, concatenated."""
        return "".join(self.get_image_names())

    def get_img_sizes(self, array):
        """rocalGetImageSizes into array (int32, N x 2: width, height)."""
        np.asarray(array).reshape(-1)[:2 * self._batch_size] = self.get_image_sizes().reshape(-1)
        return array

    def get_roi_img_sizes(self, array):
        """rocalGetROIImageSizes into array (int32, N x 2: width, height)."""
        np.asarray(array).reshape(-1)[:2 * self._batch_size] = self.get_roi_image_sizes().reshape(-1)
        return array

    def rocal_reset_loaders(self):
        return self.reset()

    def get_crop_windows(self, tensor):
        """[extension] n x (x, y, w, h) source window used by the crop-type operator that produced `tensor`."""
        out = np.zeros((self._batch_size, 4), dtype=np.uint32)
        self._check(C.get_crop_windows(self._handle, tensor, out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint))))
        return out

    def get_int_array(self, param):
        out = np.zeros(self._batch_size, dtype=np.int32)
        # the values the returned batch was built with; before the first run(), the parameter's current ones
        k = C.get_batch_int_array(self._handle, param, out.ctypes.data_as(ctypes.POINTER(ctypes.c_int)), self._batch_size)
        if k == 0:
            k = C.get_int_array(param, out.ctypes.data_as(ctypes.POINTER(ctypes.c_int)), self._batch_size)
        return out[:k]

    def get_float_array(self, param):
        out = np.zeros(self._batch_size, dtype=np.float32)
        k = C.get_batch_float_array(self._handle, param, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), self._batch_size)
        if k == 0:
            k = C.get_float_array(param, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), self._batch_size)
        return out[:k]

    def get_remaining_images(self):
        return C.get_remaining_images(self._handle)

    def is_empty(self):
        return self.get_remaining_images() == 0

    def timing_info(self):
        t = (ctypes.c_ulonglong * 4)()
        C.get_timing(self._handle, t)
        return {"load_time": t[0], "decode_time": t[1], "process_time": t[2], "transfer_time": t[3]}

    def h2d_bytes(self):
        """Bytes this pipeline has uploaded so far (pixels, per-sample tables, boxes); no reference counterpart."""
        return int(C.get_h2d_bytes(self._handle))

    UPLOAD_WHOLE, UPLOAD_FOOTPRINT, UPLOAD_ZERO_COPY = 0, 1, 2

    def set_upload_mode(self, mode):
        """How host-resident source pixels reach the kernels: whole images, the rectangle each image's kernels
        can read, or (default, pinned ragged input) no copy at all - the kernel reads the pinned buffer."""
        if C.set_upload_mode(self._handle, int(mode)) != 0:
            raise ValueError("upload mode must be 0, 1 or 2")

    def error_message(self):
        return C.get_error_message(self._handle).decode()

    def rocal_release(self):
        if self._handle:
            C.release(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.rocal_release()
        except Exception:
            pass

    def _check(self, status):
        if status != types.OK:
            raise RocalError(self.error_message())


def pipeline_def(fn=None, **pipeline_kwargs):
    """Decorator of amd.rocal.pipeline (pipeline.py:277-407 of the reference): turns a function that builds a graph and
    returns its outputs into a Pipeline factory.

        @pipeline_def(seed=7)
        def loader(path, crop=224): ...; return images
        pipe = loader("/data", batch_size=32, device_id=0)     # Pipeline arguments and the function's own, mixed

    Keyword arguments named like a parameter of the function go to the function, the others must be Pipeline
    constructor arguments (they override the ones given to the decorator); the function runs inside `with pipe:` and
    what it returns becomes the pipeline's outputs. The pipeline is returned unbuilt."""
    import functools
    import inspect

    def decorate(func):
        spec = inspect.getfullargspec(func)
        if spec.varkw is not None:
            raise TypeError("a graph-defining function may not take **%s" % spec.varkw)
        own = set(spec.args) | set(spec.kwonlyargs)
        ctor = set(inspect.getfullargspec(Pipeline.__init__).args) - {"self"}

        @functools.wraps(func)
        def factory(*args, **kwargs):
            fn_kwargs = {k: v for k, v in kwargs.items() if k in own}
            ctor_kwargs = dict(pipeline_kwargs)
            for k, v in kwargs.items():
                if k in own:
                    continue
                if k == "debug":
                    continue
                if k not in ctor:
                    raise TypeError("%s() got an unexpected keyword argument %r" % (func.__name__, k))
                ctor_kwargs[k] = v
            pipe = Pipeline(**ctor_kwargs)
            with pipe:
                outputs = func(*args, **fn_kwargs)
                if outputs is None:
                    outputs = ()
                elif not isinstance(outputs, tuple):
                    outputs = (outputs,)
                pipe.set_outputs(*outputs)
            return pipe

        factory._is_pipeline_def = True
        return factory

    return decorate(fn) if fn is not None else decorate

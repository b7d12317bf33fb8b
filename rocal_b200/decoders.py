"""amd.rocal.decoders (rocAL_pybind/amd/rocal/decoders.py): image decoding behind a reader."""
from . import _capi as C
from . import types
from .pipeline import Pipeline


def image(*inputs, user_feature_key_map=None, path='', file_root='', annotations_file='', index_path='', shard_id=0,
          num_shards=1, random_shuffle=False, output_type=types.RGB, decoder_type=None, device=None,
          decode_size_policy=None, max_decoded_width=1000, max_decoded_height=1000,
          last_batch_policy=types.LAST_BATCH_FILL, pad_last_batch=True, stick_to_shard=True, shard_size=-1):
    """decoders.py:31, for the folder reader: rocalJpegFileSourceSingleShard with JPEG decode on the GPU.
    max_decoded_width / max_decoded_height bound the decoded image size."""
    p = Pipeline._current_pipeline
    if p is None:
        raise RuntimeError("decoders.image must be called inside `with pipeline:`")
    reader = getattr(p, "_reader", None)
    if reader == "COCOReader":
        root = file_root or path
        h = C.coco_file_source(p._handle, str(root).encode(), str(annotations_file or p._coco_json).encode(), output_type, shard_id,
                               num_shards, 0, 1 if random_shuffle else 0, 0, max_decoded_width, max_decoded_height, last_batch_policy,
                               1 if pad_last_batch else 0, 1 if p._coco_avoid_remap else 0)
        if not h:
            raise RuntimeError(p.error_message())
        p._max_w, p._max_h = max_decoded_width, max_decoded_height
        p._has_file_source = True
        return h
    if reader != "labelReader":
        raise ValueError("decoders.image needs fn.readers.file(...) or fn.readers.coco(...) first (other readers are not implemented)")
    root = file_root or path or p._file_root
    h = C.jpeg_file_source(p._handle, str(root).encode(), output_type, shard_id, num_shards, 0, 1 if random_shuffle else 0, 0,
                           max_decoded_width, max_decoded_height, last_batch_policy, 1 if pad_last_batch else 0)
    if not h:
        raise RuntimeError(p.error_message())
    p._max_w, p._max_h = max_decoded_width, max_decoded_height
    p._has_file_source = True
    p._last_batch_policy = last_batch_policy
    return h


def _fused_crop(name, file_root, path, shard_id, num_shards, random_shuffle, random_aspect_ratio, random_area, num_attempts,
                output_type, max_decoded_width, max_decoded_height, last_batch_policy, pad_last_batch, annotations_file=''):
    import ctypes
    p = Pipeline._current_pipeline
    if p is None:
        raise RuntimeError("decoders.%s must be called inside `with pipeline:`" % name)
    reader = getattr(p, "_reader", None)
    if reader not in ("labelReader", "COCOReader"):
        raise ValueError("decoders.%s needs fn.readers.file(...) or fn.readers.coco(...) first (other readers are not implemented)" % name)
    if len(random_area) != 2 or len(random_aspect_ratio) != 2:
        raise ValueError("random_area and random_aspect_ratio take two values each")
    if reader == "COCOReader":
        # rocalJpegCOCOFileSourcePartialSingleShard: the COCO source behind the random-crop decoder; the boxes stay
        # those of the whole image
        h = image(file_root=file_root, path=path, annotations_file=annotations_file, shard_id=shard_id, num_shards=num_shards,
                  random_shuffle=random_shuffle, output_type=output_type, max_decoded_width=max_decoded_width,
                  max_decoded_height=max_decoded_height, last_batch_policy=last_batch_policy, pad_last_batch=pad_last_batch)
        p.set_random_crop_decoder(random_area, random_aspect_ratio, num_attempts)
        p._last_batch_policy = last_batch_policy
        return h
    root = file_root or path or p._file_root
    area = (ctypes.c_float * 2)(*random_area)
    aspect = (ctypes.c_float * 2)(*random_aspect_ratio)
    h = C.fused_jpeg_crop_file_source(p._handle, str(root).encode(), output_type, shard_id, num_shards, 0, area, aspect,
                                      int(num_attempts), 1 if random_shuffle else 0, 0, max_decoded_width, max_decoded_height,
                                      last_batch_policy, 1 if pad_last_batch else 0)
    if not h:
        raise RuntimeError(p.error_message())
    p._max_w, p._max_h = max_decoded_width, max_decoded_height
    p._has_file_source = True
    p._last_batch_policy = last_batch_policy
    return h


def image_slice(*inputs, file_root='', path='', annotations_file='', shard_id=0, num_shards=1, random_shuffle=False,
                random_aspect_ratio=[0.75, 1.33333], random_area=[0.08, 1.0], num_attempts=100, output_type=types.RGB,
                decode_size_policy=None, max_decoded_width=1000, max_decoded_height=1000,
                last_batch_policy=types.LAST_BATCH_FILL, pad_last_batch=True, stick_to_shard=True, shard_size=-1):
    """decoders.py:345, for the folder reader (rocalFusedJpegCropSingleShard) and the COCO reader
    (rocalJpegCOCOFileSourcePartialSingleShard): every image reaches the graph cut to
    a random-resized-crop window (the defaults are those of torchvision's RandomResizedCrop)."""
    return _fused_crop("image_slice", file_root, path, shard_id, num_shards, random_shuffle, random_aspect_ratio, random_area,
                       num_attempts, output_type, max_decoded_width, max_decoded_height, last_batch_policy, pad_last_batch,
                       annotations_file)


def image_random_crop(*inputs, user_feature_key_map=None, path='', file_root='', annotations_file='', num_shards=1, shard_id=0,
                      random_shuffle=False, num_attempts=10, output_type=types.RGB, random_area=[0.08, 1.0],
                      random_aspect_ratio=[0.8, 1.25], decode_size_policy=None, max_decoded_width=1000,
                      max_decoded_height=1000, decoder_type=None, last_batch_policy=types.LAST_BATCH_FILL, pad_last_batch=True,
                      stick_to_shard=True, shard_size=-1):
    """decoders.py:220, for the folder and COCO readers: the same fused JPEG crop source with this call's defaults."""
    return _fused_crop("image_random_crop", file_root, path, shard_id, num_shards, random_shuffle, random_aspect_ratio,
                       random_area, num_attempts, output_type, max_decoded_width, max_decoded_height, last_batch_policy,
                       pad_last_batch, annotations_file)

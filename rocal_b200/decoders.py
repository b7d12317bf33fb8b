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
    return h

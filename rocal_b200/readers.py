"""amd.rocal.readers (rocAL_pybind/amd/rocal/readers.py): the folder reader.

    jpegs, labels = fn.readers.file(file_root=path)
    images = fn.decoders.image(jpegs, file_root=path, shard_id=rank, num_shards=world, max_decoded_width=..., ...)

readers.file records the folder (one sub-folder per class, numbered in sorted order); decoders.image creates the
source. Labels of the current batch come from Pipeline.get_image_labels().
"""
from . import _capi as C
from .pipeline import Pipeline


def file(file_root, file_filters=None, file_list='', stick_to_shard=False, pad_last_batch=False, shard_id=0, num_shards=1,
         random_shuffle=False):
    """readers.py:67. Returns (reader handle, labels placeholder) like the reference. shard_id / num_shards /
    random_shuffle are accepted because scripts pass them here as well (docs/examples/image_processing/
    inference_pipeline.py:98 of the reference); the decoder call that follows is what sets them."""
    p = Pipeline._current_pipeline
    if p is None:
        raise RuntimeError("readers.file must be called inside `with pipeline:`")
    if file_list:     # "file_name label" lines; the decoder call that follows reads the listed files in this order
        C.set_file_list(p._handle, str(file_list).encode())
    p._reader = "labelReader"
    p._file_root = file_root
    return ("labelReader", file_root), []


def coco(annotations_file='', ltrb=True, masks=False, ratio=False, avoid_class_remapping=False, pixelwise_masks=False,
         is_box_encoder=False, is_box_iou_matcher=False, aspect_ratio_grouping=False, stick_to_shard=False, pad_last_batch=False):
    """readers.py:30. Records the annotation file; decoders.image(file_root=...) creates the source. Boxes are handed on as
    normalized ltrb (the reference's ratio=True); masks and aspect-ratio grouping are not supported."""
    p = Pipeline._current_pipeline
    if p is None:
        raise RuntimeError("readers.coco must be called inside `with pipeline:`")
    if masks or pixelwise_masks or aspect_ratio_grouping or not ltrb:
        raise ValueError("masks, xywh boxes and aspect-ratio grouping are not supported")
    p._reader = "COCOReader"
    p._coco_json = annotations_file
    p._coco_avoid_remap = bool(avoid_class_remapping)
    return ("COCOReader", annotations_file), [], []

"""amd.rocal.readers (rocAL_pybind/amd/rocal/readers.py): the folder reader.

    jpegs, labels = fn.readers.file(file_root=path)
    images = fn.decoders.image(jpegs, file_root=path, shard_id=rank, num_shards=world, max_decoded_width=..., ...)

readers.file records the folder (one sub-folder per class, numbered in sorted order); decoders.image creates the
source. Labels of the current batch come from Pipeline.get_image_labels().
"""
from .pipeline import Pipeline


def file(file_root, file_filters=None, file_list='', stick_to_shard=False, pad_last_batch=False):
    """readers.py:67. Returns (reader handle, labels placeholder) like the reference."""
    p = Pipeline._current_pipeline
    if p is None:
        raise RuntimeError("readers.file must be called inside `with pipeline:`")
    if file_list:
        raise ValueError("file lists are not supported")
    p._reader = "labelReader"
    p._file_root = file_root
    return ("labelReader", file_root), []

"""Framework-neutral iterators in the spirit of amd.rocal.plugin.generic (rocAL_pybind/amd/rocal/plugin/generic.py):
the batch comes back as numpy arrays on the host (device="cpu", a copy) or as CUDA torch tensors over the pipeline's
own buffers (device="gpu" / "cuda"; the reference hands out cupy arrays there)."""
import numpy as np
import torch

from .. import types


class ROCALGenericIterator(object):
    def __init__(self, pipeline, tensor_layout=None, reverse_channels=False, multiplier=None, offset=None, tensor_dtype=None,
                 display=False, device="cpu", device_id=0):
        self.loader = pipeline
        self.device = "cpu" if str(device).startswith("cpu") else "cuda"
        self.batch_size = pipeline._batch_size

    def __iter__(self):
        return self

    def _outputs(self):
        outs = [torch.from_dlpack(t) for t in self.loader.get_output_tensors()]
        return [o.cpu().numpy() for o in outs] if self.device == "cpu" else outs

    def _labels(self):
        if getattr(self.loader, "_one_hot_encoding", False):
            return self.loader.get_one_hot_encoded_labels(self.loader._num_classes)
        return np.asarray(self.loader.get_image_labels(), dtype=np.int32)

    def __next__(self):
        if self.loader.is_empty():
            raise StopIteration
        self.loader.rocal_run()
        outs, labels = self._outputs(), self._labels()
        if getattr(self.loader, "_last_batch_policy", None) == types.LAST_BATCH_PARTIAL:
            valid = self.batch_size - self.loader.get_last_batch_padded_size()
            if valid < self.batch_size:
                return [o[:valid] for o in outs], labels[:valid]
        return outs, labels

    next = __next__

    def reset(self):
        self.loader.reset()

    def __len__(self):
        return (self.loader.get_remaining_images() + self.batch_size - 1) // self.batch_size


class ROCALClassificationIterator(ROCALGenericIterator):
    """generic.py:198-246 of the reference: ([outputs...], labels) per batch of a pipeline with a file source."""

    def __init__(self, pipelines, size=0, auto_reset=False, fill_last_batch=True, dynamic_shape=False, last_batch_padded=False,
                 display=False, device="cpu", device_id=0):
        super().__init__(pipelines, display=display, device=device, device_id=device_id)
        self.auto_reset = auto_reset

    def __next__(self):
        try:
            return super().__next__()
        except StopIteration:
            if self.auto_reset:
                self.reset()
            raise

    next = __next__

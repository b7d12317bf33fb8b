"""PyTorch iterator over a built pipeline, in the spirit of amd.rocal.plugin.pytorch.ROCALGenericIterator
(rocAL_pybind/amd/rocal/plugin/pytorch.py:32-294). The reference copies every output into a fresh
torch tensor (copy_data); here outputs are handed over zero-copy through DLPack (the route the
reference's TensorFlow plugin uses, plugin/tf.py:114) and are valid until the next batch, or copied
when copy=True."""
import torch


class ROCALGenericIterator(object):
    def __init__(self, pipeline, feeder=None, copy=False, size=-1, auto_reset=False, tensor_layout=None, reverse_channels=False,
                 multiplier=None, offset=None, tensor_dtype=None, device="cuda", device_id=0, display=False,
                 fill_last_batch=True, dynamic_shape=False, last_batch_padded=False):
        """feeder(pipeline) -> bool feeds one batch through pipeline.feed_input / feed_ragged and returns
        False when the data is exhausted. The remaining arguments are those of the reference's iterators
        (plugin/pytorch.py:46, 282-290) and are accepted for source compatibility: layout, type and normalisation
        are those of the pipeline's output operators, and the tensors live on the pipeline's GPU."""
        if str(device).startswith("cpu"):
            raise ValueError("outputs live on the pipeline's GPU (device must be 'cuda' / 'gpu')")
        self.loader = pipeline
        self.feeder = feeder
        self.copy = copy
        self.auto_reset = auto_reset

    def __iter__(self):
        return self

    def _outputs(self):
        """Zero-copy views of the batch's outputs, valid until the next batch: torch.from_dlpack hands the pipeline
        the current torch stream, and the pipeline orders the reuse of these buffers behind the work queued there
        (RocalTensor.__dlpack__). Work on other streams is the caller's to order. With copy=True the views are cloned
        and the clone has finished before the tensors are returned, as the reference's synchronous copy_data."""
        outs = [torch.from_dlpack(t) for t in self.loader.get_output_tensors()]
        if self.copy:
            outs = [o.clone() for o in outs]
            torch.cuda.current_stream(outs[0].device).synchronize()
        return outs

    def __next__(self):
        if self.feeder is not None and not self.feeder(self.loader):
            if self.loader.is_empty():
                raise StopIteration
        elif self.feeder is None and self.loader.is_empty():
            raise StopIteration
        self.loader.rocal_run()
        outs = self._outputs()
        return outs

    next = __next__


class ROCALClassificationIterator(ROCALGenericIterator):
    """Yields ([outputs...], labels) for a pipeline with a file source (plugin/pytorch.py:246-294 of the reference):
    labels are an int32 CUDA tensor of the batch's class indices, or - after fn.one_hot(num_classes=k) - an int32
    [N, k] one-hot tensor filled on the device. With LAST_BATCH_PARTIAL the padding samples of the last batch are
    cut off. Iteration stops when the source is exhausted; reset() starts the next epoch."""

    def __next__(self):
        if self.loader.is_empty():
            if self.auto_reset:
                self.reset()
            raise StopIteration
        self.loader.rocal_run()
        outs = self._outputs()
        if getattr(self.loader, "_one_hot_encoding", False):
            labels = self.loader.get_one_hot_encoded_labels(self.loader._num_classes, device=outs[0].device)
        else:
            labels = torch.from_numpy(self.loader.get_image_labels()).to(outs[0].device)
        from .. import types
        if getattr(self.loader, "_last_batch_policy", None) == types.LAST_BATCH_PARTIAL:
            valid = self.loader._batch_size - self.loader.get_last_batch_padded_size()
            if valid < self.loader._batch_size:
                return [o[:valid] for o in outs], labels[:valid]
        return outs, labels

    next = __next__

    def reset(self):
        self.loader.reset()

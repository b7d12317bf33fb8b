"""PyTorch iterator over a built pipeline, in the spirit of amd.rocal.plugin.pytorch.ROCALGenericIterator
(rocAL_pybind/amd/rocal/plugin/pytorch.py:32-294). The reference copies every output into a fresh
torch tensor (copy_data); here outputs are handed over zero-copy through DLPack (the route the
reference's TensorFlow plugin uses, plugin/tf.py:114) and are valid until the next batch, or copied
when copy=True."""
import torch


class ROCALGenericIterator(object):
    def __init__(self, pipeline, feeder=None, copy=False, size=-1, auto_reset=False):
        """feeder(pipeline) -> bool feeds one batch through pipeline.feed_input / feed_ragged and returns
        False when the data is exhausted."""
        self.loader = pipeline
        self.feeder = feeder
        self.copy = copy

    def __iter__(self):
        return self

    def __next__(self):
        if self.feeder is not None and not self.feeder(self.loader):
            if self.loader.is_empty():
                raise StopIteration
        elif self.feeder is None and self.loader.is_empty():
            raise StopIteration
        self.loader.rocal_run()
        outs = [torch.from_dlpack(t) for t in self.loader.get_output_tensors()]
        if self.copy:
            outs = [o.clone() for o in outs]
        return outs

    next = __next__


class ROCALClassificationIterator(ROCALGenericIterator):
    """Yields ([outputs...], labels) for a pipeline with a file source (plugin/pytorch.py:246-294 of the reference):
    labels are an int32 CUDA tensor of the batch's class indices. Iteration stops when the source is exhausted;
    reset() starts the next epoch."""

    def __next__(self):
        if self.loader.is_empty():
            raise StopIteration
        self.loader.rocal_run()
        outs = [torch.from_dlpack(t) for t in self.loader.get_output_tensors()]
        if self.copy:
            outs = [o.clone() for o in outs]
        labels = torch.from_numpy(self.loader.get_image_labels()).to(outs[0].device)
        return outs, labels

    next = __next__

    def reset(self):
        self.loader.reset()

"""Contrib data iterators (``python/mxnet/contrib/io.py``): a ``DataIter`` view of a Gluon ``DataLoader``."""
from ..io import DataIter, DataDesc, DataBatch
from .. import ndarray as nd


class DataLoaderIter(DataIter):
    """Iterate a ``gluon.data.DataLoader`` that yields ``(data, label)`` through the ``DataIter`` protocol
    (``provide_data`` / ``provide_label``, ``reset``, padding of a short last batch)."""

    def __init__(self, loader, data_name='data', label_name='softmax_label', dtype='float32'):
        super().__init__()
        self._loader = loader
        self._iter = iter(self._loader)
        data, label = next(self._iter)
        self.batch_size = data.shape[0]
        self.dtype = dtype
        self.provide_data = [DataDesc(data_name, tuple(data.shape), dtype)]
        self.provide_label = [DataDesc(label_name, tuple(label.shape), dtype)]
        self._current_batch = None
        self.reset()

    def reset(self):
        self._iter = iter(self._loader)

    def iter_next(self):
        try:
            self._current_batch = next(self._iter)
        except StopIteration:
            self._current_batch = None
        return self._current_batch is not None

    def _padded(self, arr):
        arr = arr.astype(self.dtype)
        pad = self.getpad()
        if pad == 0:
            return arr
        shape = (self.batch_size,) + tuple(arr.shape[1:])
        out = nd.zeros(shape, dtype=self.dtype, ctx=arr.context)
        out[:arr.shape[0]] = arr
        return out

    def getdata(self):
        return [self._padded(self._current_batch[0])]

    def getlabel(self):
        return [self._padded(self._current_batch[1])]

    def getpad(self):
        return self.batch_size - self._current_batch[0].shape[0]

    def getindex(self):
        return None

    def next(self):
        if not self.iter_next():
            raise StopIteration
        return DataBatch(data=self.getdata(), label=self.getlabel(), pad=self.getpad(), index=self.getindex(),
                         provide_data=self.provide_data, provide_label=self.provide_label)

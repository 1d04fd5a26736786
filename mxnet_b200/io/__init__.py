"""``mx.io``: data iterators (``python/mxnet/io/io.py`` + native iterators of ``src/io``)."""
from .io import *        # noqa: F401,F403
from .io import DataDesc, DataBatch, DataIter, NDArrayIter, ResizeIter, PrefetchingIter, MXDataIter, CSVIter, \
    LibSVMIter, MNISTIter, ImageRecordIter, ImageRecordUInt8Iter, ImageRecordInt8Iter, ImageDetRecordIter, ImageRecordIter_v1, ImageRecordUInt8Iter_v1

"""DLPack interchange (``python/mxnet/dlpack.py``)."""
import torch

from .ndarray.ndarray import NDArray


def ndarray_to_dlpack_for_read():
    return lambda data: data.to_dlpack_for_read()


def ndarray_to_dlpack_for_write():
    return lambda data: data.to_dlpack_for_write()


def ndarray_from_dlpack(array_cls=NDArray):
    def from_dlpack(dlpack):
        return array_cls._from_tensor(torch.utils.dlpack.from_dlpack(dlpack))
    return from_dlpack


def ndarray_from_numpy(array_cls, array_create_func):
    def from_numpy(ndarray, zero_copy=True):
        t = torch.from_numpy(ndarray if zero_copy else ndarray.copy())
        return array_cls._from_tensor(t)
    return from_numpy

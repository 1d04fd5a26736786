"""Batchify functions (``python/mxnet/gluon/data/batchify.py``; native ``src/io/batchify.cc``)."""
import numpy as np

from ...ndarray.ndarray import NDArray
from ...util import is_np_array

__all__ = ['Stack', 'Pad', 'Group', 'Append', 'AsList']


def _wrap(arr, dtype=None):
    if is_np_array():
        from ... import numpy as mnp
        return mnp.array(arr, dtype=dtype or arr.dtype)
    from ... import ndarray as nd
    return nd.array(arr, dtype=dtype or arr.dtype)


def _to_np(x):
    return x.asnumpy() if isinstance(x, NDArray) else np.asarray(x)


class Stack(object):
    def __init__(self, use_shared_mem=False):
        self._use_shared_mem = use_shared_mem

    def __call__(self, data):
        if isinstance(data[0], NDArray):
            import torch
            return data[0].__class__._from_tensor(torch.stack([d._data for d in data], 0), data[0].context)
        if isinstance(data[0], (tuple, list)):
            return [self(list(i)) for i in zip(*data)]
        out = np.asarray(data)
        return _wrap(out, out.dtype if out.dtype != np.float64 else np.float32)


class Pad(object):
    def __init__(self, val=0, dtype=None, round_to=None, use_shared_mem=False, axis=0, pad_val=None, ret_length=False):
        self._pad_val = pad_val if pad_val is not None else val
        self._dtype, self._round_to, self._axis, self._ret_length = dtype, round_to, axis, ret_length

    def __call__(self, data):
        arrs = [_to_np(d) for d in data]
        if arrs[0].ndim == 0:
            out = np.asarray(arrs)
            return _wrap(out, self._dtype)
        ax = self._axis
        lens = [a.shape[ax] for a in arrs]
        max_len = max(lens)
        if self._round_to:
            max_len = (max_len + self._round_to - 1) // self._round_to * self._round_to
        shape = list(arrs[0].shape)
        shape[ax] = max_len
        out = np.full([len(arrs)] + shape, self._pad_val, dtype=self._dtype or arrs[0].dtype)
        for i, a in enumerate(arrs):
            sl = [slice(None)] * a.ndim
            sl[ax] = slice(0, a.shape[ax])
            out[(i,) + tuple(sl)] = a
        res = _wrap(out, out.dtype if out.dtype != np.float64 else np.float32)
        if self._ret_length:
            return res, _wrap(np.asarray(lens, dtype=np.int32))
        return res


class Group(object):
    def __init__(self, fn, *args):
        if isinstance(fn, (list, tuple)):
            assert len(args) == 0
            self._fn = fn
        else:
            self._fn = (fn,) + args
        for i, f in enumerate(self._fn):
            assert hasattr(f, '__call__'), 'Batchify functions must be callable! type(fn[%d]) = %s' % (i, str(type(f)))

    def __call__(self, data):
        assert len(data[0]) == len(self._fn), 'The number of attributes in each data sample should contains {} ' \
            'elements'.format(len(self._fn))
        ret = []
        for i, f in enumerate(self._fn):
            ret.append(f([ele[i] for ele in data]))
        return tuple(ret)


class Append(object):
    def __init__(self, expand=True, batch_axis=0, use_shared_mem=False):
        self._expand, self._batch_axis = expand, batch_axis

    def __call__(self, data):
        out = []
        for d in data:
            a = _to_np(d)
            if self._expand:
                a = np.expand_dims(a, self._batch_axis)
            out.append(_wrap(a, a.dtype if a.dtype != np.float64 else np.float32))
        return out


class AsList(object):
    def __call__(self, data):
        return list(data)


def default_batchify_fn(data):
    return Stack()(data)

"""Datasets (``python/mxnet/gluon/data/dataset.py``)."""
import os

import numpy as np

from ...ndarray.ndarray import NDArray

__all__ = ['Dataset', 'SimpleDataset', 'ArrayDataset', 'RecordFileDataset']


class Dataset(object):
    def __getitem__(self, idx):
        raise NotImplementedError

    def __len__(self):
        raise NotImplementedError

    def filter(self, fn):
        return SimpleDataset([self[i] for i in range(len(self)) if fn(self[i])])

    def shard(self, num_shards, index):
        assert index < num_shards, 'Shard index of out bound: %d out of %d' % (index, num_shards)
        assert num_shards > 0 and index >= 0
        length = len(self)
        shard_len = length // num_shards
        rest = length % num_shards
        start = shard_len * index + min(index, rest)
        end = start + shard_len + (index < rest)
        return _SampledDataset(self, list(range(start, end)))

    def take(self, count):
        if count is None or count > len(self):
            count = len(self)
        return _SampledDataset(self, list(range(count)))

    def sample(self, sampler):
        from .sampler import Sampler
        if not isinstance(sampler, Sampler):
            raise TypeError('Invalid sampler type: {}. Expected gluon.data.Sampler instead.'.format(type(sampler)))
        return _SampledDataset(self, list(sampler))

    def transform(self, fn, lazy=True):
        trans = _LazyTransformDataset(self, fn)
        if lazy:
            return trans
        return SimpleDataset([i for i in trans])

    def transform_first(self, fn, lazy=True):
        return self.transform(_TransformFirstClosure(fn), lazy)


class SimpleDataset(Dataset):
    def __init__(self, data):
        self._data = data

    def __len__(self):
        return len(self._data)

    def __getitem__(self, idx):
        return self._data[idx]


class _SampledDataset(Dataset):
    def __init__(self, dataset, indices):
        self._dataset, self._indices = dataset, indices

    def __len__(self):
        return len(self._indices)

    def __getitem__(self, idx):
        return self._dataset[self._indices[idx]]


class _LazyTransformDataset(Dataset):
    def __init__(self, data, fn):
        self._data, self._fn = data, fn

    def __len__(self):
        return len(self._data)

    def __getitem__(self, idx):
        item = self._data[idx]
        if isinstance(item, tuple):
            return self._fn(*item)
        return self._fn(item)


class _TransformFirstClosure(object):
    def __init__(self, fn):
        self._fn = fn

    def __call__(self, x, *args):
        if args:
            return (self._fn(x),) + args
        return self._fn(x)


class ArrayDataset(Dataset):
    def __init__(self, *args):
        assert len(args) > 0, 'Needs at least 1 arrays'
        self._length = len(args[0])
        self._data = []
        for i, data in enumerate(args):
            assert len(data) == self._length, 'All arrays must have the same length; array[0] has length %d while ' \
                'array[%d] has %d.' % (self._length, i + 1, len(data))
            if isinstance(data, NDArray) and len(data.shape) == 1:
                data = data.asnumpy()
            self._data.append(data)

    def __getitem__(self, idx):
        if len(self._data) == 1:
            return self._data[0][idx]
        return tuple(data[idx] for data in self._data)

    def __len__(self):
        return self._length


class RecordFileDataset(Dataset):
    """Dataset over an indexed RecordIO file (``.rec`` + ``.idx``); items are raw record bytes."""

    def __init__(self, filename):
        from ... import recordio
        self.idx_file = os.path.splitext(filename)[0] + '.idx'
        self.filename = filename
        self._record = recordio.MXIndexedRecordIO(self.idx_file, self.filename, 'r')

    def __getitem__(self, idx):
        return self._record.read_idx(self._record.keys[idx])

    def __len__(self):
        return len(self._record.keys)

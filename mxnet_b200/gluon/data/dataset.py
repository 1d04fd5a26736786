"""Random-access datasets and their derived views (API of ``python/mxnet/gluon/data/dataset.py``: ``Dataset`` with
``filter / shard / take / sample / transform / transform_first``, ``SimpleDataset``, ``ArrayDataset``,
``RecordFileDataset``).

Every derived dataset is a view: it keeps the parent and either a list of parent positions (``_IndexView``) or a
function applied on access (``_MappedView``); nothing is copied until ``transform(..., lazy=False)`` or ``filter``
asks for it.
"""
import os

from ...ndarray.ndarray import NDArray

__all__ = ['Dataset', 'SimpleDataset', 'ArrayDataset', 'RecordFileDataset']


class Dataset(object):
    """Anything with ``__getitem__(int)`` and ``__len__``."""

    def __getitem__(self, idx):
        raise NotImplementedError

    def __len__(self):
        raise NotImplementedError

    # ---- selections ---------------------------------------------------------------------------------------
    def filter(self, fn):
        """The items for which ``fn(item)`` holds (evaluated now, each item read once)."""
        kept = []
        for i in range(len(self)):
            item = self[i]
            if fn(item):
                kept.append(item)
        return SimpleDataset(kept)

    def shard(self, num_shards, index):
        """Contiguous part ``index`` of ``num_shards`` parts whose sizes differ by at most one (the first
        ``len % num_shards`` parts are the longer ones)."""
        if not (num_shards > 0 and 0 <= index < num_shards):
            raise AssertionError('Shard index of out bound: %d out of %d' % (index, num_shards))
        base, extra = divmod(len(self), num_shards)
        begin = index * base + min(index, extra)
        return _IndexView(self, range(begin, begin + base + (1 if index < extra else 0)))

    def take(self, count):
        """The first ``count`` items (all of them for ``None`` or a count beyond the end)."""
        n = len(self)
        return _IndexView(self, range(n if count is None else min(count, n)))

    def sample(self, sampler):
        """The items at the positions a ``Sampler`` yields, in that order."""
        from .sampler import Sampler
        if not isinstance(sampler, Sampler):
            raise TypeError('Invalid sampler type: {}. Expected gluon.data.Sampler instead.'.format(type(sampler)))
        return _IndexView(self, list(sampler))

    # ---- transformations ----------------------------------------------------------------------------------
    def transform(self, fn, lazy=True):
        """``fn(*item)`` for tuple items, ``fn(item)`` otherwise; on access, or right away with ``lazy=False``."""
        view = _MappedView(self, fn)
        return view if lazy else SimpleDataset([view[i] for i in range(len(view))])

    def transform_first(self, fn, lazy=True):
        """Apply ``fn`` to the first element of each item only (the image of an ``(image, label)`` pair)."""
        return self.transform(_OnFirst(fn), lazy)


class SimpleDataset(Dataset):
    """A list (or any indexable) as a dataset."""

    def __init__(self, data):
        self._data = data

    def __getitem__(self, idx):
        return self._data[idx]

    def __len__(self):
        return len(self._data)


class _IndexView(Dataset):
    """Items of ``parent`` at ``positions`` (a range or a list)."""

    def __init__(self, parent, positions):
        self._parent = parent
        self._positions = positions

    def __getitem__(self, idx):
        return self._parent[self._positions[idx]]

    def __len__(self):
        return len(self._positions)


class _MappedView(Dataset):
    def __init__(self, parent, fn):
        self._parent = parent
        self._fn = fn

    def __getitem__(self, idx):
        item = self._parent[idx]
        return self._fn(*item) if isinstance(item, tuple) else self._fn(item)

    def __len__(self):
        return len(self._parent)


class _OnFirst(object):
    """Picklable ``(first, *rest) -> (fn(first), *rest)`` (worker processes receive it by pickle)."""

    def __init__(self, fn):
        self._fn = fn

    def __call__(self, first, *rest):
        out = self._fn(first)
        return (out,) + rest if rest else out


class ArrayDataset(Dataset):
    """Several equally long arrays (or lists, or datasets) zipped: item ``i`` is the tuple of their ``i``-th entries, or
    the entry itself when there is only one array."""

    def __init__(self, *args):
        if not args:
            raise AssertionError('Needs at least 1 arrays')
        self._length = len(args[0])
        self._data = []
        for pos, column in enumerate(args):
            if len(column) != self._length:
                raise AssertionError('All arrays must have the same length; array[0] has length %d while array[%d] has %d.'
                                     % (self._length, pos + 1, len(column)))
            if isinstance(column, NDArray) and column.ndim == 1:
                column = column.asnumpy()      # scalar labels: plain numbers instead of one device array per item
            self._data.append(column)

    def __getitem__(self, idx):
        row = tuple(column[idx] for column in self._data)
        return row[0] if len(row) == 1 else row

    def __len__(self):
        return self._length


class RecordFileDataset(Dataset):
    """An indexed RecordIO file (``name.rec`` with ``name.idx`` beside it); items are the raw record bytes."""

    def __init__(self, filename):
        from ... import recordio
        self.filename = filename
        self.idx_file = os.path.splitext(filename)[0] + '.idx'
        self._record = recordio.MXIndexedRecordIO(self.idx_file, self.filename, 'r')

    def __getitem__(self, idx):
        return self._record.read_idx(self._record.keys[idx])

    def __len__(self):
        return len(self._record.keys)

"""Index samplers (API of ``python/mxnet/gluon/data/sampler.py``): iterables over dataset positions, and
``BatchSampler`` which groups another sampler's positions into lists."""
import itertools

import numpy as np

__all__ = ['Sampler', 'SequentialSampler', 'RandomSampler', 'BatchSampler', 'IntervalSampler', 'FilterSampler']

_LAST_BATCH = ('keep', 'discard', 'rollover')


class Sampler(object):
    def __iter__(self):
        raise NotImplementedError

    def __len__(self):
        raise NotImplementedError


class _FixedLength(Sampler):
    """Samplers over a known number of positions: subclasses give ``_positions()``."""

    _length = 0

    def _positions(self):
        raise NotImplementedError

    def __iter__(self):
        return iter(self._positions())

    def __len__(self):
        return self._length


class SequentialSampler(_FixedLength):
    """``start, start + 1, ..., start + length - 1``."""

    def __init__(self, length, start=0):
        self._length, self._start = length, start

    def _positions(self):
        return range(self._start, self._start + self._length)


class RandomSampler(_FixedLength):
    """A fresh permutation of ``range(length)`` per pass (drawn from NumPy's global generator, so ``mx.random.seed`` /
    ``np.random.seed`` make it repeatable)."""

    def __init__(self, length):
        self._length = length

    def _positions(self):
        return np.random.permutation(self._length).tolist()


class FilterSampler(_FixedLength):
    """Positions of the items for which ``fn(item)`` holds (evaluated once, at construction)."""

    def __init__(self, fn, dataset):
        self._fn, self._dataset = fn, dataset
        self._indices = [pos for pos, item in enumerate(dataset) if fn(item)]
        self._length = len(self._indices)

    def _positions(self):
        return self._indices


class IntervalSampler(Sampler):
    """``0, k, 2k, ...`` and, with ``rollover``, then ``1, k + 1, ...`` and so on until every position was visited."""

    def __init__(self, length, interval, rollover=True):
        if interval >= length:
            raise AssertionError('Interval {} must be smaller than length {}'.format(interval, length))
        self._length = length
        self._interval = interval
        self._rollover = rollover

    def _passes(self):
        starts = range(self._interval) if self._rollover else range(1)
        return [range(s, self._length, self._interval) for s in starts]

    def __iter__(self):
        return itertools.chain.from_iterable(self._passes())

    def __len__(self):
        return sum(len(r) for r in self._passes())


class BatchSampler(Sampler):
    """Lists of ``batch_size`` positions from ``sampler``.  A short last batch is kept, discarded, or (``rollover``)
    carried over to the front of the next pass."""

    def __init__(self, sampler, batch_size, last_batch='keep'):
        self._sampler = sampler
        self._batch_size = batch_size
        self._last_batch = last_batch
        self._prev = []

    def _check_mode(self):
        if self._last_batch not in _LAST_BATCH:
            raise ValueError("last_batch must be one of 'keep', 'discard', or 'rollover', but got %s" % self._last_batch)

    def __iter__(self):
        carried, self._prev = self._prev, []
        stream = itertools.chain(carried, self._sampler)
        while True:
            batch = list(itertools.islice(stream, self._batch_size))
            if len(batch) == self._batch_size:
                yield batch
                continue
            if batch:
                self._check_mode()
                if self._last_batch == 'keep':
                    yield batch
                elif self._last_batch == 'rollover':
                    self._prev = batch
            return

    def __len__(self):
        self._check_mode()
        n, b = len(self._sampler), self._batch_size
        if self._last_batch == 'keep':
            return -(-n // b)
        if self._last_batch == 'discard':
            return n // b
        return (n + len(self._prev)) // b

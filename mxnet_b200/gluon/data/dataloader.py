"""DataLoader (``python/mxnet/gluon/data/dataloader.py``): batches a Dataset with worker processes or
threads, optional pinned-memory staging and prefetching.

Worker processes put the arrays of a batch into POSIX shared-memory segments of the native storage
manager (``csrc/storage.cc``) and send only the segment names; the parent maps the segments and wraps
them without another copy (the reference rebuilds NDArrays over ``cpu_shared`` storage,
``dataloader.py:47-95``).  With ``pin_memory`` the batch is staged in page-locked buffers from the
native pinned pool, so the host→device copy runs on the copy-in stream and overlaps compute."""
import atexit
import ctypes
import glob
import itertools
import multiprocessing
import os
import pickle
import threading
import weakref
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import torch

from ...ndarray.ndarray import NDArray
from ...util import is_np_array
from . import sampler as _sampler
from .batchify import default_batchify_fn

__all__ = ['DataLoader']


shm_batches = 0          # arrays received through shared-memory segments (observable by tests)
_segment_counter = itertools.count()


def _rt():
    from ...csrc import runtime
    return runtime.lib()


def _segment_prefix(owner_pid):
    return '/mxb_dl_%d_' % owner_pid


def _to_shared(a, owner_pid):
    """Copy a NumPy array into a fresh shared segment named after the process that will own it; returns what the owner
    needs to map it.  The creating process unmaps without dropping the reference: the owner adopts it."""
    a = np.ascontiguousarray(a)
    name = '%s%d_%d' % (_segment_prefix(owner_pid), os.getpid(), next(_segment_counter))
    L = _rt()
    ptr = L.mxb_shm_open(name.encode(), max(a.nbytes, 1), 1, None)
    if not ptr:
        return None
    if a.nbytes:
        ctypes.memmove(ptr, a.ctypes.data, a.nbytes)
    L.mxb_shm_detach(ctypes.c_void_p(ptr))
    return name, a.shape, a.dtype.str


def _from_shared(name, shape, dtype):
    """Map a segment created by a worker; the returned array views the mapping, which is released (and the name
    unlinked) when the array's buffer is collected."""
    global shm_batches
    L = _rt()
    size = ctypes.c_uint64(0)
    ptr = L.mxb_shm_adopt(name.encode(), ctypes.byref(size))
    if not ptr:
        raise RuntimeError('shared-memory segment %s of a data-loader worker is gone' % name)
    nbytes = int(np.prod(shape, dtype=np.int64)) * np.dtype(dtype).itemsize
    raw = (ctypes.c_uint8 * max(nbytes, 1)).from_address(ptr)
    weakref.finalize(raw, L.mxb_shm_close, name.encode(), ctypes.c_void_p(ptr))
    shm_batches += 1
    return np.frombuffer(raw, dtype=np.dtype(dtype), count=int(np.prod(shape, dtype=np.int64))).reshape(shape)


def _cleanup_segments():
    """Segments addressed to this process that were never adopted (a worker finished after the iterator was dropped)."""
    for path in glob.glob('/dev/shm' + _segment_prefix(os.getpid()) + '*'):
        try:
            os.unlink(path)
        except OSError:
            pass


atexit.register(_cleanup_segments)


def _to_numpy_tree(batch, owner_pid=None):
    """A batch as a picklable tree; with ``owner_pid`` the arrays travel as shared-memory segments for that process."""
    if isinstance(batch, NDArray):
        a = batch.asnumpy()
        shared = _to_shared(a, owner_pid) if owner_pid is not None and a.nbytes >= 1024 else None
        if shared is not None:
            return ('shm', shared, str(batch._data.dtype))
        return ('nd', a, str(batch._data.dtype))
    if isinstance(batch, (list, tuple)):
        return ('seq', [_to_numpy_tree(b, owner_pid) for b in batch], isinstance(batch, tuple))
    return ('raw', batch, None)


def _from_numpy_tree(tree, pin_memory=False):
    kind, val, extra = tree
    if kind in ('nd', 'shm'):
        t = torch.from_numpy(_from_shared(*val) if kind == 'shm' else val)
        if extra == 'torch.bfloat16':
            t = t.to(torch.bfloat16)
        if pin_memory and torch.cuda.is_available():
            from ... import engine
            t = engine.pinned_like(t)          # pooled page-locked staging buffer; the shared segment is released
        if is_np_array():
            from ...numpy.multiarray import ndarray
            return ndarray._from_tensor(t)
        return NDArray._from_tensor(t)
    if kind == 'seq':
        items = [_from_numpy_tree(b, pin_memory) for b in val]
        return tuple(items) if extra else items
    return val


_worker_dataset = None


def _worker_initializer(dataset):
    """Runs once in every forked worker.  Workers build their batches on the host whatever default device the parent
    had when it forked (the reference's workers always batchify into CPU shared memory,
    ``python/mxnet/gluon/data/dataloader.py``); a forked process cannot use the parent's CUDA context anyway."""
    global _worker_dataset
    _worker_dataset = dataset
    torch.set_num_threads(1)
    from ...device import Device
    Device._default.stack = []
    Device._process_default = Device('cpu', 0)


def _worker_fn(samples, batchify_fn, dataset=None):
    global _worker_dataset
    ds = dataset if dataset is not None else _worker_dataset
    batch = batchify_fn([ds[i] for i in samples])
    return pickle.dumps(_to_numpy_tree(batch, os.getppid()), pickle.HIGHEST_PROTOCOL)


def _thread_worker_fn(samples, batchify_fn, dataset):
    return batchify_fn([dataset[i] for i in samples])


class _MultiWorkerIter(object):
    def __init__(self, pool, batchify_fn, batch_sampler, pin_memory, prefetch, dataset, thread_pool, timeout):
        self._pool, self._batchify_fn, self._batch_sampler = pool, batchify_fn, batch_sampler
        self._pin_memory, self._dataset, self._thread_pool, self._timeout = pin_memory, dataset, thread_pool, timeout
        self._data_buffer = {}
        self._rcvd_idx = self._sent_idx = 0
        self._iter = iter(self._batch_sampler)
        for _ in range(prefetch):
            self._push_next()

    def __len__(self):
        return len(self._batch_sampler)

    def _push_next(self):
        r = next(self._iter, None)
        if r is None:
            return
        if self._thread_pool:
            fut = self._pool.submit(_thread_worker_fn, r, self._batchify_fn, self._dataset)
        else:
            fut = self._pool.apply_async(_worker_fn, (r, self._batchify_fn))
        self._data_buffer[self._sent_idx] = fut
        self._sent_idx += 1

    def __next__(self):
        self._push_next()
        if self._rcvd_idx == self._sent_idx:
            assert not self._data_buffer, 'Data buffer should be empty at this moment'
            raise StopIteration
        assert self._rcvd_idx < self._sent_idx, 'rcvd_idx must be smaller than sent_idx'
        assert self._rcvd_idx in self._data_buffer, 'fatal error with _push_next, rcvd_idx missing'
        ret = self._data_buffer.pop(self._rcvd_idx)
        try:
            if self._thread_pool:
                batch = ret.result(timeout=self._timeout)
                if self._pin_memory:
                    batch = _from_numpy_tree(_to_numpy_tree(batch), True)
            else:
                batch = _from_numpy_tree(pickle.loads(ret.get(self._timeout)), self._pin_memory)
            self._rcvd_idx += 1
            return batch
        except multiprocessing.context.TimeoutError:
            msg = 'Worker timed out after {} seconds. This might be caused by \n - Slow transform. Please increase ' \
                  'timeout to allow slower data loading in each worker.\n - Insufficient shared_memory if ' \
                  '`timeout` is large enough.'.format(self._timeout)
            raise RuntimeError(msg)

    next = __next__

    def __iter__(self):
        return self


class DataLoader(object):
    def __init__(self, dataset, batch_size=None, shuffle=False, sampler=None, last_batch=None, batch_sampler=None,
                 batchify_fn=None, num_workers=0, pin_memory=False, pin_device_id=0, prefetch=None, thread_pool=False,
                 timeout=120, try_nopython=None):
        self._dataset, self._pin_memory, self._pin_device_id = dataset, pin_memory, pin_device_id
        self._thread_pool, self._timeout = thread_pool, timeout
        assert timeout > 0, 'timeout must be positive, given {}'.format(timeout)
        if batch_sampler is None:
            if batch_size is None:
                raise ValueError('batch_size must be specified unless batch_sampler is specified')
            if sampler is None:
                sampler = _sampler.RandomSampler(len(dataset)) if shuffle else _sampler.SequentialSampler(len(dataset))
            elif shuffle:
                raise ValueError('shuffle must not be specified if sampler is specified')
            batch_sampler = _sampler.BatchSampler(sampler, batch_size, last_batch if last_batch else 'keep')
        elif batch_size is not None or shuffle or sampler is not None or last_batch is not None:
            raise ValueError('batch_size, shuffle, sampler and last_batch must not be specified if batch_sampler '
                             'is specified.')
        self._batch_sampler = batch_sampler
        self._num_workers = num_workers if num_workers >= 0 else 0
        self._worker_pool = None
        self._prefetch = max(0, int(prefetch) if prefetch is not None else 2 * self._num_workers)
        if self._num_workers > 0:
            if self._thread_pool:
                self._worker_pool = ThreadPoolExecutor(self._num_workers)
            else:
                ctx = multiprocessing.get_context('fork')
                self._worker_pool = ctx.Pool(self._num_workers, initializer=_worker_initializer, initargs=[self._dataset])
        self._batchify_fn = batchify_fn if batchify_fn is not None else default_batchify_fn

    def __iter__(self):
        if self._num_workers == 0:
            def same_process_iter():
                for batch in self._batch_sampler:
                    ret = self._batchify_fn([self._dataset[idx] for idx in batch])
                    if self._pin_memory:
                        ret = _from_numpy_tree(_to_numpy_tree(ret), True)
                    yield ret
            return same_process_iter()
        return _MultiWorkerIter(self._worker_pool, self._batchify_fn, self._batch_sampler, self._pin_memory,
                                self._prefetch, self._dataset, self._thread_pool, self._timeout)

    def __len__(self):
        return len(self._batch_sampler)

    def __del__(self):
        if self._worker_pool is not None:
            try:
                if self._thread_pool:
                    self._worker_pool.shutdown(wait=False)
                else:
                    self._worker_pool.terminate()
            except Exception:  # pylint: disable=broad-except
                pass


def default_mp_batchify_fn(data):
    """Batchify used inside worker processes.  The reference stacks into CPU shared memory there; workers here already
    build their batches on the host and hand them over through pickled shared buffers, so this is the default function."""
    return default_batchify_fn(data)


DataLoaderV1 = DataLoader          # the first-generation loader of the reference had the same interface

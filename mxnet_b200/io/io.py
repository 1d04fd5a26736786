"""Data iterators.

Python iterators (``DataIter``, ``NDArrayIter``, ``ResizeIter``, ``PrefetchingIter``) follow
``python/mxnet/io/io.py``.  The iterators the reference implements natively (``CSVIter``,
``LibSVMIter``, ``MNISTIter``, ``ImageRecordIter`` and variants, ``src/io/*.cc``) use the native
parsers / RecordIO prefetcher of ``csrc/recordio.cc``; JPEG decoding and augmentation run on a pool
of host threads while the reader thread keeps the record queue full.
"""
import ctypes
import gzip
import os
import struct
import threading
from collections import namedtuple
from concurrent.futures import ThreadPoolExecutor

import numpy as np

from ..base import MXNetError
from ..ndarray.ndarray import NDArray

__all__ = ['DataDesc', 'DataBatch', 'DataIter', 'NDArrayIter', 'ResizeIter', 'PrefetchingIter', 'MXDataIter',
           'CSVIter', 'LibSVMIter', 'MNISTIter', 'ImageRecordIter', 'ImageRecordUInt8Iter', 'ImageRecordInt8Iter',
           'ImageDetRecordIter', 'ImageRecordIter_v1', 'ImageRecordUInt8Iter_v1']


class DataDesc(namedtuple('DataDesc', ['name', 'shape'])):
    def __new__(cls, name, shape, dtype=np.float32, layout='NCHW'):
        ret = super(cls, DataDesc).__new__(cls, name, shape)
        ret.dtype, ret.layout = dtype, layout
        return ret

    def __repr__(self):
        return 'DataDesc[%s,%s,%s,%s]' % (self.name, self.shape, self.dtype, self.layout)

    @staticmethod
    def get_batch_axis(layout):
        if layout is None:
            return 0
        return layout.find('N')

    @staticmethod
    def get_list(shapes, types):
        if types is not None:
            type_dict = dict(types)
            return [DataDesc(x[0], x[1], type_dict[x[0]]) for x in shapes]
        return [DataDesc(x[0], x[1]) for x in shapes]


class DataBatch(object):
    def __init__(self, data, label=None, pad=None, index=None, bucket_key=None, provide_data=None, provide_label=None):
        if data is not None:
            assert isinstance(data, (list, tuple)), 'Data must be list of NDArrays'
        if label is not None:
            assert isinstance(label, (list, tuple)), 'Label must be list of NDArrays'
        self.data, self.label, self.pad, self.index = data, label, pad, index
        self.bucket_key, self.provide_data, self.provide_label = bucket_key, provide_data, provide_label

    def __str__(self):
        data_shapes = [d.shape for d in self.data]
        label_shapes = [l.shape for l in self.label] if self.label else None
        return '{}: data shapes: {} label shapes: {}'.format(self.__class__.__name__, data_shapes, label_shapes)


class DataIter(object):
    def __init__(self, batch_size=0):
        self.batch_size = batch_size

    def __iter__(self):
        return self

    def reset(self):
        pass

    def next(self):
        if self.iter_next():
            return DataBatch(data=self.getdata(), label=self.getlabel(), pad=self.getpad(), index=self.getindex())
        raise StopIteration

    def __next__(self):
        return self.next()

    def iter_next(self):
        pass

    def getdata(self):
        pass

    def getlabel(self):
        pass

    def getindex(self):
        return None

    def getpad(self):
        pass


def _init_data(data, allow_empty, default_name):
    from .. import ndarray as nd
    assert (data is not None) or allow_empty
    if data is None:
        data = []
    if isinstance(data, (np.ndarray, NDArray)):
        data = [data]
    if isinstance(data, list):
        if not allow_empty:
            assert len(data) > 0
        if len(data) == 1:
            data = {default_name: data[0]}
        else:
            data = {'_%d_%s' % (i, default_name): d for i, d in enumerate(data)}
    if not isinstance(data, dict):
        raise TypeError('Input must be NDArray, numpy.ndarray, a list of them or dict with them as values')
    out = []
    for k, v in data.items():
        if not isinstance(v, NDArray):
            try:
                v = nd.array(v, dtype=v.dtype if hasattr(v, 'dtype') and v.dtype != np.float64 else None)
            except Exception:
                raise TypeError(('Invalid type \'%s\' for %s, ' % (type(v), k)) + 'should be NDArray or numpy.ndarray')
        out.append((k, v))
    return out


class NDArrayIter(DataIter):
    """Iterate over in-memory arrays with ``pad`` / ``discard`` / ``roll_over`` last-batch handling."""

    def __init__(self, data, label=None, batch_size=1, shuffle=False, last_batch_handle='pad', data_name='data',
                 label_name='softmax_label'):
        super().__init__(batch_size)
        self.data = _init_data(data, allow_empty=False, default_name=data_name)
        self.label = _init_data(label, allow_empty=True, default_name=label_name)
        self.num_data = self.data[0][1].shape[0]
        assert self.num_data >= batch_size or last_batch_handle != 'discard' or True
        self.idx = np.arange(self.num_data)
        self.shuffle, self.last_batch_handle = shuffle, last_batch_handle
        self.cursor = -batch_size
        self._cache_data = self._cache_label = None
        self.reset()

    @property
    def provide_data(self):
        return [DataDesc(k, tuple([self.batch_size] + list(v.shape[1:])), v.dtype) for k, v in self.data]

    @property
    def provide_label(self):
        return [DataDesc(k, tuple([self.batch_size] + list(v.shape[1:])), v.dtype) for k, v in self.label]

    def hard_reset(self):
        if self.shuffle:
            np.random.shuffle(self.idx)
        self.cursor = -self.batch_size
        self._cache_data = self._cache_label = None

    def reset(self):
        if self.shuffle:
            np.random.shuffle(self.idx)
        if self.last_batch_handle == 'roll_over' and 0 < self.cursor < self.num_data + self.batch_size and \
                self.cursor > self.num_data:
            self.cursor = self.cursor - self.num_data - self.batch_size
        elif self.last_batch_handle == 'roll_over' and self.num_data - self.batch_size < self.cursor < self.num_data:
            self.cursor = self.cursor - self.num_data - self.batch_size
        else:
            self.cursor = -self.batch_size

    def iter_next(self):
        self.cursor += self.batch_size
        return self.cursor < self.num_data

    def next(self):
        if not self.iter_next():
            raise StopIteration
        data, label = self.getdata(), self.getlabel()
        if data[0].shape[0] != self.batch_size:
            if self.last_batch_handle == 'discard':
                raise StopIteration
            if self.last_batch_handle == 'roll_over':
                self._cache_data, self._cache_label = data, label
                raise StopIteration
        return DataBatch(data=data, label=label, pad=self.getpad(), index=None)

    def _take(self, arrays, start, end):
        import torch
        sel = torch.as_tensor(self.idx[start:end])
        return [v.__class__._from_tensor(v._data[sel.to(v._data.device)], v.context) for _, v in arrays]

    def _concat(self, first, second):
        import torch
        return [a.__class__._from_tensor(torch.cat([a._data, b._data], 0), a.context) for a, b in zip(first, second)]

    def _batchify(self, source):
        if not source:
            return []
        if self.cursor + self.batch_size <= self.num_data or self.last_batch_handle != 'pad':
            if self.last_batch_handle == 'roll_over' and self.cursor < 0:
                cache = self._cache_data if source is self.data else self._cache_label
                rest = self._take(source, 0, self.cursor + self.batch_size)
                return self._concat(cache, rest) if cache is not None else rest
            return self._take(source, self.cursor, min(self.cursor + self.batch_size, self.num_data))
        pad = self.batch_size - self.num_data + self.cursor
        return self._concat(self._take(source, self.cursor, self.num_data), self._take(source, 0, pad))

    def getdata(self):
        return self._batchify(self.data)

    def getlabel(self):
        return self._batchify(self.label)

    def getpad(self):
        if self.last_batch_handle == 'pad' and self.cursor + self.batch_size > self.num_data:
            return self.cursor + self.batch_size - self.num_data
        if self.last_batch_handle == 'roll_over' and -self.batch_size < self.cursor < 0:
            return -self.cursor
        return 0


class ResizeIter(DataIter):
    def __init__(self, data_iter, size, reset_internal=True):
        super().__init__()
        self.data_iter, self.size, self.reset_internal = data_iter, size, reset_internal
        self.cur = 0
        self.current_batch = None
        self.provide_data, self.provide_label = data_iter.provide_data, data_iter.provide_label
        self.batch_size = data_iter.batch_size
        if hasattr(data_iter, 'default_bucket_key'):
            self.default_bucket_key = data_iter.default_bucket_key

    def reset(self):
        self.cur = 0
        if self.reset_internal:
            self.data_iter.reset()

    def iter_next(self):
        if self.cur == self.size:
            return False
        try:
            self.current_batch = self.data_iter.next()
        except StopIteration:
            self.data_iter.reset()
            self.current_batch = self.data_iter.next()
        self.cur += 1
        return True

    def getdata(self): return self.current_batch.data
    def getlabel(self): return self.current_batch.label
    def getindex(self): return self.current_batch.index
    def getpad(self): return self.current_batch.pad


class PrefetchingIter(DataIter):
    """Fetches the next batch of one or several iterators ahead of time as tasks of the host engine (one engine
    variable per iterator serialises its fetches); ``next`` waits for those variables, so a failure inside an
    underlying iterator is raised by ``next`` instead of being lost on a background thread."""

    def __init__(self, iters, rename_data=None, rename_label=None):
        super().__init__()
        from .. import engine
        if not isinstance(iters, list):
            iters = [iters]
        self.n_iter = len(iters)
        assert self.n_iter > 0
        self.iters, self.rename_data, self.rename_label = iters, rename_data, rename_label
        self.batch_size = self.provide_data[0][1][0]
        self.current_batch = None
        self.next_batch = [None] * self.n_iter
        self._engine = engine
        self._vars = [engine.native().new_var() for _ in range(self.n_iter)]
        self.started = True
        self._fetch()

    def _fetch(self):
        def load(i):
            try:
                self.next_batch[i] = self.iters[i].next()
            except StopIteration:
                self.next_batch[i] = None
        for i in range(self.n_iter):
            self._engine.push(lambda i=i: load(i), writes=[self._vars[i]], name='prefetch')

    def _wait(self, swallow=False):
        for v in self._vars:
            try:
                self._engine.native().wait_for_var(v)
            except Exception:  # pylint: disable=broad-except
                if not swallow:
                    raise

    def __del__(self):
        self.started = False

    @property
    def provide_data(self):
        if self.rename_data is None:
            return sum([i.provide_data for i in self.iters], [])
        return sum([[DataDesc(r[x.name], x.shape, x.dtype) if isinstance(x, DataDesc) else DataDesc(*x) for x in i.provide_data]
                    for r, i in zip(self.rename_data, self.iters)], [])

    @property
    def provide_label(self):
        if self.rename_label is None:
            return sum([i.provide_label for i in self.iters], [])
        return sum([[DataDesc(r[x.name], x.shape, x.dtype) if isinstance(x, DataDesc) else DataDesc(*x) for x in i.provide_label]
                    for r, i in zip(self.rename_label, self.iters)], [])

    def reset(self):
        self._wait(swallow=True)         # the fetch in flight ends first; what it raised belongs to the old epoch
        for i in self.iters:
            i.reset()
        self._fetch()

    def iter_next(self):
        self._wait()
        if self.next_batch[0] is None:
            for i in self.next_batch:
                assert i is None, 'Number of entry mismatches between iterators'
            return False
        for batch in self.next_batch:
            assert batch.pad == self.next_batch[0].pad, 'Number of entry mismatches between iterators'
        self.current_batch = DataBatch(sum([batch.data for batch in self.next_batch], []),
                                       sum([batch.label for batch in self.next_batch], []),
                                       self.next_batch[0].pad, self.next_batch[0].index,
                                       provide_data=self.provide_data, provide_label=self.provide_label)
        self._fetch()
        return True

    def next(self):
        if self.iter_next():
            return self.current_batch
        raise StopIteration

    def getdata(self): return self.current_batch.data
    def getlabel(self): return self.current_batch.label
    def getindex(self): return self.current_batch.index
    def getpad(self): return self.current_batch.pad


class MXDataIter(DataIter):
    """Base of the natively backed iterators: subclasses fill ``_arrays`` (data, label) once or stream."""

    def __init__(self, batch_size, data_name='data', label_name='softmax_label'):
        super().__init__(batch_size)
        self.data_name, self.label_name = data_name, label_name
        self._inner = None

    def reset(self):
        self._inner.reset()

    def next(self):
        return self._inner.next()

    def iter_next(self):
        return self._inner.iter_next()

    @property
    def provide_data(self):
        return self._inner.provide_data

    @property
    def provide_label(self):
        return self._inner.provide_label


def _rt():
    from ..csrc import runtime
    return runtime.lib()


class CSVIter(MXDataIter):
    """CSV reader (``src/io/iter_csv.cc``): rows are parsed natively into float32 matrices."""

    def __init__(self, data_csv, data_shape, label_csv=None, label_shape=(1,), batch_size=1, round_batch=True,
                 dtype='float32', **kwargs):
        super().__init__(batch_size)
        data = self._load(data_csv).reshape((-1,) + tuple(data_shape))
        if label_csv is not None:
            label = self._load(label_csv).reshape((-1,) + tuple(label_shape))
            if tuple(label_shape) == (1,):
                label = label.reshape(-1)
        else:
            label = np.zeros((data.shape[0],), dtype=np.float32)
        self._inner = NDArrayIter(data.astype(dtype), label, batch_size, last_batch_handle='pad' if round_batch else 'discard')

    @staticmethod
    def _load(path):
        rows, cols = ctypes.c_int64(0), ctypes.c_int64(0)
        p = _rt().mxb_csv_load(str(path).encode(), ctypes.byref(rows), ctypes.byref(cols))
        if not p:
            raise MXNetError('cannot read %s' % path)
        n = rows.value * cols.value
        out = np.ctypeslib.as_array(p, shape=(n,)).copy().reshape(rows.value, cols.value)
        _rt().mxb_free(p)
        return out


class LibSVMIter(MXDataIter):
    """LibSVM reader (``src/io/iter_libsvm.cc``): batches are CSR arrays."""

    def __init__(self, data_libsvm, data_shape, label_libsvm=None, label_shape=(1,), batch_size=1, round_batch=True,
                 **kwargs):
        super().__init__(batch_size)
        L = _rt()
        f32p, i64p = ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_int64)
        labels, values, indices, indptr = f32p(), f32p(), i64p(), i64p()
        rows, nnz = ctypes.c_int64(0), ctypes.c_int64(0)
        rc = L.mxb_libsvm_load(str(data_libsvm).encode(), ctypes.byref(labels), ctypes.byref(values),
                               ctypes.byref(indices), ctypes.byref(indptr), ctypes.byref(rows), ctypes.byref(nnz))
        if rc != 0:
            raise MXNetError('cannot read %s' % data_libsvm)
        n, z = rows.value, nnz.value
        lab = np.ctypeslib.as_array(labels, shape=(max(n, 1),))[:n].copy()
        val = np.ctypeslib.as_array(values, shape=(max(z, 1),))[:z].copy()
        idx = np.ctypeslib.as_array(indices, shape=(max(z, 1),))[:z].copy()
        ptr = np.ctypeslib.as_array(indptr, shape=(n + 1,)).copy()
        for p in (labels, values, indices, indptr):
            L.mxb_free(p)
        import scipy.sparse as sp
        dim = int(np.prod(data_shape))
        if z and int(idx.max()) >= dim:
            raise MXNetError('%s has feature index %d but data_shape is %s' % (data_libsvm, int(idx.max()), str(data_shape)))
        # the file stays in compressed form: a feature space of millions of columns never becomes a dense [rows, dim] array
        self._csr = sp.csr_matrix((val, idx, ptr), shape=(n, dim))
        self._csr.sort_indices()
        self._label, self._n, self._dim = lab, n, dim
        self._round = round_batch
        self._cursor = 0

    def reset(self):
        self._cursor = 0

    @property
    def provide_data(self):
        return [DataDesc('data', (self.batch_size, self._dim))]

    @property
    def provide_label(self):
        return [DataDesc('softmax_label', (self.batch_size,))]

    def next(self):
        from ..ndarray import sparse
        from .. import ndarray as nd
        if self._cursor >= self._n:
            raise StopIteration
        end = self._cursor + self.batch_size
        idx = np.arange(self._cursor, end) % self._n
        pad = max(0, end - self._n)
        self._cursor = end
        return DataBatch([sparse.csr_matrix(self._csr[idx])], [nd.array(self._label[idx])], pad=pad)   # compressed CSR batch

    def iter_next(self):
        return self._cursor < self._n


class MNISTIter(MXDataIter):
    """MNIST idx-file reader (``src/io/iter_mnist.cc``)."""

    def __init__(self, image='./train-images-idx3-ubyte', label='./train-labels-idx1-ubyte', batch_size=128,
                 shuffle=True, flat=False, seed=0, silent=False, num_parts=1, part_index=0, **kwargs):
        super().__init__(batch_size)
        opener = gzip.open if str(image).endswith('.gz') else open
        with opener(image, 'rb') as f:
            _, n, r, c = struct.unpack('>IIII', f.read(16))
            img = np.frombuffer(f.read(), dtype=np.uint8).reshape(n, 1, r, c).astype(np.float32) / 255.0
        opener = gzip.open if str(label).endswith('.gz') else open
        with opener(label, 'rb') as f:
            struct.unpack('>II', f.read(8))
            lab = np.frombuffer(f.read(), dtype=np.uint8).astype(np.float32)
        if num_parts > 1:
            per = n // num_parts
            img, lab = img[part_index * per:(part_index + 1) * per], lab[part_index * per:(part_index + 1) * per]
        if flat:
            img = img.reshape(img.shape[0], -1)
        if shuffle:
            rng = np.random.RandomState(seed)
            perm = rng.permutation(img.shape[0])
            img, lab = img[perm], lab[perm]
        self._inner = NDArrayIter(img, lab, batch_size, shuffle=False, last_batch_handle='discard')


class ImageRecordIter(MXDataIter):
    """RecordIO image iterator (``src/io/iter_image_recordio_2.cc``): a native reader thread prefetches
    records, ``preprocess_threads`` host threads decode + augment, batches come out as NCHW arrays."""
    _out_dtype = np.float32

    def __init__(self, path_imgrec, data_shape, batch_size, path_imgidx=None, label_width=1, shuffle=False, seed=0,
                 preprocess_threads=4, prefetch_buffer=4, rand_crop=False, rand_mirror=False, resize=-1,
                 mean_r=0.0, mean_g=0.0, mean_b=0.0, std_r=1.0, std_g=1.0, std_b=1.0, scale=1.0, round_batch=True,
                 num_parts=1, part_index=0, data_name='data', label_name='softmax_label', mean_img=None,
                 max_random_scale=1.0, min_random_scale=1.0, layout='NCHW', device=None, dtype=None, random_resized_crop=False,
                 min_random_area=0.08, max_random_area=1.0, min_aspect_ratio=0.75, max_aspect_ratio=4.0 / 3.0, **kwargs):
        super().__init__(batch_size, data_name, label_name)
        self._path, self._shape, self._label_width = str(path_imgrec), tuple(data_shape), label_width
        # device=mx.gpu(i): decode (nvJPEG) and augment on that GPU (io/gpu_pipeline.py); batches are born on the device in
        # `dtype` (default float32) and only the compressed bytes cross the bus.  Host decode otherwise.
        # random_resized_crop: a rectangle of random area and aspect ratio resampled to data_shape (image_aug_default.cc)
        self._rrc = (float(min_random_area), float(max_random_area), float(min_aspect_ratio), float(max_aspect_ratio)) \
            if random_resized_crop else None
        self._gpu_pipe = None
        if device is not None and getattr(device, 'device_type', 'cpu') == 'gpu' and tuple(data_shape)[0] == 3:
            from .gpu_pipeline import GPUImagePipeline
            self._gpu_pipe = GPUImagePipeline(device, tuple(data_shape)[1:], layout=layout, dtype=dtype or 'float32',
                                              mean=(mean_r, mean_g, mean_b), std=(std_r, std_g, std_b), scale=scale, resize=resize,
                                              rand_crop=rand_crop, rand_mirror=rand_mirror, seed=seed, threads=preprocess_threads,
                                              random_resized_crop=self._rrc)
        self._shuffle, self._rng = shuffle, np.random.RandomState(seed)
        self._rand_crop, self._rand_mirror, self._resize = rand_crop, rand_mirror, resize
        self._mean = np.array([mean_r, mean_g, mean_b], dtype=np.float32).reshape(3, 1, 1)
        self._std = np.array([std_r, std_g, std_b], dtype=np.float32).reshape(3, 1, 1)
        self._scale, self._round, self._layout = scale, round_batch, layout
        self._pool = ThreadPoolExecutor(max(1, int(preprocess_threads)))
        self._depth = max(2, int(prefetch_buffer)) * batch_size
        self._offsets = None
        if path_imgidx and os.path.exists(path_imgidx):
            offs = []
            with open(path_imgidx) as f:
                for line in f:
                    parts = line.strip().split('\t')
                    if len(parts) >= 2:
                        offs.append(int(parts[1]))
            per = len(offs) // num_parts
            self._offsets = np.asarray(offs[part_index * per:(part_index + 1) * per] if num_parts > 1 else offs, dtype=np.int64)
        self._h = None
        self.reset()

    @property
    def provide_data(self):
        shp = self._shape if self._layout == 'NCHW' else (self._shape[1], self._shape[2], self._shape[0])
        return [DataDesc(self.data_name, (self.batch_size,) + tuple(shp), self._out_dtype, self._layout)]

    @property
    def provide_label(self):
        shp = (self.batch_size,) if self._label_width == 1 else (self.batch_size, self._label_width)
        return [DataDesc(self.label_name, shp)]

    def reset(self):
        L = _rt()
        if self._h:
            L.mxb_rec_prefetch_close(self._h)
        offs, n = None, 0
        if self._offsets is not None:
            order = self._rng.permutation(len(self._offsets)) if self._shuffle else np.arange(len(self._offsets))
            self._cur_offsets = np.ascontiguousarray(self._offsets[order])
            offs = self._cur_offsets.ctypes.data_as(ctypes.POINTER(ctypes.c_int64))
            n = len(self._cur_offsets)
        self._h = L.mxb_rec_prefetch_open(self._path.encode(), offs, n, self._depth)
        if not self._h:
            raise MXNetError('cannot open %s' % self._path)
        self._done = False

    def __del__(self):
        try:
            if self._h:
                _rt().mxb_rec_prefetch_close(self._h)
                self._h = None
        except Exception:  # pylint: disable=broad-except
            pass

    def _process(self, rec):
        from .. import recordio
        from ..image.image import _decode_to_numpy
        header, buf = recordio.unpack(rec)
        img = _decode_to_numpy(buf, 1 if self._shape[0] == 3 else 0)
        c, h, w = self._shape
        if self._rrc is not None:
            from PIL import Image
            ih, iw = img.shape[:2]
            amin, amax, rmin, rmax = self._rrc
            box = None
            for _ in range(10):
                area = np.random.uniform(amin, amax) * ih * iw
                ratio = np.exp(np.random.uniform(np.log(rmin), np.log(rmax)))
                cw, ch = int(round(np.sqrt(area * ratio))), int(round(np.sqrt(area / ratio)))
                if 0 < cw <= iw and 0 < ch <= ih:
                    x0, y0 = np.random.randint(0, iw - cw + 1), np.random.randint(0, ih - ch + 1)
                    box = (x0, y0, x0 + cw, y0 + ch)
                    break
            if box is None:
                side = min(ih, iw)
                box = ((iw - side) // 2, (ih - side) // 2, (iw - side) // 2 + side, (ih - side) // 2 + side)
            img = np.asarray(Image.fromarray(img.squeeze()).resize((w, h), Image.BILINEAR, box=box))
            if img.ndim == 2:
                img = img[:, :, None]
            if self._rand_mirror and np.random.rand() < 0.5:
                img = img[:, ::-1]
            return img, header.label
        if self._resize > 0:
            from PIL import Image
            ih, iw = img.shape[:2]
            s = self._resize / min(ih, iw)
            img = np.asarray(Image.fromarray(img.squeeze()).resize((max(w, int(iw * s + 0.5)), max(h, int(ih * s + 0.5))),
                                                                   Image.BILINEAR))
            if img.ndim == 2:
                img = img[:, :, None]
        ih, iw = img.shape[:2]
        if ih < h or iw < w:
            from PIL import Image
            img = np.asarray(Image.fromarray(img.squeeze()).resize((max(w, iw), max(h, ih)), Image.BILINEAR))
            if img.ndim == 2:
                img = img[:, :, None]
            ih, iw = img.shape[:2]
        if self._rand_crop:
            y0, x0 = np.random.randint(0, ih - h + 1), np.random.randint(0, iw - w + 1)
        else:
            y0, x0 = (ih - h) // 2, (iw - w) // 2
        img = img[y0:y0 + h, x0:x0 + w]
        if self._rand_mirror and np.random.rand() < 0.5:
            img = img[:, ::-1]
        return img, header.label

    def _finish(self, imgs):
        x = np.stack(imgs).transpose(0, 3, 1, 2).astype(np.float32)
        x = (x - self._mean[:x.shape[1]]) / self._std[:x.shape[1]] * self._scale
        if self._layout != 'NCHW':
            x = x.transpose(0, 2, 3, 1)
        return np.ascontiguousarray(x.astype(self._out_dtype))

    def next(self):
        from .. import ndarray as nd
        if self._done:
            raise StopIteration
        L = _rt()
        recs = []
        size = ctypes.c_uint64(0)
        while len(recs) < self.batch_size:
            p = L.mxb_rec_prefetch_next(self._h, ctypes.byref(size))
            if not p:
                self._done = True
                break
            recs.append(ctypes.string_at(p, size.value))
        if not recs:
            raise StopIteration
        pad = self.batch_size - len(recs)
        if pad and not self._round:
            raise StopIteration
        while len(recs) < self.batch_size:
            recs.append(recs[len(recs) % max(1, self.batch_size - pad)])
        if self._gpu_pipe is not None:
            from .. import recordio
            pairs = [recordio.unpack(r) for r in recs]
            data = self._gpu_pipe([bytes(buf) for _, buf in pairs])
            label = np.asarray([np.asarray(h.label, dtype=np.float32).reshape(-1)[:self._label_width] for h, _ in pairs],
                               dtype=np.float32)
            if self._label_width == 1:
                label = label.reshape(-1)
            return DataBatch([data], [nd.array(label, ctx=self._gpu_pipe.ctx)], pad=pad, provide_data=self.provide_data,
                             provide_label=self.provide_label)
        out = list(self._pool.map(self._process, recs))
        data = self._finish([o[0] for o in out])
        label = np.asarray([np.asarray(o[1], dtype=np.float32).reshape(-1)[:self._label_width] for o in out], dtype=np.float32)
        if self._label_width == 1:
            label = label.reshape(-1)
        return DataBatch([nd.array(data, dtype=data.dtype)], [nd.array(label)], pad=pad,
                         provide_data=self.provide_data, provide_label=self.provide_label)

    def iter_next(self):
        return not self._done


class ImageRecordUInt8Iter(ImageRecordIter):
    _out_dtype = np.uint8

    def _finish(self, imgs):
        x = np.stack(imgs).transpose(0, 3, 1, 2)
        return np.ascontiguousarray(x.astype(np.uint8))


class ImageRecordInt8Iter(ImageRecordIter):
    _out_dtype = np.int8

    def _finish(self, imgs):
        x = np.stack(imgs).transpose(0, 3, 1, 2).astype(np.int16) - 128
        return np.ascontiguousarray(x.astype(np.int8))


ImageRecordIter_v1 = ImageRecordIter


class ImageDetRecordIter(ImageRecordIter):
    """Detection records: the label is ``[header_width, object_width, ..., objects...]`` padded with -1."""

    def __init__(self, path_imgrec, data_shape, batch_size, label_pad_width=350, label_pad_value=-1.0, **kwargs):
        self._pad_width, self._pad_value = label_pad_width, label_pad_value
        super().__init__(path_imgrec, data_shape, batch_size, label_width=label_pad_width, **kwargs)

    def next(self):
        from .. import ndarray as nd
        batch = super().next()
        return batch

    def _process(self, rec):
        from .. import recordio
        from ..image.image import _decode_to_numpy
        from PIL import Image
        header, buf = recordio.unpack(rec)
        img = _decode_to_numpy(buf, 1)
        c, h, w = self._shape
        img = np.asarray(Image.fromarray(img).resize((w, h), Image.BILINEAR))
        label = np.full((self._pad_width,), self._pad_value, dtype=np.float32)
        raw = np.asarray(header.label, dtype=np.float32).reshape(-1)
        label[:min(raw.size, self._pad_width)] = raw[:self._pad_width]
        return img, label


ImageRecordUInt8Iter_v1 = ImageRecordUInt8Iter        # the first-generation iterator of the reference: same arguments and batches

"""Sparse arrays: ``CSRNDArray`` and ``RowSparseNDArray`` (``python/mxnet/ndarray/sparse.py``).

Storage types of the reference (``include/mxnet/ndarray.h:61-66``): default=0, row_sparse=1, csr=2.
On a 180 GB device the dense form is the fast path, so a sparse array here keeps its logical
dense value plus the storage-type tag; the compressed components (``data``/``indices``/``indptr``)
are derived on demand and are what the ``.params`` / ``.npz`` writers serialise, so files stay
interchangeable with the reference.
"""
from __future__ import annotations

import numpy as _np
import torch

from ..base import MXNetError, to_torch_dtype
from ..device import current_device
from .ndarray import NDArray, _to_tensor

__all__ = ['BaseSparseNDArray', 'CSRNDArray', 'RowSparseNDArray', 'csr_matrix', 'row_sparse_array', 'zeros',
           'empty', 'array', 'cast_storage', 'retain', 'dot', 'add_n']


class BaseSparseNDArray(NDArray):
    __slots__ = ()

    def __repr__(self):
        shape_info = 'x'.join(['%d' % x for x in self.shape])
        return '\n<%s %s @%s>' % (self.__class__.__name__, shape_info, self._ctx)

    def asscipy(self):
        raise NotImplementedError

    def tostype(self, stype):
        return cast_storage(self, stype)

    def _wrap_component(self, t):
        return NDArray._from_tensor(t, self._ctx)

    def copyto(self, other):
        r = super().copyto(other)
        if isinstance(r, NDArray) and not isinstance(r, BaseSparseNDArray) and not isinstance(other, NDArray):
            r = self.__class__._from_tensor(r._data, r._ctx)
            r._stype = self._stype
        return r


class CSRNDArray(BaseSparseNDArray):
    """Compressed sparse row matrix (2-D)."""
    __slots__ = ()

    @property
    def data(self):
        return self._wrap_component(self._data[self._data != 0])

    @property
    def indices(self):
        return self._wrap_component(torch.nonzero(self._data)[:, 1].contiguous())

    @property
    def indptr(self):
        counts = (self._data != 0).sum(1)
        ptr = torch.zeros(self._data.shape[0] + 1, dtype=torch.int64, device=self._data.device)
        ptr[1:] = torch.cumsum(counts, 0)
        return self._wrap_component(ptr)

    def asscipy(self):
        import scipy.sparse as sp
        return sp.csr_matrix((self.data.asnumpy(), self.indices.asnumpy(), self.indptr.asnumpy()), shape=self.shape)


class RowSparseNDArray(BaseSparseNDArray):
    """Array whose non-zero content is a subset of its rows."""
    __slots__ = ()

    def _rows(self):
        d = self._data
        if d.dim() == 1:
            return torch.nonzero(d != 0).reshape(-1)
        return torch.nonzero((d != 0).reshape(d.shape[0], -1).any(1)).reshape(-1)

    @property
    def indices(self):
        return self._wrap_component(self._rows())

    @property
    def data(self):
        return self._wrap_component(self._data[self._rows()])

    def retain(self, row_ids):
        return retain(self, row_ids)


def _tag(t, ctx, cls, stype):
    r = cls._from_tensor(t, ctx)
    r._stype = stype
    return r


def csr_matrix(arg1, shape=None, ctx=None, dtype=None, device=None):
    """Build a CSR array from (data, indices, indptr), a dense array, a scipy matrix or a shape."""
    ctx = ctx or device or current_device()
    if isinstance(arg1, tuple) and len(arg1) == 3:
        data, indices, indptr = (x.asnumpy() if isinstance(x, NDArray) else _np.asarray(x) for x in arg1)
        if shape is None:
            shape = (len(indptr) - 1, int(indices.max()) + 1 if indices.size else 0)
        dense = _np.zeros(shape, dtype=dtype or (data.dtype if data.dtype != _np.float64 else _np.float32))
        for r in range(shape[0]):
            sl = slice(int(indptr[r]), int(indptr[r + 1]))
            dense[r, indices[sl].astype(_np.int64)] = data[sl]
        return _tag(_to_tensor(dense, ctx, dense.dtype), ctx, CSRNDArray, 'csr')
    if isinstance(arg1, tuple) and len(arg1) == 2 and all(isinstance(x, int) for x in arg1):
        return _tag(torch.zeros(arg1, dtype=to_torch_dtype(dtype) or torch.float32, device=ctx.torch_device), ctx,
                    CSRNDArray, 'csr')
    if hasattr(arg1, 'tocsr'):
        arg1 = arg1.toarray()
    return _tag(_to_tensor(arg1, ctx, dtype), ctx, CSRNDArray, 'csr')


def row_sparse_array(arg1, shape=None, ctx=None, dtype=None, device=None):
    """Build a row-sparse array from (data, indices), a dense array or a shape."""
    ctx = ctx or device or current_device()
    if isinstance(arg1, tuple) and len(arg1) == 2 and not all(isinstance(x, int) for x in arg1):
        data, indices = (x.asnumpy() if isinstance(x, NDArray) else _np.asarray(x) for x in arg1)
        if shape is None:
            shape = (int(indices.max()) + 1 if indices.size else 0,) + tuple(data.shape[1:])
        dense = _np.zeros(shape, dtype=dtype or (data.dtype if data.dtype != _np.float64 else _np.float32))
        if indices.size:
            dense[indices.astype(_np.int64)] = data
        return _tag(_to_tensor(dense, ctx, dense.dtype), ctx, RowSparseNDArray, 'row_sparse')
    if isinstance(arg1, tuple) and all(isinstance(x, int) for x in arg1):
        return _tag(torch.zeros(arg1, dtype=to_torch_dtype(dtype) or torch.float32, device=ctx.torch_device), ctx,
                    RowSparseNDArray, 'row_sparse')
    return _tag(_to_tensor(arg1, ctx, dtype), ctx, RowSparseNDArray, 'row_sparse')


def zeros(stype, shape, ctx=None, dtype=None, **kwargs):
    ctx = ctx or current_device()
    t = torch.zeros(tuple(shape) if not isinstance(shape, int) else (shape,),
                    dtype=to_torch_dtype(dtype) or torch.float32, device=ctx.torch_device)
    if stype == 'csr':
        return _tag(t, ctx, CSRNDArray, 'csr')
    if stype == 'row_sparse':
        return _tag(t, ctx, RowSparseNDArray, 'row_sparse')
    return NDArray._from_tensor(t, ctx)


empty = zeros


def array(source_array, ctx=None, dtype=None):
    if isinstance(source_array, BaseSparseNDArray):
        return cast_storage(source_array.as_in_context(ctx or source_array._ctx), source_array.stype)
    if hasattr(source_array, 'tocsr'):
        return csr_matrix(source_array, ctx=ctx, dtype=dtype)
    raise ValueError('Unexpected source_array type: ', type(source_array))


def cast_storage(data, stype):
    """``cast_storage`` operator: change the storage type tag (values are preserved)."""
    if stype == 'default':
        return NDArray._from_tensor(data._data, data._ctx)
    if stype == 'csr':
        if data._data.dim() != 2:
            raise MXNetError('csr storage needs a 2-D array')
        return _tag(data._data, data._ctx, CSRNDArray, 'csr')
    if stype == 'row_sparse':
        return _tag(data._data, data._ctx, RowSparseNDArray, 'row_sparse')
    raise MXNetError('unknown storage type %s' % stype)


def retain(data, indices):
    """``_sparse_retain``: keep only the given rows."""
    idx = indices._data.long() if isinstance(indices, NDArray) else torch.as_tensor(indices, dtype=torch.long)
    out = torch.zeros_like(data._data)
    out[idx] = data._data[idx]
    return _tag(out, data._ctx, RowSparseNDArray, 'row_sparse')


def dot(lhs, rhs, transpose_a=False, transpose_b=False, forward_stype=None):
    a = lhs._data.t() if transpose_a else lhs._data
    b = rhs._data.t() if transpose_b else rhs._data
    r = NDArray._from_tensor(torch.matmul(a, b), lhs._ctx)
    if forward_stype in ('row_sparse', 'csr'):
        return cast_storage(r, forward_stype)
    return r


def add_n(*args):
    out = args[0]._data.clone()
    for a in args[1:]:
        out += a._data
    return _tag(out, args[0]._ctx, args[0].__class__, args[0].stype)

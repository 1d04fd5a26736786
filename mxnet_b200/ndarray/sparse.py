"""Sparse arrays: ``CSRNDArray`` and ``RowSparseNDArray`` (``python/mxnet/ndarray/sparse.py``).

Storage types of the reference (``include/mxnet/ndarray.h:61-66``): default=0, row_sparse=1, csr=2.

A sparse array here has two representations and is in exactly one of them at a time:

* **compressed**: only the components exist (``data`` / ``indices`` / ``indptr`` for CSR, ``data`` / ``indices`` for
  row-sparse), as in the reference (``src/ndarray/ndarray.cc`` aux arrays).  Arrays built from components, loaded from
  files, or produced by the sparse kernels (``dot`` with a CSR operand, ``retain``, ``cast_storage`` of a compressed array)
  are in this form, so a matrix whose dense form would not fit (10^6 x 10^6 features) can be created, moved and multiplied.
* **dense-backed**: the logical dense tensor plus the storage-type tag; the components are derived on demand (they are
  what the ``.params`` / ``.npz`` writers serialise).  This is the storage-fallback path of the reference
  (``src/common/exec_utils.h``: operators without a sparse implementation run on a dense copy): the first access to the
  dense tensor materialises it, and from then on the array stays dense-backed because the caller may write through it.
"""
from __future__ import annotations

import numpy as _np
import torch

from ..base import MXNetError, to_torch_dtype, to_numpy_dtype
from ..device import current_device, from_torch_device
from .ndarray import NDArray, _to_tensor

__all__ = ['BaseSparseNDArray', 'CSRNDArray', 'RowSparseNDArray', 'csr_matrix', 'row_sparse_array', 'zeros',
           'empty', 'array', 'cast_storage', 'retain', 'dot', 'add_n']


class BaseSparseNDArray(NDArray):
    __slots__ = ('_dense', '_comp', '_cshape')

    # ---- the two representations ---------------------------------------------------------------------------------------
    @property
    def _data(self):
        """The dense tensor.  Reading it materialises a compressed array and makes it dense-backed."""
        if self._dense is None:
            self._dense = self._densify()
            self._comp = None
        return self._dense

    @_data.setter
    def _data(self, t):
        self._dense = t
        self._comp = None
        self._cshape = None

    @classmethod
    def _from_components(cls, comp, shape, ctx=None):
        obj = cls.__new__(cls)
        obj._dense = None
        obj._comp = tuple(comp)
        obj._cshape = tuple(int(v) for v in shape)
        obj._ctx = ctx if ctx is not None else from_torch_device(comp[0].device)
        obj._grad = None
        obj._grad_req = 'null'
        obj._stype = cls._storage
        obj._sym = None
        obj._fresh_grad = False
        obj._hook = None
        obj._grad_pass = -1
        return obj

    @property
    def is_compressed(self):
        """True while only the components exist (no dense tensor has been materialised)."""
        return self._comp is not None

    @property
    def shape(self):
        return self._cshape if self._comp is not None else tuple(self._dense.shape)

    @property
    def dtype(self):
        d = to_numpy_dtype((self._comp[0] if self._comp is not None else self._dense).dtype)
        return d.type if isinstance(d, _np.dtype) else d

    @property
    def size(self):
        n = 1
        for v in self.shape:
            n *= v
        return n

    @property
    def ndim(self):
        return len(self.shape)

    def __repr__(self):
        shape_info = 'x'.join(['%d' % x for x in self.shape])
        return '\n<%s %s @%s>' % (self.__class__.__name__, shape_info, self._ctx)

    def asscipy(self):
        raise NotImplementedError

    def check_format(self, full_check=True):
        """Raise if the components do not describe a valid array (``MXNDArraySyncCheckFormat``): sorted, in-range,
        duplicate-free indices, consistent lengths; ``full_check=False`` checks lengths only."""
        if self._comp is None:
            return                                      # dense-backed: the components are derived, always consistent
        if self._stype == 'csr':
            data, indices, indptr = self._comp
            if indptr.numel() != self._cshape[0] + 1 or data.numel() != indices.numel() or int(indptr[-1]) != indices.numel() \
                    or int(indptr[0]) != 0:
                raise MXNetError('invalid CSR array: inconsistent component lengths')
            if full_check and indices.numel():
                if bool((indptr[1:] < indptr[:-1]).any()):
                    raise MXNetError('invalid CSR array: indptr is not non-decreasing')
                if int(indices.min()) < 0 or int(indices.max()) >= self._cshape[1]:
                    raise MXNetError('invalid CSR array: column index out of range')
                rows = torch.repeat_interleave(torch.arange(self._cshape[0], device=indices.device), indptr[1:] - indptr[:-1])
                key = rows * self._cshape[1] + indices
                if bool((key[1:] <= key[:-1]).any()):
                    raise MXNetError('invalid CSR array: column indices of a row are not strictly increasing')
        else:
            data, indices = self._comp
            if data.shape[0] != indices.numel():
                raise MXNetError('invalid row-sparse array: inconsistent component lengths')
            if full_check and indices.numel():
                if int(indices.min()) < 0 or int(indices.max()) >= self._cshape[0]:
                    raise MXNetError('invalid row-sparse array: row index out of range')
                if bool((indices[1:] <= indices[:-1]).any()):
                    raise MXNetError('invalid row-sparse array: row indices are not strictly increasing')

    def tostype(self, stype):
        return cast_storage(self, stype)

    def _wrap_component(self, t):
        return NDArray._from_tensor(t, self._ctx)

    def copy(self):
        if self._comp is not None:
            return self.__class__._from_components([c.clone() for c in self._comp], self._cshape, self._ctx)
        return _tag(self._dense.clone(), self._ctx, self.__class__, self._stype)

    def as_in_context(self, context):
        if self._comp is not None:
            if context == self._ctx:
                return self
            return self.__class__._from_components([c.to(context.torch_device) for c in self._comp], self._cshape, context)
        r = super().as_in_context(context)
        if r is not self:
            r._stype = self._stype
        return r

    as_in_ctx = as_in_context
    to_device = as_in_context

    def astype(self, dtype, copy=True):
        if self._comp is not None:
            td = to_torch_dtype(dtype)
            return self.__class__._from_components([self._comp[0].to(td)] + list(self._comp[1:]), self._cshape, self._ctx)
        r = super().astype(dtype, copy)
        if isinstance(r, NDArray) and not isinstance(r, BaseSparseNDArray):
            r = _tag(r._data, r._ctx, self.__class__, self._stype)
        return r

    def copyto(self, other):
        if self._comp is not None and not isinstance(other, NDArray):
            return self.as_in_context(other) if other != self._ctx else self.copy()
        r = super().copyto(other)
        if isinstance(r, NDArray) and not isinstance(r, BaseSparseNDArray) and not isinstance(other, NDArray):
            r = self.__class__._from_tensor(r._data, r._ctx)
            r._stype = self._stype
        return r


class CSRNDArray(BaseSparseNDArray):
    """Compressed sparse row matrix (2-D)."""
    __slots__ = ()
    _storage = 'csr'

    def _densify(self):
        data, indices, indptr = self._comp
        out = torch.zeros(self._cshape, dtype=data.dtype, device=data.device)
        if data.numel():
            counts = indptr[1:] - indptr[:-1]
            rows = torch.repeat_interleave(torch.arange(self._cshape[0], device=data.device), counts)
            out[rows, indices.long()] = data
        return out

    def _components(self):
        """(data, indices, indptr) tensors, int64 indices, without materialising anything the array does not already hold."""
        if self._comp is not None:
            return self._comp
        d = self._dense
        nz = torch.nonzero(d)
        counts = (d != 0).sum(1)
        ptr = torch.zeros(d.shape[0] + 1, dtype=torch.int64, device=d.device)
        ptr[1:] = torch.cumsum(counts, 0)
        return d[nz[:, 0], nz[:, 1]], nz[:, 1].contiguous(), ptr

    @property
    def data(self):
        return self._wrap_component(self._components()[0])

    @property
    def indices(self):
        return self._wrap_component(self._components()[1])

    @property
    def indptr(self):
        return self._wrap_component(self._components()[2])

    @property
    def nnz(self):
        return int(self._components()[0].numel())

    def asscipy(self):
        import scipy.sparse as sp
        d, i, p = (c.detach().cpu() for c in self._components())
        if d.dtype == torch.bfloat16:
            d = d.float()
        return sp.csr_matrix((d.numpy(), i.numpy(), p.numpy()), shape=self.shape)


class RowSparseNDArray(BaseSparseNDArray):
    """Array whose non-zero content is a subset of its rows."""
    __slots__ = ()
    _storage = 'row_sparse'

    def _densify(self):
        data, indices = self._comp
        out = torch.zeros(self._cshape, dtype=data.dtype, device=data.device)
        if indices.numel():
            out[indices.long()] = data
        return out

    def _rows(self):
        if self._comp is not None:
            return self._comp[1]
        d = self._dense
        if d.dim() == 1:
            return torch.nonzero(d != 0).reshape(-1)
        return torch.nonzero((d != 0).reshape(d.shape[0], -1).any(1)).reshape(-1)

    def _components(self):
        if self._comp is not None:
            return self._comp
        rows = self._rows()
        return self._dense[rows], rows

    @property
    def indices(self):
        return self._wrap_component(self._components()[1])

    @property
    def data(self):
        return self._wrap_component(self._components()[0])

    def retain(self, row_ids):
        return retain(self, row_ids)


def _tag(t, ctx, cls, stype):
    r = cls._from_tensor(t, ctx)
    r._stype = stype
    return r


def _component_tensor(x, ctx, dtype=None):
    if isinstance(x, NDArray):
        t = x._data
        if dtype is not None and t.dtype != dtype:
            t = t.to(dtype)
        return t.to(ctx.torch_device)
    a = _np.asarray(x)
    if dtype is None and a.dtype == _np.float64:
        dtype = torch.float32
    return torch.as_tensor(a, dtype=dtype, device=ctx.torch_device)


def csr_matrix(arg1, shape=None, ctx=None, dtype=None, device=None):
    """Build a CSR array from (data, indices, indptr), (data, (row, col)), a dense array, a scipy matrix or a shape.  From
    components (and from scipy matrices) the array is compressed: no dense tensor is allocated."""
    ctx = ctx or device or current_device()
    td = to_torch_dtype(dtype) if dtype is not None else None
    if hasattr(arg1, 'tocsr'):
        m = arg1.tocsr()
        m.sort_indices()
        arg1, shape = (m.data, m.indices, m.indptr), (shape or m.shape)
    if isinstance(arg1, tuple) and len(arg1) == 2 and isinstance(arg1[1], tuple) and len(arg1[1]) == 2:
        import scipy.sparse as sp                                    # coordinate form (data, (row, col))
        vals = arg1[0].asnumpy() if isinstance(arg1[0], NDArray) else _np.asarray(arg1[0])
        rc = [x.asnumpy() if isinstance(x, NDArray) else _np.asarray(x) for x in arg1[1]]
        m = sp.coo_matrix((vals, (rc[0], rc[1])), shape=shape).tocsr()
        m.sort_indices()
        arg1, shape = (m.data, m.indices, m.indptr), m.shape
    if isinstance(arg1, tuple) and len(arg1) == 3:
        data = _component_tensor(arg1[0], ctx, td)
        indices = _component_tensor(arg1[1], ctx, torch.int64)
        indptr = _component_tensor(arg1[2], ctx, torch.int64)
        if shape is None:
            shape = (indptr.numel() - 1, int(indices.max()) + 1 if indices.numel() else 0)
        if indptr.numel() != shape[0] + 1 or data.numel() != indices.numel():
            raise MXNetError('inconsistent CSR components')
        return CSRNDArray._from_components((data, indices, indptr), shape, ctx)
    if isinstance(arg1, tuple) and len(arg1) == 2 and all(isinstance(x, int) for x in arg1):
        return zeros('csr', arg1, ctx, dtype)
    return _tag(_to_tensor(arg1, ctx, dtype), ctx, CSRNDArray, 'csr')


def row_sparse_array(arg1, shape=None, ctx=None, dtype=None, device=None):
    """Build a row-sparse array from (data, indices), a dense array or a shape; from components it is compressed."""
    ctx = ctx or device or current_device()
    td = to_torch_dtype(dtype) if dtype is not None else None
    if isinstance(arg1, tuple) and len(arg1) == 2 and not all(isinstance(x, int) for x in arg1):
        data = _component_tensor(arg1[0], ctx, td)
        indices = _component_tensor(arg1[1], ctx, torch.int64).reshape(-1)
        if shape is None:
            shape = (int(indices.max()) + 1 if indices.numel() else 0,) + tuple(data.shape[1:])
        if data.shape[0] != indices.numel() or tuple(data.shape[1:]) != tuple(shape[1:]):
            raise MXNetError('inconsistent row-sparse components')
        order = torch.argsort(indices)
        return RowSparseNDArray._from_components((data[order], indices[order]), shape, ctx)
    if isinstance(arg1, tuple) and all(isinstance(x, int) for x in arg1):
        return zeros('row_sparse', arg1, ctx, dtype)
    return _tag(_to_tensor(arg1, ctx, dtype), ctx, RowSparseNDArray, 'row_sparse')


def zeros(stype, shape, ctx=None, dtype=None, **kwargs):
    """All-zero array of the storage type; the sparse ones hold no elements (nothing of the dense size is allocated)."""
    ctx = ctx or current_device()
    shape = tuple(shape) if not isinstance(shape, int) else (shape,)
    td = to_torch_dtype(dtype) or torch.float32
    dev = ctx.torch_device
    if stype == 'csr':
        if len(shape) != 2:
            raise MXNetError('csr storage needs a 2-D array')
        return CSRNDArray._from_components((torch.zeros(0, dtype=td, device=dev), torch.zeros(0, dtype=torch.int64, device=dev),
                                            torch.zeros(shape[0] + 1, dtype=torch.int64, device=dev)), shape, ctx)
    if stype == 'row_sparse':
        return RowSparseNDArray._from_components((torch.zeros((0,) + shape[1:], dtype=td, device=dev),
                                                  torch.zeros(0, dtype=torch.int64, device=dev)), shape, ctx)
    return NDArray._from_tensor(torch.zeros(shape, dtype=td, device=dev), ctx)


empty = zeros


def array(source_array, ctx=None, dtype=None):
    if isinstance(source_array, BaseSparseNDArray):
        return cast_storage(source_array.as_in_context(ctx or source_array._ctx), source_array.stype)
    if hasattr(source_array, 'tocsr'):
        return csr_matrix(source_array, ctx=ctx, dtype=dtype)
    raise ValueError('Unexpected source_array type: ', type(source_array))


def cast_storage(data, stype):
    """``cast_storage`` operator (``src/operator/tensor/cast_storage-inl.h``): values are preserved.  A compressed array stays
    compressed when the type does not change; every other combination goes through the dense tensor and is dense-backed."""
    if isinstance(data, BaseSparseNDArray) and data.is_compressed and data.stype == stype:
        return data.copy()
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
    if isinstance(data, RowSparseNDArray) and data.is_compressed:
        vals, rows = data._comp
        keep = torch.isin(rows, idx.to(rows.device))
        return RowSparseNDArray._from_components((vals[keep], rows[keep]), data.shape, data._ctx)
    out = torch.zeros_like(data._data)
    out[idx] = data._data[idx]
    return _tag(out, data._ctx, RowSparseNDArray, 'row_sparse')


def _spmm(comp, shape, dense, transpose_a):
    """csr (or its transpose) times a dense matrix from the components: the in-tree kernels on a GPU
    (``ops/cuda/sparse.cu``), the tensor library's CSR product on the host."""
    data, indices, indptr = comp
    M, K = shape
    if dense.dim() == 1:
        return _spmm(comp, shape, dense.reshape(-1, 1), transpose_a).reshape(-1)
    if dense.shape[0] != (M if transpose_a else K):
        raise MXNetError('dot: shapes %s%s and %s do not match' % (shape, '.T' if transpose_a else '', tuple(dense.shape)))
    if data.is_cuda:
        from ..ops import cuda
        if cuda.available():
            from ..ops.cuda import sparse_ops
            if sparse_ops.supported(data, dense):
                return sparse_ops.csr_dot_dense(data, indices, indptr, M, K, dense, transpose_a)
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter('ignore', UserWarning)            # the tensor library announces its CSR support as beta
        a = torch.sparse_csr_tensor(indptr, indices, data.float(), size=(M, K), check_invariants=False)
    if transpose_a:
        a = a.to_sparse_coo().t().coalesce()
        return torch.sparse.mm(a, dense.float()).to(dense.dtype)
    return (a @ dense.float()).to(dense.dtype)


def dot(lhs, rhs, transpose_a=False, transpose_b=False, forward_stype=None):
    """``dot`` with sparse operands (``src/operator/tensor/dot-inl.h``): csr x dense and csr.T x dense run from the compressed
    components; csr.T x dense with ``forward_stype='row_sparse'`` returns only the rows that received a contribution.  Other
    combinations use the dense tensors."""
    if isinstance(lhs, CSRNDArray) and lhs.is_compressed and not transpose_b and not isinstance(rhs, CSRNDArray):
        dense = rhs._data
        out = _spmm(lhs._comp, lhs.shape, dense, transpose_a)
        if transpose_a and forward_stype == 'row_sparse':
            rows = torch.unique(lhs._comp[1])
            return RowSparseNDArray._from_components((out[rows], rows), tuple(out.shape), lhs._ctx)
        r = NDArray._from_tensor(out, lhs._ctx)
        return cast_storage(r, forward_stype) if forward_stype in ('row_sparse', 'csr') else r
    a = lhs._data.t() if transpose_a else lhs._data
    b = rhs._data.t() if transpose_b else rhs._data
    r = NDArray._from_tensor(torch.matmul(a, b), lhs._ctx)
    if forward_stype in ('row_sparse', 'csr'):
        return cast_storage(r, forward_stype)
    return r


def add_n(*args):
    if all(isinstance(a, RowSparseNDArray) and a.is_compressed for a in args):
        rows = torch.unique(torch.cat([a._comp[1] for a in args]))
        vals = torch.zeros((rows.numel(),) + tuple(args[0].shape[1:]), dtype=args[0]._comp[0].dtype, device=rows.device)
        for a in args:
            vals.index_add_(0, torch.searchsorted(rows, a._comp[1]), a._comp[0])
        return RowSparseNDArray._from_components((vals, rows), args[0].shape, args[0]._ctx)
    out = args[0]._data.clone()
    for a in args[1:]:
        out += a._data
    return _tag(out, args[0]._ctx, args[0].__class__, args[0].stype)


def _elementwise(name, torch_fn, keeps_zero_rows):
    def fn(lhs, rhs):
        """Element-wise arithmetic with sparse operands (``python/mxnet/ndarray/sparse.py``: add / subtract / multiply /
        divide).  Two row-sparse arrays (or a row-sparse array and a scalar, for multiply and divide) give a row-sparse
        result computed on the stored rows only; every other combination uses the dense tensors and returns a dense array."""
        ls, rs = isinstance(lhs, RowSparseNDArray) and lhs.is_compressed, isinstance(rhs, RowSparseNDArray) and rhs.is_compressed
        if ls and rs and name in ('add', 'subtract'):
            return add_n(lhs, rhs if name == 'add' else RowSparseNDArray._from_components((-rhs._comp[0], rhs._comp[1]), rhs.shape,
                                                                                          rhs._ctx))
        if ls and not isinstance(rhs, NDArray) and keeps_zero_rows:
            return RowSparseNDArray._from_components((torch_fn(lhs._comp[0], rhs), lhs._comp[1]), lhs.shape, lhs._ctx)
        a = lhs._data if isinstance(lhs, NDArray) else lhs
        b = rhs._data if isinstance(rhs, NDArray) else rhs
        ctx = lhs._ctx if isinstance(lhs, NDArray) else rhs._ctx
        return NDArray._from_tensor(torch_fn(a, b), ctx)
    fn.__name__ = name
    return fn


add = _elementwise('add', torch.add, False)
subtract = _elementwise('subtract', torch.sub, False)
multiply = _elementwise('multiply', torch.mul, True)
divide = _elementwise('divide', torch.true_divide, True)
__all__ += ['add', 'subtract', 'multiply', 'divide']

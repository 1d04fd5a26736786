"""``mx.nd.NDArray``: the legacy array class, a thin owner of a ``torch.Tensor``.

Reference: ``include/mxnet/ndarray.h:82-1180`` (native chunk + engine variable) and
``python/mxnet/ndarray/ndarray.py`` (Python methods).  Here the storage, the asynchronous
execution and the autograd entry all come from the wrapped tensor: CUDA work is asynchronous on
the current stream, ``wait_to_read`` synchronises on it, and the gradient buffer attached by
:meth:`attach_grad` is owned by this class so that its address stays stable for the fused
KVStore kernels that read it in place.
"""
from __future__ import annotations

import numbers

import numpy as _np
import torch

from .. import _state
from ..base import (MXNetError, to_torch_dtype, to_numpy_dtype, numeric_types, integer_types)
from ..device import Device, current_device, from_torch_device
from ..ops import registry as _reg

__all__ = ['NDArray', 'array', 'empty', 'zeros', 'ones', 'full', 'arange', 'concatenate',
           'waitall', 'from_numpy', 'from_dlpack', 'to_dlpack_for_read', 'to_dlpack_for_write',
           'onehot_encode', 'moveaxis', 'imdecode']

_STORAGE_TYPE_STR = {0: 'default', 1: 'row_sparse', 2: 'csr'}

def _torch_device_of(ctx):
    return ctx.torch_device if ctx is not None else current_device().torch_device


class NDArray(object):
    """N-dimensional array on a device.  ``_kind`` selects legacy (``nd``) or NumPy (``np``) semantics."""
    __slots__ = ('_data', '_ctx', '_grad', '_grad_req', '_stype', '_sym', '_fresh_grad', '_hook', '_grad_pass', '_prov', '_freed',
                 '__weakref__')
    _kind = 'nd'
    __array_priority__ = 1000.0

    def __init__(self, data=None, ctx=None, dtype=None):
        if isinstance(data, NDArray):
            data = data._data
        if not isinstance(data, torch.Tensor):
            data = _to_tensor(data, ctx, dtype)
        self._data = data
        self._ctx = ctx if ctx is not None else from_torch_device(data.device)
        self._grad = None
        self._grad_req = 'null'
        self._stype = 'default'
        self._sym = None
        self._fresh_grad = False
        self._hook = None
        self._grad_pass = -1

    @classmethod
    def _from_tensor(cls, t, ctx=None):
        obj = cls.__new__(cls)
        obj._data = t
        obj._ctx = ctx if (ctx is not None and t.device.type == ('cuda' if ctx.device_typeid == 2 else 'cpu')) \
            else from_torch_device(t.device)
        obj._grad = None
        obj._grad_req = 'null'
        obj._stype = 'default'
        obj._sym = None
        obj._fresh_grad = False
        obj._hook = None
        obj._grad_pass = -1
        return obj

    # ------------------------------------------------------------------ basic properties
    @property
    def shape(self):
        return tuple(self._data.shape)

    @property
    def dtype(self):
        d = to_numpy_dtype(self._data.dtype)
        return d.type if isinstance(d, _np.dtype) else d

    @property
    def size(self):
        return self._data.numel()

    @property
    def ndim(self):
        return self._data.dim()

    @property
    def context(self):
        return self._ctx

    ctx = context
    device = context

    @property
    def stype(self):
        return self._stype

    @property
    def T(self):
        if self._data.dim() < 2:
            return self
        return self.transpose()

    @property
    def handle(self):
        """Opaque identity of the underlying storage (address), for engine/KVStore bookkeeping."""
        return self._data.data_ptr()

    @property
    def writable(self):
        return True

    def __repr__(self):
        shape_info = 'x'.join(['%d' % x for x in self.shape])
        return '\n%s\n<%s %s @%s>' % (str(self.asnumpy()), self.__class__.__name__, shape_info, self._ctx)

    def __reduce__(self):
        return (_rebuild, (self.__class__, self.asnumpy(), self._ctx.device_type, self._ctx.device_id,
                           str(self._data.dtype)))

    def __len__(self):
        if self._data.dim() == 0:
            raise TypeError('len() of unsized object')
        return self._data.shape[0]

    def __bool__(self):
        n = self._data.numel()
        if n == 0:
            return False
        if n == 1:
            return bool(self._data.item())
        raise ValueError('The truth value of an NDArray with multiple elements is ambiguous.')

    __nonzero__ = __bool__

    def __float__(self):
        return float(self.asscalar())

    def __int__(self):
        return int(self.asscalar())

    def __index__(self):
        return int(self.asscalar())

    def __iter__(self):
        for i in range(len(self)):
            yield self[i]

    def __hash__(self):
        return id(self) // 16

    def __array__(self, dtype=None, copy=None):
        a = self.asnumpy()
        return a.astype(dtype) if dtype is not None else a

    # ------------------------------------------------------------------ host transfer / sync
    def asnumpy(self):
        """Blocking copy to a ``numpy.ndarray`` (``SyncCopyToCPU``)."""
        from .. import engine
        engine.wait_for(self)                   # host tasks that write this array (and their exceptions)
        t = self._data.detach()
        if t.dtype == torch.bfloat16:
            t = t.float()
        if t.is_cuda:
            t = t.cpu()
        return t.numpy().copy() if t.dim() else _np.array(t.numpy())

    def asscalar(self):
        if self._data.numel() != 1:
            raise ValueError('The current array is not a scalar')
        return self.asnumpy().reshape(-1)[0]

    def item(self, *args):
        return self.asnumpy().item(*args)

    def tolist(self):
        return self.asnumpy().tolist()

    def wait_to_read(self):
        """Block until every pending write to this array has finished (``WaitToRead``)."""
        from .. import engine
        engine.wait_for(self)
        if self._data.is_cuda:
            engine._sync_device(self._data.device)
        engine._rethrow_pending()

    wait_to_write = wait_to_read

    # ------------------------------------------------------------------ conversion
    def astype(self, dtype, copy=True):
        td = to_torch_dtype(dtype)
        if not copy and td == self._data.dtype:
            return self
        return _reg.invoke('Cast' if self._kind == 'nd' else '_npi_cast', [self], {'dtype': td})

    def copy(self):
        return _reg.invoke('_copy', [self], {})

    def copyto(self, other):
        """Copy into another array, or onto a device (returns the new array)."""
        if isinstance(other, NDArray):
            if other is self:
                return other
            with torch.no_grad():
                other._data.copy_(self._data, non_blocking=True)
            return other
        if isinstance(other, Device):
            t = self._data.to(other.torch_device, copy=True)
            return self.__class__._from_tensor(t, other)
        raise TypeError('copyto does not support type ' + str(type(other)))

    def as_in_context(self, context):
        if self._ctx == context:
            return self
        if context.torch_device == self._data.device:
            # another logical id of the same physical device (e.g. cpu(1)): share nothing
            r = self.__class__._from_tensor(self._data.clone() if not _state.state.recording
                                            else _identity_copy(self._data), context)
            r._ctx = context
            return r
        if _state.state.recording and self._data.requires_grad:
            t = self._data.to(context.torch_device)
        elif context.torch_device.type == 'cuda' and not self._data.is_cuda:
            from .. import engine
            engine.wait_for(self)
            t = engine.to_device_async(self._data.detach(), context.torch_device)   # copy-in stream when the source is pinned
        else:
            t = self._data.detach().to(context.torch_device, non_blocking=True)
        return self.__class__._from_tensor(t, context)

    as_in_ctx = as_in_context
    to_device = as_in_context

    def as_np_ndarray(self):
        from ..numpy.multiarray import ndarray
        r = ndarray._from_tensor(self._data, self._ctx)
        r._grad, r._grad_req = self._grad, self._grad_req
        return r

    def as_nd_ndarray(self):
        r = NDArray._from_tensor(self._data, self._ctx)
        r._grad, r._grad_req = self._grad, self._grad_req
        return r

    def tostype(self, stype):
        if stype == 'default':
            return self
        from . import sparse
        return sparse.cast_storage(self, stype)

    def to_dlpack_for_read(self):
        return torch.utils.dlpack.to_dlpack(self._data.detach())

    to_dlpack_for_write = to_dlpack_for_read

    def __dlpack__(self, stream=None):
        return self._data.detach().__dlpack__()

    def __dlpack_device__(self):
        return self._data.__dlpack_device__()

    # ------------------------------------------------------------------ autograd
    def attach_grad(self, grad_req='write', stype=None):
        """Allocate a gradient buffer and mark this array as a differentiable leaf.

        Reference: ``MXAutogradMarkVariables`` → ``Imperative::MarkVariables``
        (``src/imperative/imperative.cc:143-172``).
        """
        from .. import autograd
        stype = stype or getattr(self, '_stype', 'default')
        if stype in ('csr', 'row_sparse'):
            from . import sparse
            cls = sparse.CSRNDArray if stype == 'csr' else sparse.RowSparseNDArray
            grad = sparse._tag(torch.zeros_like(self._data), self._ctx, cls, stype)       # gradient with the asked storage type
        else:
            from .ndarray import NDArray as _Dense
            base = self.__class__ if getattr(self, '_stype', 'default') == 'default' else _Dense
            grad = base._from_tensor(torch.zeros_like(self._data), self._ctx)
        autograd.mark_variables([self], [grad], grad_req)

    @property
    def grad(self):
        return self._grad

    def detach(self):
        r = self.__class__._from_tensor(self._data.detach(), self._ctx)
        r._stype = getattr(self, '_stype', 'default')
        return r

    def backward(self, out_grad=None, retain_graph=False, train_mode=True):
        from .. import autograd
        autograd.backward([self], [out_grad] if out_grad is not None else None,
                          retain_graph=retain_graph, train_mode=train_mode)

    def zero_grad(self):
        if self._grad is not None:
            self._grad._data.zero_()

    # ------------------------------------------------------------------ indexing
    def _index_key(self, key):
        if isinstance(key, NDArray):
            t = key._data
            return t if t.dtype in (torch.bool, torch.int64) else t.long()
        if isinstance(key, tuple):
            return tuple(self._index_key(k) for k in key)
        if isinstance(key, list):
            return torch.as_tensor(key, device=self._data.device)
        if isinstance(key, _np.ndarray):
            t = torch.from_numpy(key).to(self._data.device)
            return t if t.dtype in (torch.bool, torch.int64) else t.long()
        if isinstance(key, _np.integer):
            return int(key)
        return key

    def __getitem__(self, key):
        k = self._index_key(key)
        st = _state.state
        if st.tracer is not None or st.recording:
            return _reg.invoke('_index', [self], {'key': k})
        with torch.no_grad():
            t = self._data[k]
        return self.__class__._from_tensor(t, self._ctx)

    def __setitem__(self, key, value):
        if isinstance(value, NDArray):
            v = value._data
            if v.device != self._data.device:
                v = v.to(self._data.device)
        elif isinstance(value, (_np.ndarray, list, tuple)):
            v = torch.as_tensor(_np.asarray(value), device=self._data.device).to(self._data.dtype)
        else:
            v = value
        k = self._index_key(key)
        if _state.state.recording and (self._data.requires_grad or
                                      (isinstance(v, torch.Tensor) and v.requires_grad)):
            # functional update so the tape sees it (reference: _npi_slice_assign et al.)
            new = self._data.clone()
            new[k] = v if not isinstance(v, torch.Tensor) else v.to(new.dtype)
            self._data = new
            return
        with torch.no_grad():
            if isinstance(v, torch.Tensor):
                v = v.to(self._data.dtype)
            elif isinstance(v, _np.generic):
                v = v.item()                                   # numpy scalars (np.float32(1.5), ...)
            elif isinstance(v, _np.ndarray):
                v = torch.as_tensor(v, dtype=self._data.dtype, device=self._data.device)
            self._data[k] = v

    # ------------------------------------------------------------------ shape manipulation
    def reshape(self, *shape, **kwargs):
        if len(shape) == 1 and isinstance(shape[0], (list, tuple)):
            shape = tuple(shape[0])
        elif not shape:
            shape = kwargs.get('shape')
        reverse = kwargs.get('reverse', False)
        if self._kind == 'nd':
            try:
                return _reg.invoke('Reshape', [self], {'shape': tuple(shape), 'reverse': reverse})
            except MXNetError as e:
                if 'invalid for input of size' in str(e):
                    raise ValueError('cannot reshape array of size %d into shape %s' % (self.size, str(tuple(shape)))) from e
                raise
        return _reg.invoke('_npi_reshape', [self], {'newshape': tuple(shape)})

    def reshape_like(self, other):
        return _reg.invoke('reshape_like', [self, other], {})

    def transpose(self, *axes, **kwargs):
        if not axes and 'axes' in kwargs:
            axes = (kwargs['axes'],)
        if len(axes) == 1 and (isinstance(axes[0], (list, tuple)) or axes[0] is None):
            axes = axes[0]
        return _reg.invoke('transpose', [self], {'axes': tuple(axes) if axes else None})

    # flatten / expand_dims / squeeze return a copy; with inplace=True a view that shares memory with this array
    # (python/mxnet/ndarray/ndarray.py: the inplace forms reshape the same storage)
    def _own(self, result, inplace):
        if inplace or self._kind == 'np' or result._data.requires_grad:
            return result
        if result._data.untyped_storage().data_ptr() == self._data.untyped_storage().data_ptr():
            result._data = result._data.clone()
        return result

    def flatten(self, inplace=False):
        if self._kind == 'np':
            return self.reshape(-1)
        return self._own(_reg.invoke('Flatten', [self], {}), inplace)

    def expand_dims(self, axis, inplace=False):
        return self._own(_reg.invoke('expand_dims', [self], {'axis': axis}), inplace)

    def squeeze(self, axis=None, inplace=False):
        return self._own(_reg.invoke('squeeze', [self], {'axis': axis}), inplace)

    def swapaxes(self, dim1, dim2):
        return _reg.invoke('SwapAxis', [self], {'dim1': dim1, 'dim2': dim2})

    def broadcast_to(self, shape):
        return _reg.invoke('broadcast_to', [self], {'shape': tuple(shape)})

    def broadcast_like(self, other):
        return _reg.invoke('broadcast_like', [self, other], {})

    def slice_assign(self, rhs, begin, end, step):
        return _reg.invoke('_slice_assign', [self, rhs], {'begin': begin, 'end': end, 'step': step})

    # ------------------------------------------------------------------ arithmetic
    def _binary(self, other, name, reverse=False):
        np_mode = self._kind == 'np'
        if isinstance(other, NDArray):
            opn = ('_npi_' + name) if np_mode else ('broadcast_' + name)
            args = [other, self] if reverse else [self, other]
            return _reg.invoke(opn, args, {})
        if isinstance(other, (numbers.Number, _np.generic, bool)):
            if isinstance(other, _np.generic):
                other = other.item()
            if np_mode:
                opn = '_npi_r%s_scalar' % name if reverse else '_npi_%s_scalar' % name
            else:
                opn = '_r%s_scalar' % name if reverse else '_%s_scalar' % name
            return _reg.invoke(opn, [self], {'scalar': other})
        if isinstance(other, (_np.ndarray, list, tuple)):
            o = self.__class__(_np.asarray(other), ctx=self._ctx)
            return self._binary(o, name, reverse)
        return NotImplemented

    def __add__(self, o): return self._binary(o, 'add')
    def __radd__(self, o): return self._binary(o, 'add', True)
    def __sub__(self, o): return self._binary(o, 'sub')
    def __rsub__(self, o): return self._binary(o, 'sub', True)
    def __mul__(self, o): return self._binary(o, 'mul')
    def __rmul__(self, o): return self._binary(o, 'mul', True)
    def __truediv__(self, o): return self._binary(o, 'div')
    def __rtruediv__(self, o): return self._binary(o, 'div', True)
    __div__ = __truediv__
    __rdiv__ = __rtruediv__
    def __floordiv__(self, o): return self._binary(o, 'floordiv')
    def __rfloordiv__(self, o): return self._binary(o, 'floordiv', True)
    def __mod__(self, o): return self._binary(o, 'mod')
    def __rmod__(self, o): return self._binary(o, 'mod', True)
    def __pow__(self, o): return self._binary(o, 'power')
    def __rpow__(self, o): return self._binary(o, 'power', True)
    def __matmul__(self, o): return _reg.invoke('_npi_matmul', [self, o], {})
    def __rmatmul__(self, o): return _reg.invoke('_npi_matmul', [o, self], {})
    def __and__(self, o): return self._binary(o, 'bitwise_and')
    def __or__(self, o): return self._binary(o, 'bitwise_or')
    def __xor__(self, o): return self._binary(o, 'bitwise_xor')
    __rand__ = __and__
    __ror__ = __or__
    __rxor__ = __xor__
    def __invert__(self): return _reg.invoke('_npi_invert', [self], {})
    def __neg__(self): return _reg.invoke('negative', [self], {})
    def __pos__(self): return self
    def __abs__(self): return _reg.invoke('abs', [self], {})

    def __eq__(self, o):
        if o is None:
            return False
        return self._binary(o, 'equal')

    def __ne__(self, o):
        if o is None:
            return True
        return self._binary(o, 'not_equal')

    def __gt__(self, o): return self._binary(o, 'greater')
    def __ge__(self, o): return self._binary(o, 'greater_equal')
    def __lt__(self, o): return self._binary(o, 'lesser')
    def __le__(self, o): return self._binary(o, 'lesser_equal')

    def _inplace(self, other, name):
        if _state.state.recording and self._data.requires_grad:
            raise MXNetError('Inplace operations (+=, -=, x[:]=, etc) are not supported when '
                             'recording with autograd.')
        res = self._binary(other, name)
        if res is NotImplemented:
            return res
        with torch.no_grad():
            if res._data.dtype != self._data.dtype or res._data.shape != self._data.shape:
                self._data.copy_(res._data.to(self._data.dtype).expand_as(self._data)
                                 if res._data.shape != self._data.shape else res._data)
            else:
                self._data.copy_(res._data)
        return self

    def __iadd__(self, o): return self._inplace(o, 'add')
    def __isub__(self, o): return self._inplace(o, 'sub')
    def __imul__(self, o): return self._inplace(o, 'mul')
    def __itruediv__(self, o): return self._inplace(o, 'div')
    __idiv__ = __itruediv__
    def __imod__(self, o): return self._inplace(o, 'mod')

    # ------------------------------------------------------------------ fluent methods
    def _reduce(self, opname, axis=None, keepdims=False, **kw):
        attrs = {'axis': axis, 'keepdims': keepdims}
        attrs.update(kw)
        return _reg.invoke(opname, [self], attrs)

    def sum(self, axis=None, keepdims=False, **kw): return self._reduce('sum', axis, keepdims, **kw)
    def mean(self, axis=None, keepdims=False, **kw): return self._reduce('mean', axis, keepdims, **kw)
    def prod(self, axis=None, keepdims=False, **kw): return self._reduce('prod', axis, keepdims, **kw)
    def max(self, axis=None, keepdims=False, **kw): return self._reduce('max', axis, keepdims, **kw)
    def min(self, axis=None, keepdims=False, **kw): return self._reduce('min', axis, keepdims, **kw)
    def nansum(self, axis=None, keepdims=False, **kw): return self._reduce('nansum', axis, keepdims)
    def nanprod(self, axis=None, keepdims=False, **kw): return self._reduce('nanprod', axis, keepdims)

    def norm(self, ord=2, axis=None, keepdims=False, **kw):
        return _reg.invoke('norm', [self], {'ord': ord, 'axis': axis, 'keepdims': keepdims})

    def argmax(self, axis=None, keepdims=False):
        return _reg.invoke('argmax' if self._kind == 'nd' else '_npi_argmax', [self],
                           {'axis': axis, 'keepdims': keepdims})

    def argmin(self, axis=None, keepdims=False):
        return _reg.invoke('argmin' if self._kind == 'nd' else '_npi_argmin', [self],
                           {'axis': axis, 'keepdims': keepdims})

    def argsort(self, axis=-1, is_ascend=True, dtype='float32'):
        return _reg.invoke('argsort', [self], {'axis': axis, 'is_ascend': is_ascend, 'dtype': dtype})

    def sort(self, axis=-1, is_ascend=True):
        return _reg.invoke('sort', [self], {'axis': axis, 'is_ascend': is_ascend})

    def topk(self, **kw):
        return _reg.invoke('topk', [self], kw)

    def clip(self, a_min=None, a_max=None, **kw):
        return _reg.invoke('clip', [self], {'a_min': a_min, 'a_max': a_max})

    def dot(self, other, **kw):
        return _reg.invoke('dot', [self, other], kw)

    def take(self, indices, axis=0, mode='clip'):
        return _reg.invoke('take', [self, indices], {'axis': axis, 'mode': mode})

    def pick(self, index, axis=-1, keepdims=False, mode='clip'):
        return _reg.invoke('pick', [self, index], {'axis': axis, 'keepdims': keepdims, 'mode': mode})

    def one_hot(self, depth, **kw):
        kw['depth'] = depth
        return _reg.invoke('one_hot', [self], kw)

    def tile(self, reps):
        return _reg.invoke('tile', [self], {'reps': reps})

    def repeat(self, repeats, axis=None):
        return _reg.invoke('repeat', [self], {'repeats': repeats, 'axis': axis})

    def flip(self, axis):
        return _reg.invoke('reverse', [self], {'axis': axis})

    def split(self, num_outputs, axis=1, squeeze_axis=False):
        return _reg.invoke('SliceChannel', [self], {'num_outputs': num_outputs, 'axis': axis,
                                                    'squeeze_axis': squeeze_axis})

    def slice(self, begin, end, step=None):
        return _reg.invoke('slice', [self], {'begin': begin, 'end': end, 'step': step})

    def slice_axis(self, axis, begin, end):
        return _reg.invoke('slice_axis', [self], {'axis': axis, 'begin': begin, 'end': end})

    def slice_like(self, other=None, axes=None, shape_like=None):
        return _reg.invoke('slice_like', [self, other if other is not None else shape_like], {'axes': axes})

    def softmax(self, axis=-1, **kw):
        kw['axis'] = axis
        return _reg.invoke('softmax', [self], kw)

    def log_softmax(self, axis=-1, **kw):
        kw['axis'] = axis
        return _reg.invoke('log_softmax', [self], kw)

    def diag(self, k=0, **kw):
        return _reg.invoke('diag', [self], {'k': k})

    def zeros_like(self): return _reg.invoke('zeros_like', [self], {})
    def ones_like(self): return _reg.invoke('ones_like', [self], {})

    def fill(self, value):
        with torch.no_grad():
            self._data.fill_(value)

    def all(self, axis=None, keepdims=False, out=None, **_ignored):
        return _reg.invoke('_npi_all', [self], {'axis': axis, 'keepdims': keepdims})

    def any(self, axis=None, keepdims=False, out=None, **_ignored):
        return _reg.invoke('_npi_any', [self], {'axis': axis, 'keepdims': keepdims})

    def std(self, axis=None, dtype=None, ddof=0, keepdims=False):
        return _reg.invoke('_npi_std', [self], {'axis': axis, 'ddof': ddof, 'keepdims': keepdims})

    def var(self, axis=None, dtype=None, ddof=0, keepdims=False):
        return _reg.invoke('_npi_var', [self], {'axis': axis, 'ddof': ddof, 'keepdims': keepdims})

    def cumsum(self, axis=None, dtype=None):
        return _reg.invoke('_npi_cumsum', [self], {'axis': axis, 'dtype': dtype})

    def round(self, decimals=0):
        return _reg.invoke('_npi_around', [self], {'decimals': decimals})


def _unary_method(opname):
    def method(self, *args, **kwargs):
        return _reg.invoke(opname, [self], kwargs)
    method.__name__ = opname
    return method


for _n in ('abs', 'sign', 'sqrt', 'rsqrt', 'cbrt', 'rcbrt', 'square', 'reciprocal', 'relu', 'sigmoid',
           'exp', 'expm1', 'log', 'log10', 'log2', 'log1p', 'sin', 'cos', 'tan', 'arcsin', 'arccos',
           'arctan', 'sinh', 'cosh', 'tanh', 'arcsinh', 'arccosh', 'arctanh', 'degrees', 'radians',
           'floor', 'ceil', 'trunc', 'rint', 'fix', 'erf', 'gamma', 'gammaln', 'softsign'):
    if not hasattr(NDArray, _n):
        setattr(NDArray, _n, _unary_method(_n))

_reg._set_array_class('nd', NDArray)


def _identity_copy(t):
    return t.clone()


def _rebuild(cls, arr, devtype, devid, tdtype):
    ctx = Device(devtype, devid)
    if devtype == 'gpu' and not torch.cuda.is_available():
        ctx = Device('cpu', 0)
    t = torch.from_numpy(_np.ascontiguousarray(arr)).to(ctx.torch_device)
    if tdtype == 'torch.bfloat16':
        t = t.to(torch.bfloat16)
    return cls._from_tensor(t, ctx)


def _default_float():
    return torch.float64 if _state.state.np_default_dtype else torch.float32


def _to_tensor(src, ctx=None, dtype=None, default_float32=True):
    """Build a tensor from python / numpy data with MXNet's dtype defaults (float32 unless asked)."""
    dev = _torch_device_of(ctx)
    td = to_torch_dtype(dtype)
    if isinstance(src, NDArray):
        t = src._data
        return t.to(device=dev, dtype=td or t.dtype)
    if isinstance(src, torch.Tensor):
        return src.to(device=dev, dtype=td or src.dtype)
    if isinstance(src, _np.ndarray):
        a = src
        if td is None:
            if a.dtype == _np.float64 and default_float32:
                td = _default_float()
            elif a.dtype.kind in 'OUS':
                raise TypeError('unsupported array dtype %s' % a.dtype)
        if not a.flags.c_contiguous or not a.flags.writeable:
            a = _np.array(a, order='C')
        if a.dtype == _np.uint16 or a.dtype == _np.uint32 or a.dtype == _np.uint64:
            a = a.astype(_np.int64)
        t = torch.from_numpy(a)
        return t.to(device=dev, dtype=td or t.dtype)
    a = _np.asarray(src)
    if a.dtype.kind in 'OUS':
        raise TypeError('cannot convert %r to an array' % type(src))
    if td is None:
        if a.dtype.kind == 'f':
            td = _default_float() if default_float32 else to_torch_dtype(a.dtype)
        elif default_float32 and a.dtype.kind in 'iu' and not _state.state.np_array:
            td = torch.float32   # legacy nd.array defaults to float32 even for python ints
        elif a.dtype.kind == 'b':
            td = torch.bool
        else:
            td = torch.int64
    return torch.from_numpy(_np.ascontiguousarray(a)).to(device=dev, dtype=td)


# ------------------------------------------------------------------------------------------
# creation routines of mx.nd
# ------------------------------------------------------------------------------------------
def array(source_array, ctx=None, dtype=None, device=None):
    ctx = ctx or device
    if dtype is None:
        # python/mxnet/ndarray/ndarray.py:3450-3453: an NDArray source keeps its dtype, anything else is float32
        dtype = source_array._data.dtype if isinstance(source_array, NDArray) else _np.float32
    t = _to_tensor(source_array, ctx, dtype)
    return NDArray._from_tensor(t, ctx or current_device())


def empty(shape, ctx=None, dtype=None, device=None, stype=None):
    ctx = ctx or device or current_device()
    if isinstance(shape, integer_types):
        shape = (shape,)
    return NDArray._from_tensor(torch.empty(tuple(shape), dtype=to_torch_dtype(dtype) or torch.float32,
                                            device=ctx.torch_device), ctx)


def zeros(shape, ctx=None, dtype=None, stype=None, device=None, out=None, **kwargs):
    if out is not None:
        with torch.no_grad():
            out._data.zero_()
        return out
    ctx = ctx or device or current_device()
    if isinstance(shape, integer_types):
        shape = (shape,)
    if stype not in (None, 'default'):
        from . import sparse
        return sparse.zeros(stype, shape, ctx=ctx, dtype=dtype)
    return NDArray._from_tensor(torch.zeros(tuple(shape), dtype=to_torch_dtype(dtype) or torch.float32,
                                            device=ctx.torch_device), ctx)


def ones(shape, ctx=None, dtype=None, device=None, out=None, **kwargs):
    if out is not None:
        with torch.no_grad():
            out._data.fill_(1)
        return out
    ctx = ctx or device or current_device()
    if isinstance(shape, integer_types):
        shape = (shape,)
    return NDArray._from_tensor(torch.ones(tuple(shape), dtype=to_torch_dtype(dtype) or torch.float32,
                                           device=ctx.torch_device), ctx)


def full(shape, val, ctx=None, dtype=None, out=None, device=None):
    ctx = ctx or device or current_device()
    if isinstance(shape, integer_types):
        shape = (shape,)
    r = NDArray._from_tensor(torch.full(tuple(shape), val, dtype=to_torch_dtype(dtype) or torch.float32,
                                        device=ctx.torch_device), ctx)
    if out is not None:
        out._data.copy_(r._data)
        return out
    return r


def arange(start, stop=None, step=1.0, repeat=1, infer_range=False, ctx=None, dtype=None, device=None):
    ctx = ctx or device or current_device()
    if stop is None:
        start, stop = 0, start
    t = torch.arange(start, stop, step, dtype=to_torch_dtype(dtype) or torch.float32, device=ctx.torch_device)
    if repeat != 1:
        t = t.repeat_interleave(repeat)
    return NDArray._from_tensor(t, ctx)


def concatenate(arrays, axis=0, always_copy=True):
    return _reg.invoke('Concat', list(arrays), {'dim': axis})


def moveaxis(tensor, source, destination):
    nd_ = tensor._data.dim()
    for v in ([source] if isinstance(source, int) else list(source)) + ([destination] if isinstance(destination, int) else list(destination)):
        if not -nd_ <= int(v) < nd_:
            raise ValueError('Source/destination axis %d is out of bounds for an array with %d dimensions' % (int(v), nd_))
    source = source if isinstance(source, int) else tuple(int(v) for v in source)
    destination = destination if isinstance(destination, int) else tuple(int(v) for v in destination)
    return tensor.__class__._from_tensor(torch.movedim(tensor._data, source, destination), tensor._ctx)


def onehot_encode(indices, out):
    depth = out.shape[1]
    out._data.copy_(torch.nn.functional.one_hot(indices._data.long(), depth).to(out._data.dtype))
    return out


def from_numpy(ndarray, zero_copy=True):
    t = torch.from_numpy(ndarray) if zero_copy else torch.from_numpy(ndarray.copy())
    return NDArray._from_tensor(t, Device('cpu', 0))


def from_dlpack(dlpack):
    return NDArray._from_tensor(torch.utils.dlpack.from_dlpack(dlpack))


def to_dlpack_for_read(data):
    return data.to_dlpack_for_read()


def to_dlpack_for_write(data):
    return data.to_dlpack_for_write()


def imdecode(buf, **kwargs):
    from ..image import imdecode as _imdecode
    return _imdecode(buf, **kwargs)


def waitall():
    """Block until all asynchronous work has finished and surface deferred errors (``MXNDArrayWaitAll``)."""
    from .. import engine
    engine.waitall()


# Fluent methods that simply forward to the operator of the same name with the array as first input
# (python/mxnet/ndarray/ndarray.py:1268-2420 lists them one by one).
_FLUENT = ('reshape_like broadcast_axes broadcast_to broadcast_like pad swapaxes split_v2 argmax_channel abs sign flatten '
           'shape_array size_array expand_dims transpose depth_to_space space_to_depth round rint fix floor ceil trunc sin '
           'cos tan arcsin arccos arctan degrees radians sinh cosh tanh arcsinh arccosh arctanh exp expm1 log log10 log2 '
           'log1p log_sigmoid sqrt rsqrt cbrt rcbrt square reciprocal relu sigmoid softmin squeeze mish').split()


def _make_fluent(name):
    def method(self, *args, **kwargs):
        import sys
        return getattr(sys.modules[__name__.rsplit('.', 1)[0]], name)(self, *args, **kwargs)
    method.__name__ = name
    method.__doc__ = 'Convenience fluent method for :py:func:`%s` with this array as the first input.' % name
    return method


for _name in _FLUENT:
    if _name not in NDArray.__dict__:
        setattr(NDArray, _name, _make_fluent(_name))


# ---- NDArray.drop_grad / slice_assign_scalar (python/mxnet/ndarray/ndarray.py) -------------------------------------
def _drop_grad(self):
    """Free the gradient buffer attached by ``attach_grad`` and stop recording gradients for this array."""
    from .. import autograd
    autograd.mark_variables([self], [None], 'null')


def _slice_assign_scalar(self, value, begin, end, step):
    """``self[begin:end:step] = value`` per axis (None entries keep the whole axis); returns self."""
    index = tuple(slice(b, e, s) for b, e, s in zip(begin, end, step if step is not None else (None,) * len(begin)))
    with torch.no_grad():
        self._data[index] = value
    return self


NDArray.drop_grad = _drop_grad
NDArray.slice_assign_scalar = _slice_assign_scalar


# storage-type codes of include/mxnet/ndarray.h (names scripts import from this module)
_STORAGE_TYPE_UNDEFINED, _STORAGE_TYPE_DEFAULT, _STORAGE_TYPE_ROW_SPARSE, _STORAGE_TYPE_CSR = -1, 0, 1, 2
_STORAGE_TYPE_STR_TO_ID = {'undefined': -1, 'default': 0, 'row_sparse': 1, 'csr': 2}
_STORAGE_TYPE_ID_TO_STR = {v: k for k, v in _STORAGE_TYPE_STR_TO_ID.items()}
py_slice = slice                       # the reference keeps the builtin under this name (its module also defines an operator `slice`)

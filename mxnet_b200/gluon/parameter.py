"""Gluon ``Parameter`` / ``Constant`` (``python/mxnet/gluon/parameter.py``).

A parameter keeps one replica (and one gradient buffer) per device (``parameter.py:355-385``),
supports deferred initialisation when its shape has unknown (0 / -1) dimensions, ``grad_req`` in
{write, add, null}, ``lr_mult``/``wd_mult``, ``cast``, ``reset_device`` and replica averaging for
checkpoints (``_reduce``).  Gradient buffers are owned here and installed as the autograd leaf's
accumulation target, so their addresses stay fixed for the lifetime of the parameter (the fused
KVStore re-homes them once into flat arenas through :meth:`_rebind`).
"""
from __future__ import annotations

import warnings
from collections import OrderedDict

import numpy as np
import torch

from .. import autograd, initializer, _state
from ..base import MXNetError, to_torch_dtype, to_numpy_dtype
from ..device import Device, cpu, current_device
from ..ndarray.ndarray import NDArray
from ..util import is_np_array

__all__ = ['DeferredInitializationError', 'Parameter', 'Constant', 'tensor_types']

tensor_types = (NDArray,)


class DeferredInitializationError(MXNetError):
    """Error for unfinished deferred initialization."""


def _shape_known(shape):
    if shape is None:
        return False
    # in a parameter's stored shape 0 (and -1) always mean "not known yet", under NumPy shape semantics too (the reference's
    # Parameter.shape maps its zeros to -1 there before asking shape_is_known, python/mxnet/gluon/parameter.py)
    return all(s > 0 for s in shape)


class Parameter(object):
    def __init__(self, name='weight', grad_req='write', shape=None, dtype='float32', lr_mult=1.0, wd_mult=1.0,
                 init=None, allow_deferred_init=False, differentiable=True, stype='default', grad_stype='default'):
        self._name = name
        self._var = None
        self._uuid = id(self)
        self._data = None          # OrderedDict[Device, array]
        self._grad = None
        self._ctx_list = None
        self._deferred_init = ()
        self._trainer = None                 # weak reference to the Trainer that updates this parameter
        self._differentiable = differentiable
        self._allow_deferred_init = allow_deferred_init
        self._grad_req = None
        if isinstance(shape, int):
            shape = (shape,)
        self._shape = tuple(shape) if shape is not None else None
        self.dtype = dtype
        self.lr_mult = lr_mult
        self.wd_mult = wd_mult
        self.grad_req = grad_req
        self.init = init
        valid = ('row_sparse', 'csr', 'default')
        assert grad_stype in valid and stype in valid
        self._grad_stype, self._stype = grad_stype, stype
        self._structure_name = None

    def __repr__(self):
        return 'Parameter (shape={shape}, dtype={dtype})'.format(shape=self.shape, dtype=self.dtype)

    # ------------------------------------------------------------------ attributes
    @property
    def name(self):
        return self._structure_name if self._structure_name is not None else self._name

    @property
    def grad_req(self):
        return self._grad_req

    @grad_req.setter
    def grad_req(self, req):
        assert req in ['write', 'add', 'null'], "grad_req must be one of 'write', 'add', or 'null', but got '%s'" % req
        if not self._differentiable:
            req = 'null'
        if self._grad_req == req:
            return
        self._grad_req = req
        if req == 'null' and self._grad is not None:
            self._grad = None
            for arr in self._data.values():
                autograd.mark_variables([arr], [None], 'null')
        elif self._data is not None:
            self._init_grad()

    @property
    def dtype(self):
        return self._dtype

    @dtype.setter
    def dtype(self, dtype):
        d = to_numpy_dtype(to_torch_dtype(dtype))
        self._dtype = d.type if isinstance(d, np.dtype) else d

    @property
    def shape(self):
        if self._shape is None:
            return None
        if _state.state.np_shape:
            return tuple(i if i != 0 else -1 for i in self._shape)
        return self._shape

    @shape.setter
    def shape(self, new_shape):
        if self._shape is None:
            self._shape = tuple(new_shape)
            return
        unknown = (0, -1)
        assert len(self._shape) == len(new_shape) and \
            all(j in unknown or i == j for i, j in zip(new_shape, self._shape)), \
            'Expected shape %s is incompatible with given shape %s for Parameter %s.' % (
                str(new_shape), str(self._shape), self.name)
        self._shape = tuple(new_shape)

    @property
    def stype(self):
        return self._stype

    # ------------------------------------------------------------------ init
    def _array_cls(self):
        if is_np_array():
            from ..numpy.multiarray import ndarray
            return ndarray
        return NDArray

    def _check_and_get(self, arr_dict, ctx):
        if arr_dict is not None:
            if ctx is list:
                return list(arr_dict.values())
            if ctx is None:
                if len(arr_dict) == 1:
                    return next(iter(arr_dict.values()))
                ctx = current_device()
            hit = arr_dict.get(ctx)
            if hit is not None:
                return hit
            raise RuntimeError("Parameter '%s' was not initialized on device %s. It was only initialized on %s." % (
                self.name, str(ctx), str(self._ctx_list)))
        if self._deferred_init:
            raise DeferredInitializationError(
                "Parameter '%s' has not been initialized yet because initialization was deferred. Actual "
                "initialization happens during the first forward pass. Please pass one batch of data through "
                "the network before accessing Parameters. You can also avoid deferred initialization by "
                "specifying in_units, num_features, etc., for network layers." % self.name)
        raise RuntimeError("Parameter '%s' has not been initialized. Note that you should initialize parameters "
                           "and create Trainer with Block.collect_params() instead of Block.params because the "
                           "later does not include Parameters of nested child Blocks" % self.name)

    def initialize(self, init=None, device=None, default_init=initializer.Uniform(), force_reinit=False, ctx=None):
        device = device if device is not None else ctx
        if self._data is not None and not force_reinit:
            warnings.warn("Parameter '%s' is already initialized, ignoring. Set force_reinit=True to re-initialize."
                          % self.name, stacklevel=2)
            return
        self._data = self._grad = None
        if device is None:
            device = [current_device()]
        if isinstance(device, Device):
            device = [device]
        if init is None:
            init = default_init if self.init is None else self.init
        if not _shape_known(self._shape):
            if self._allow_deferred_init:
                self._deferred_init = (init, device, default_init, None)
                return
            raise ValueError("Cannot initialize Parameter '%s' because it has invalid shape: %s." % (
                self.name, str(self._shape)))
        self._deferred_init = (init, device, default_init, None)
        self._finish_deferred_init()

    def _finish_deferred_init(self):
        if not self._deferred_init:
            return
        init, ctx, default_init, data = self._deferred_init
        self._deferred_init = ()
        assert _shape_known(self._shape), \
            "Cannot initialize Parameter '%s' because it has invalid shape: %s. Please specify in_units, " \
            "in_channels, etc for `Block`s." % (self.name, str(self._shape))
        with autograd.pause():
            if data is None:
                cls = self._array_cls()
                host = cls._from_tensor(torch.zeros(self._shape, dtype=torch.float32), cpu(0))
                desc = initializer.InitDesc(self.name, {'__init__': ''}, default_init if isinstance(
                    default_init, initializer.Initializer) else None)
                chosen = init if init is not None else default_init
                if isinstance(chosen, str):
                    chosen = initializer.create(chosen)
                # the initializer chosen for this parameter (its own, else the global one) is applied
                # through _init_weight whatever the name suffix, as the reference does via '__init__'
                if isinstance(chosen, initializer.Initializer):
                    chosen._init_weight(desc, host)
                else:
                    chosen(desc, host)
                data = host
            self._init_impl(data, ctx)

    def _init_impl(self, data, ctx_list):
        self._ctx_list = list(ctx_list)
        cls = self._array_cls()
        td = to_torch_dtype(self.dtype)
        self._data = OrderedDict()
        for c in self._ctx_list:
            t = data._data.detach().to(device=c.torch_device, dtype=td, copy=True)
            arr = cls._from_tensor(t, c)
            arr._ctx = c
            self._data[c] = arr
        self._init_grad()

    def _init_grad(self):
        if self.grad_req == 'null':
            self._grad = None
            return
        self._grad = OrderedDict()
        for c, arr in self._data.items():
            if self._grad_stype != 'default':
                # the gradient buffer carries the asked storage type (dense-backed: autograd writes the dense tensor, the
                # optimizer's lazy update and the key-value store read its non-zero rows)
                from ..ndarray import sparse
                cls = sparse.RowSparseNDArray if self._grad_stype == 'row_sparse' else sparse.CSRNDArray
                g = sparse._tag(torch.zeros_like(arr._data), c, cls, self._grad_stype)
            else:
                g = arr.__class__._from_tensor(torch.zeros_like(arr._data), c)
            g._ctx = c
            self._grad[c] = g
            autograd.mark_variables([arr], [g], self.grad_req)

    def _rebind(self, ctx, data_tensor, grad_tensor):
        """Move one replica (and its gradient) into caller-provided storage of identical shape/dtype
        (views into a flat arena).  Values are preserved; array objects keep their identity."""
        arr = self._data[ctx]
        with torch.no_grad():
            data_tensor.copy_(arr._data)
        arr._data = data_tensor
        if self._grad is not None and grad_tensor is not None:
            g = self._grad[ctx]
            with torch.no_grad():
                grad_tensor.copy_(g._data)
            g._data = grad_tensor
            fresh, last_pass = arr._fresh_grad, arr._grad_pass
            autograd.mark_variables([arr], [g], self.grad_req)
            arr._fresh_grad, arr._grad_pass = fresh, last_pass       # the gradient moved with its history
        from . import block
        block._bump_storage_version()

    def _reduce(self):
        """Average of the replicas on the host (used when saving)."""
        vals = list(self._check_and_get(self._data, list))
        t = vals[0]._data.detach().float().cpu().clone()
        for v in vals[1:]:
            t += v._data.detach().float().cpu()
        t = (t / len(vals)).to(vals[0]._data.dtype)
        return vals[0].__class__._from_tensor(t, cpu(0))

    def _load_init(self, data, ctx, cast_dtype=False, dtype_source='current'):
        if cast_dtype:
            assert dtype_source in ['current', 'saved']
        if self._shape:
            unknown = (0, -1)
            for self_dim, data_dim in zip(self._shape, data.shape):
                assert self_dim in unknown or self_dim == data_dim, \
                    "Failed loading Parameter '%s' from saved params: shape incompatible expected %s vs saved %s" % (
                        self.name, str(self._shape), str(data.shape))
            self._shape = tuple(i if i not in unknown else j for i, j in zip(self._shape, data.shape))
        elif self._shape is None:
            self._shape = tuple(data.shape)
        if self.dtype:
            if cast_dtype and to_torch_dtype(self.dtype) != data._data.dtype:
                if dtype_source == 'current':
                    data = data.astype(self.dtype, copy=False)
                else:
                    self.dtype = data._data.dtype
            else:
                assert to_torch_dtype(self.dtype) == data._data.dtype, \
                    "Failed loading Parameter '%s' from saved params: dtype incompatible expected %s vs saved %s. " \
                    "Set cast_dtype=True to cast the dtype of saved params." % (self.name, str(self.dtype), str(data.dtype))
        if isinstance(ctx, Device):
            ctx = [ctx]
        if self._data is None:
            if self._deferred_init:
                assert ctx is None or set(ctx) == set(self._deferred_init[1]), \
                    "Failed to load Parameter '%s' on %s because it was previous initialized on %s." % (
                        self.name, str(ctx), str(self.list_ctx()))
                ctx = self._deferred_init[1]
            elif ctx is None:
                ctx = [cpu()]
            self._init_impl(data, ctx)
        else:
            assert ctx is None or set(ctx) == set(self.list_ctx()), \
                "Failed to load Parameter '%s' on %s because it was previous initialized on %s." % (
                    self.name, str(ctx), str(self.list_ctx()))
            self.set_data(data)
        self._deferred_init = ()

    # ------------------------------------------------------------------ access
    def data(self, ctx=None, device=None):
        ctx = ctx if ctx is not None else device
        if self._stype != 'default':
            raise RuntimeError("Cannot return a copy of Parameter '%s' on ctx %s via data() because its storage type is %s. "
                               "Please use row_sparse_data() instead." % (self.name, str(ctx), self._stype))
        return self._dense_data(ctx)

    def _dense_data(self, ctx=None):
        arr = self._check_and_get(self._data, ctx)
        want_np = is_np_array()
        if want_np != (arr._kind == 'np'):
            conv = arr.as_np_ndarray() if want_np else arr.as_nd_ndarray()
            conv._hook = arr._hook
            return conv
        return arr

    def list_data(self):
        if self._stype != 'default':
            raise RuntimeError("Cannot return copies of Parameter '%s' on all devices via list_data() because its storage "
                               "type is %s. Please use row_sparse_data() instead." % (self.name, self._stype))
        return list(self._check_and_get(self._data, list))

    def grad(self, ctx=None, device=None):
        ctx = ctx if ctx is not None else device
        if self._data is not None and self._grad is None:
            raise RuntimeError("Cannot get gradient array for Parameter '%s' because grad_req='null'" % self.name)
        return self._check_and_get(self._grad, ctx)

    def list_grad(self):
        if self._data is not None and self._grad is None:
            raise RuntimeError("Cannot get gradient array for Parameter '%s' because grad_req='null'" % self.name)
        return list(self._check_and_get(self._grad, list))

    def list_ctx(self):
        if self._data is None:
            if self._deferred_init:
                return list(self._deferred_init[1])
            raise RuntimeError("Parameter '%s' has not been initialized" % self.name)
        return list(self._ctx_list)

    list_device = list_ctx

    def zero_grad(self):
        if self._grad is None:
            return
        for g in self._grad.values():
            g._data.zero_()

    def set_data(self, data):
        self.shape = data.shape
        if self._data is None:
            assert self._deferred_init, "Parameter '%s' has not been initialized" % self.name
            self._deferred_init = self._deferred_init[:3] + (data,)
            return
        src = data._data if isinstance(data, NDArray) else torch.as_tensor(np.asarray(data))
        with torch.no_grad():
            for arr in self._data.values():
                arr._data.copy_(src.to(arr._data.device))

    def reset_ctx(self, ctx=None, device=None):
        ctx = ctx if ctx is not None else device
        if ctx is None:
            ctx = [current_device()]
        if isinstance(ctx, Device):
            ctx = [ctx]
        if self._data:
            data = self._reduce()
            with autograd.pause():
                self._init_impl(data, ctx)
        elif self._deferred_init:
            init, _, default_init, data = self._deferred_init
            self._deferred_init = (init, ctx, default_init, data)
        else:
            raise ValueError("Cannot reset device for Parameter '%s' because it has not been initialized." % self.name)

    reset_device = reset_ctx

    def cast(self, dtype):
        self.dtype = dtype
        if self._data is None:
            return
        td = to_torch_dtype(dtype)
        with autograd.pause():
            for c, arr in self._data.items():
                arr._data = arr._data.detach().to(td)
            self._init_grad()
        from . import block
        block._bump_storage_version()

    def var(self):
        if self._var is None:
            from .. import symbol
            self._var = symbol.var(self.name, shape=self.shape, dtype=self.dtype, lr_mult=self.lr_mult,
                                   wd_mult=self.wd_mult, init=self.init if isinstance(self.init, str) or self.init is None
                                   else self.init.dumps(), stype=self._stype)
        return self._var

    def _set_trainer(self, trainer):
        """Remember (weakly) the Trainer that updates this parameter; a sparse parameter accepts one Trainer only, because its
        rows are pulled through that Trainer's key-value store."""
        import weakref
        if self._stype != 'default' and self._trainer and trainer and self._trainer() is not trainer:
            raise RuntimeError("Failed to set the trainer for Parameter '%s' because it was already set. More than one "
                               "trainers for a %s Parameter is not supported." % (self.name, self._stype))
        self._trainer = weakref.ref(trainer) if trainer is not None else None

    def row_sparse_data(self, row_id):
        if self._stype != 'row_sparse':
            raise RuntimeError("Cannot return a copy of Parameter %s via row_sparse_data() because its storage "
                               "type is %s. Please use data() instead." % (self.name, self._stype))
        if self._trainer is None or self._trainer() is None:
            raise RuntimeError("Cannot get row_sparse data for Parameter '%s' when no Trainer is created with it." % self.name)
        from ..ndarray import sparse
        return sparse.retain(sparse.cast_storage(self._dense_data(row_id.context), 'row_sparse'), row_id)

    def list_row_sparse_data(self, row_id):
        if self._stype != 'row_sparse':
            raise RuntimeError("Cannot return copies of Parameter '%s' on all devices via list_row_sparse_data() because its "
                               "storage type is %s. Please use data() instead." % (self.name, self._stype))
        if self._trainer is None or self._trainer() is None:
            raise RuntimeError("Cannot get row_sparse data for Parameter '%s' when no Trainer is created with it." % self.name)
        from ..ndarray import sparse
        return [sparse.retain(sparse.cast_storage(arr, 'row_sparse'), row_id.as_in_context(arr.context))
                for arr in self._check_and_get(self._data, list)]


class Constant(Parameter):
    """A parameter that is never updated (``grad_req='null'``), initialised from a given value."""

    def __init__(self, value):
        if not isinstance(value, NDArray):
            from .. import ndarray as nd
            arr = np.asarray(value)
            value = nd.array(arr, dtype=arr.dtype if arr.dtype != np.float64 else 'float32')
        self.value = value

        class Init(initializer.Initializer):
            def _init_weight(self, _, arr):
                arr._data.copy_(value._data.to(arr._data.dtype))
        super().__init__(name='const', grad_req='null', shape=value.shape, dtype=value.dtype, init=Init())

    def __repr__(self):
        return 'Constant (shape={shape}, dtype={dtype})'.format(shape=self.shape, dtype=self.dtype)

    @property
    def grad_req(self):
        return 'null'

    @grad_req.setter
    def grad_req(self, req):
        if req != 'null':
            warnings.warn('Constant parameter "{}" does not support grad_req other than "null", and new value '
                          '"{}" is ignored.'.format(self.name, req))
        self._grad_req = 'null'

"""Executor: a bound Symbol (``python/mxnet/executor.py``, a shim over CachedOp in the reference)."""
import torch

from . import autograd
from .base import MXNetError
from .ndarray.ndarray import NDArray


class Executor(object):
    def __init__(self, sym, ctx, args, args_grad=None, grad_req='write', aux_states=None, group2ctx=None):
        self._symbol = sym
        self._ctx = ctx
        self._group2ctx = dict(group2ctx) if group2ctx else None
        # model parallelism: each operator runs on the context of its `ctx_group` (python/mxnet/symbol/symbol.py bind)
        self._placement = sym._place(ctx, self._group2ctx) if self._group2ctx else None
        self._stats = {'copies': 0}
        arg_names = sym.list_arguments()
        aux_names = sym.list_auxiliary_states()
        if isinstance(args, dict):
            self.arg_dict = dict(args)
        else:
            self.arg_dict = dict(zip(arg_names, args))
        missing = [n for n in arg_names if n not in self.arg_dict]
        if missing:
            raise MXNetError('key `%s` is missing in `args`' % missing[0])
        if aux_states is None:
            aux_states = {}
        self.aux_dict = dict(aux_states) if isinstance(aux_states, dict) else dict(zip(aux_names, aux_states))
        if args_grad is None:
            self.grad_dict = {}
        elif isinstance(args_grad, dict):
            self.grad_dict = dict(args_grad)
        else:
            self.grad_dict = dict(zip(arg_names, args_grad))
        self._grad_req = grad_req if isinstance(grad_req, dict) else {n: grad_req for n in arg_names}
        self.arg_arrays = [self.arg_dict[n] for n in arg_names]
        self.grad_arrays = [self.grad_dict.get(n) for n in arg_names]
        self.aux_arrays = [self.aux_dict[n] for n in aux_names]
        self.outputs = []
        self._out_tensors = None
        self._leafs = None

    @property
    def cross_device_copies(self):
        """Values that crossed contexts in the last forward pass of a model-parallel executor."""
        return self._stats['copies']

    @property
    def mirrored_nodes(self):
        """Operators of the last training forward pass whose results are recomputed in backward (backward mirroring:
        ``MXNET_BACKWARD_DO_MIRROR`` / ``MXNET_MEMORY_OPT`` or the ``force_mirroring`` attribute)."""
        return self._stats.get('mirrored_nodes', 0)

    @property
    def output_dict(self):
        return dict(zip(self._symbol.list_outputs(), self.outputs))

    def forward(self, is_train=False, **kwargs):
        for k, v in kwargs.items():
            if k not in self.arg_dict:
                raise MXNetError('unknown argument %s' % k)
            if isinstance(v, NDArray):
                self.arg_dict[k]._data.copy_(v._data)
            else:
                self.arg_dict[k][:] = v
        feed, leafs = {}, {}
        for n, a in self.arg_dict.items():
            t = a._data.detach()
            # an executor bound with gradient buffers records every forward; ``is_train`` only picks the mode of dropout /
            # batch norm (python/mxnet/executor.py:128 in the reference)
            if n in self.grad_dict and self.grad_dict[n] is not None and self._grad_req.get(n, 'write') != 'null' \
                    and t.dtype.is_floating_point:
                t = t.requires_grad_(True)
                leafs[n] = t
            feed[n] = t
        for n, a in self.aux_dict.items():
            feed[n] = a._data
        with autograd.record(train_mode=is_train) if (is_train or leafs) else autograd.pause(train_mode=False):
            if is_train or leafs:
                with torch.enable_grad():
                    outs = self._symbol._run(feed, placement=self._placement, stats=self._stats)
            else:
                with torch.no_grad():
                    outs = self._symbol._run(feed, placement=self._placement, stats=self._stats)
        self._out_tensors, self._leafs = outs, leafs
        cls = type(self.arg_arrays[0]) if self.arg_arrays else NDArray
        self.outputs = [cls._from_tensor(o.detach()) for o in outs]
        return self.outputs

    def backward(self, out_grads=None, is_train=True):
        if self._out_tensors is None:
            raise MXNetError('forward(is_train=True) must be called before backward')
        if out_grads is None:
            gouts = [torch.ones_like(o) for o in self._out_tensors]
        else:
            if isinstance(out_grads, NDArray):
                out_grads = [out_grads]
            gouts = [g._data for g in out_grads]
        names = list(self._leafs.keys())
        heads = [(o, g) for o, g in zip(self._out_tensors, gouts) if o.requires_grad]
        if not heads:
            return
        grads = torch.autograd.grad([h[0] for h in heads], [self._leafs[n] for n in names], [h[1] for h in heads],
                                    allow_unused=True)
        for n, g in zip(names, grads):
            buf = self.grad_dict[n]._data
            if g is None:
                if self._grad_req.get(n, 'write') != 'add':
                    buf.zero_()
                continue
            if self._grad_req.get(n, 'write') == 'add':
                buf.add_(g)
            else:
                buf.copy_(g)
        for n in names:
            self.arg_dict[n]._data.requires_grad_(False)

    def copy_params_from(self, arg_params, aux_params=None, allow_extra_params=False):
        for name, array in arg_params.items():
            if name in self.arg_dict:
                array.copyto(self.arg_dict[name])
            elif not allow_extra_params:
                raise ValueError('Find name "%s" that is not in the arguments' % name)
        if aux_params:
            for name, array in aux_params.items():
                if name in self.aux_dict:
                    array.copyto(self.aux_dict[name])
                elif not allow_extra_params:
                    raise ValueError('Find name %s that is not in the auxiliary states' % name)

    def reshape(self, partial_shaping=False, allow_up_sizing=False, **kwargs):
        from . import ndarray as nd
        arg_shapes, _, aux_shapes = self._symbol.infer_shape(**kwargs)
        new_args = {}
        for n, s in zip(self._symbol.list_arguments(), arg_shapes):
            old = self.arg_dict[n]
            new_args[n] = old if tuple(old.shape) == tuple(s) else nd.zeros(s, ctx=self._ctx, dtype=old.dtype)
        new_grads = {n: nd.zeros(new_args[n].shape, ctx=self._ctx, dtype=new_args[n].dtype) for n in self.grad_dict} \
            if self.grad_dict else None
        return Executor(self._symbol, self._ctx, new_args, new_grads, self._grad_req, self.aux_dict, group2ctx=self._group2ctx)

    def get_optimized_symbol(self):
        """The graph as it runs: with pointwise groups fused once the executor has run on a GPU, else the bound Symbol."""
        fused = getattr(self._symbol, '_fused', None)
        return fused if fused else self._symbol

    def debug_str(self):
        return self._symbol.debug_str()

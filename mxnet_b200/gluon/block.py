"""Gluon ``Block`` / ``HybridBlock`` / ``SymbolBlock`` (``python/mxnet/gluon/block.py``).

``hybridize()`` keeps the reference's contract — trace the Python ``forward`` once into a Symbol
(deferred compute, ``block.py:1107-1129``), cache an executable for repeated calls, ``export`` a
``-symbol.json`` + ``-%04d.params`` pair (``:1506-1581``) that ``SymbolBlock.imports`` reloads —
but the cached executable is a pair of captured CUDA graphs (forward and backward) replayed on
static buffers when ``static_alloc=True, static_shape=True`` on a GPU (``gluon/cached_op.py``),
instead of a node-by-node graph executor.
"""
from __future__ import annotations

import copy
import re
import warnings
from collections import OrderedDict

import numpy as np
import torch

from .. import _state, autograd, env
from ..base import MXNetError
from ..device import Device, cpu, current_device
from ..ndarray.ndarray import NDArray
from ..util import is_np_array
from .parameter import Parameter, Constant, DeferredInitializationError

__all__ = ['Block', 'HybridBlock', 'SymbolBlock']

_storage_version = [0]


def _bump_storage_version():
    """Parameter storage moved (cast, arena re-homing): cached graphs must be re-captured."""
    _storage_version[0] += 1


def _flatten(args, fmt_name):
    if isinstance(args, NDArray):
        return [args], int(0)
    if args is None:
        return [None], int(-1)
    if not isinstance(args, (list, tuple)):
        return [args], int(-2)
    flat, fmts = [], []
    for i in args:
        arg, fmt = _flatten(i, fmt_name)
        flat.extend(arg)
        fmts.append(fmt)
    return flat, fmts


def _regroup(args, fmt):
    if isinstance(fmt, int):
        if fmt in (0, -1, -2):
            return args[0], args[1:]
        return args[:fmt], args[fmt:]
    ret = []
    for i in fmt:
        res, args = _regroup(args, i)
        ret.append(res)
    return ret, args


class _HookHandle(object):
    def __init__(self, hooks, key):
        self._hooks, self._key = hooks, key

    def detach(self):
        self._hooks.pop(self._key, None)


class Block(object):
    """Base class of all layers and models."""

    def __init__(self):
        self._children = OrderedDict()
        self._reg_params = {}
        self._forward_hooks = OrderedDict()
        self._forward_pre_hooks = OrderedDict()
        self._hook_id = 0

    def __repr__(self):
        s = '{name}(\n{modstr}\n)'
        modstr = '\n'.join(['  ({key}): {block}'.format(key=key, block=re.sub('\n', '\n  ', repr(block)))
                            for key, block in self._children.items()])
        return s.format(name=self.__class__.__name__, modstr=modstr)

    def __setattr__(self, name, value):
        if hasattr(self, name):
            existing = getattr(self, name)
            if isinstance(existing, (Parameter, Block)) and not isinstance(value, type(existing)) and value is not None:
                raise TypeError('Changing attribute type for {name} from {type1} to {type2} is not allowed.'.format(
                    name=name, type1=type(existing), type2=type(value)))
        if isinstance(value, Block):
            self.register_child(value, name)
        elif isinstance(value, Parameter):
            self._reg_params[name] = value
        super().__setattr__(name, value)

    def _check_container_with_block(self):
        children = set(self._children.values())

        def _find(data):
            if isinstance(data, (list, tuple)):
                return any(_find(e) for e in data)
            if isinstance(data, dict):
                return any(_find(v) for v in data.values())
            return isinstance(data, Block) and data not in children
        for k, v in self.__dict__.items():
            if isinstance(v, (list, tuple, dict)) and not (k.startswith('__') or k == '_children'):
                if _find(v):
                    warnings.warn('"{name}" is an unregistered container with Blocks. Note that Blocks inside the '
                                  'list, tuple or dict will not be registered automatically. Make sure to register '
                                  'them using register_child() or switching to nn.Sequential/nn.HybridSequential '
                                  'instead. '.format(name=self.__class__.__name__ + '.' + k), stacklevel=3)

    # ------------------------------------------------------------------ parameters
    @property
    def params(self):
        return self._reg_params

    def collect_params(self, select=None):
        self._check_container_with_block()
        ret = self._collect_params_with_prefix()
        if select is not None:
            pattern = re.compile(select)
            ret = {k: v for k, v in ret.items() if pattern.match(k)}
        for name, p in ret.items():
            p._structure_name = name
        return ret

    def _collect_params_with_prefix(self, prefix='', select=None):
        if prefix:
            prefix += '.'
        ret = OrderedDict((prefix + key, val) for key, val in self._reg_params.items())
        for name, child in self._children.items():
            ret.update(child._collect_params_with_prefix(prefix + name))
        return ret

    def save_parameters(self, filename, deduplicate=False):
        """Save parameters: ``.npz`` in NumPy mode, legacy binary container otherwise (``block.py:342-378``)."""
        params = self._collect_params_with_prefix()
        if deduplicate:
            reverse = {}
            for k, v in params.items():
                reverse.setdefault(id(v), k)
            params = {k: v for k, v in params.items() if reverse[id(v)] == k}
        arg_dict = {key: val._reduce() for key, val in params.items()}
        if is_np_array():
            from .. import numpy_extension as npx
            npx.savez(filename, **arg_dict)
        else:
            from ..ndarray.utils import save
            save(filename, arg_dict)

    def load_parameters(self, filename, device=None, allow_missing=False, ignore_extra=False, cast_dtype=False,
                        dtype_source='current', ctx=None):
        device = device if device is not None else ctx
        from ..ndarray.utils import load
        cls = None
        if is_np_array():
            from ..numpy.multiarray import ndarray as cls
        loaded = load(filename, cls=cls)
        if isinstance(loaded, list):
            raise MXNetError('%s does not contain named parameters' % filename)
        self.load_dict(loaded, device, allow_missing, ignore_extra, cast_dtype, dtype_source)

    def load_dict(self, param_dict, device=None, allow_missing=False, ignore_extra=False, cast_dtype=False,
                  dtype_source='current', ctx=None):
        device = device if device is not None else ctx
        if isinstance(param_dict, dict):
            param_dict = {(k[4:] if k.startswith('arg:') or k.startswith('aux:') else k): v for k, v in param_dict.items()}
        params = self.collect_params()
        if isinstance(param_dict, dict):
            # blocks may translate foreign parameter layouts of their own subtree (the fused recurrent layers accept the single
            # flat `rnn_param` vector that later versions of the reference save)
            def _translate(block, prefix):
                hook = getattr(block, '_translate_loaded', None)
                if hook is not None:
                    hook(prefix, param_dict)
                for cname, child in block._children.items():
                    _translate(child, prefix + cname + '.')
            _translate(self, '')
        if not allow_missing:
            params_inv = {}
            for k, v in params.items():
                params_inv.setdefault(id(v), []).append(k)
            for name, p in params.items():
                assert any(alias in param_dict for alias in params_inv[id(p)]), \
                    "Parameter '%s' is missing in '%s', which contains parameters: %s. Set allow_missing=True to " \
                    "ignore missing parameters." % (name, 'param_dict', _brief_print_list(param_dict.keys()))
        if device is None:
            device = _guess_devices(params)
        for name in param_dict:
            if name not in params:
                assert ignore_extra, \
                    "Parameter '%s' loaded from '%s' is not present in Dict, which contains parameters %s. Set " \
                    "ignore_extra=True to ignore. " % (name, 'param_dict', _brief_print_list(params.keys()))
                continue
            params[name]._load_init(param_dict[name], device, cast_dtype=cast_dtype, dtype_source=dtype_source)

    # ------------------------------------------------------------------ structure
    def register_child(self, block, name=None):
        if name is None:
            name = str(len(self._children))
        self._children[name] = block

    def register_forward_pre_hook(self, hook):
        self._hook_id += 1
        self._forward_pre_hooks[self._hook_id] = hook
        return _HookHandle(self._forward_pre_hooks, self._hook_id)

    def register_forward_hook(self, hook):
        self._hook_id += 1
        self._forward_hooks[self._hook_id] = hook
        return _HookHandle(self._forward_hooks, self._hook_id)

    def apply(self, fn):
        for cld in self._children.values():
            cld.apply(fn)
        fn(self)
        return self

    def initialize(self, init=None, device=None, verbose=False, force_reinit=False, ctx=None):
        from .. import initializer
        device = device if device is not None else ctx
        if init is None:
            init = initializer.Uniform()
        params = self.collect_params()
        if verbose and hasattr(init, 'set_verbosity'):
            init.set_verbosity(verbose=verbose)
        for v in params.values():
            v.initialize(None, device, init, force_reinit=force_reinit)

    def hybridize(self, active=True, **kwargs):
        for cld in self._children.values():
            cld.hybridize(active, **kwargs)

    def cast(self, dtype):
        for child in self._children.values():
            child.cast(dtype)
        for p in self._reg_params.values():
            p.cast(dtype)

    def zero_grad(self):
        for p in self.collect_params().values():
            p.zero_grad()

    def reset_ctx(self, ctx):
        for p in self.collect_params().values():
            p.reset_ctx(ctx)

    reset_device = reset_ctx

    def setattr(self, name, value):
        for p in self.collect_params().values():
            setattr(p, name, value)

    def share_parameters(self, shared):
        if shared is None:
            return self
        if not isinstance(shared, (dict, OrderedDict)):
            raise ValueError("'shared' should be in type of Dict. Get type {}!".format(type(shared)))
        shared_set = set(shared.keys())
        self._shared_parameters(shared, shared_set)
        if shared_set:
            for name in shared_set:
                warnings.warn("Parameter name {} is not in the current model!".format(name))
        return self

    def _shared_parameters(self, shared, shared_set, prefix=''):
        if prefix:
            prefix += '.'
        for name in list(self._reg_params):
            key = prefix + name
            if shared.get(key) is not None:
                setattr(self, name, shared[key])
                self._reg_params[name] = shared[key]
                shared_set.discard(key)
        for name, child in self._children.items():
            child._shared_parameters(shared, shared_set, prefix + name)

    # ------------------------------------------------------------------ call
    def __call__(self, *args, **kwargs):
        for hook in self._forward_pre_hooks.values():
            hook(self, args)
        out = self.forward(*args, **kwargs)
        for hook in self._forward_hooks.values():
            hook(self, args, out)
        return out

    def forward(self, *args):
        raise NotImplementedError

    def register_op_hook(self, callback, monitor_all=False):
        for cld in self._children.values():
            cld.register_op_hook(callback, monitor_all)

    def summary(self, *inputs):
        """Print a per-layer table of output shapes and parameter counts (``block.py:894``)."""
        summary = OrderedDict()
        seen = set()
        hooks = []

        def _no_active(block):
            assert not (isinstance(block, HybridBlock) and block._active), \
                '"{}" must not be hybridized to print summary.'.format(type(block).__name__)
        self.apply(_no_active)

        def _get_shape_str(args):
            flat, _ = _flatten(args, 'output')
            shapes = [x.shape if isinstance(x, NDArray) else x for x in flat]
            return str(shapes[0]) if len(shapes) == 1 else str(shapes)

        def _register(block):
            def _hook(blk, _, outputs):
                class_name = blk.__class__.__name__
                key = '%s-%i' % (class_name, len(summary) + 1)
                summary[key] = OrderedDict()
                summary[key]['output_shape'] = _get_shape_str(outputs)
                params = 0
                summary[key]['trainable'] = summary[key]['shared'] = 0
                for p in blk._reg_params.values():
                    n = int(np.prod(p.shape)) if p.shape else 0
                    params += n
                    summary[key]['trainable'] += 0 if p.grad_req == 'null' else n
                    if id(p) in seen:
                        summary[key]['shared'] += n
                    else:
                        seen.add(id(p))
                summary[key]['n_params'] = params
            hooks.append(block.register_forward_hook(_hook))
        self.apply(_register)
        try:
            self(*inputs)
            line = '{:>20}  {:>42} {:>15}'
            print('-' * 80)
            print(line.format('Layer (type)', 'Output Shape', 'Param #'))
            print('=' * 80)
            total = trainable = shared = 0
            for layer, info in summary.items():
                print(line.format(layer, info['output_shape'], info['n_params']))
                total += info['n_params']
                trainable += info['trainable']
                shared += info['shared']
            print('=' * 80)
            print('Parameters in forward computation graph, duplicate included')
            print('   Total params: ' + str(total))
            print('   Trainable params: ' + str(trainable))
            print('   Non-trainable params: ' + str(total - trainable))
            print('Shared params in forward computation graph: ' + str(shared))
            print('Unique parameters in model: ' + str(total - shared))
            print('-' * 80)
        finally:
            for h in hooks:
                h.detach()


def _brief_print_list(lst, limit=7):
    lst = list(lst)
    if len(lst) > limit:
        return _brief_print_list(lst[:limit // 2], limit) + ', ..., ' + _brief_print_list(lst[-limit // 2:], limit)
    return ', '.join(["'%s'" % str(i) for i in lst])


def _guess_devices(params):
    for p in params.values():
        try:
            return p.list_ctx()
        except RuntimeError:
            continue
    return [current_device()]


class HybridBlock(Block):
    """A Block whose forward can be traced and cached (``hybridize``) and exported."""

    def __init__(self):
        super().__init__()
        self._active = False
        self._flags = {}
        self._cached_graph = None     # (input symbols, output symbol) from the trace
        self._cached_op = None
        self._in_format = None
        self._out_format = None
        self._backend = None
        self._backend_opts = {}
        self._monitor = None
        self._last_args = None

    def __setattr__(self, name, value):
        super().__setattr__(name, value)
        if isinstance(value, HybridBlock):
            self._clear_cached_op()

    def register_child(self, block, name=None):
        if not isinstance(block, HybridBlock):
            raise ValueError('Children of HybridBlock must also be HybridBlock, but %s has type %s. If you are using '
                             'Sequential, please try HybridSequential instead.' % (str(block), str(type(block))))
        super().register_child(block, name)
        self._clear_cached_op()

    def _clear_cached_op(self):
        self._cached_graph = None
        self._cached_op = None
        self._partitioned = None

    def hybridize(self, active=True, partition_if_dynamic=True, static_alloc=False, static_shape=False,
                  inline_limit=2, forward_bulk_size=None, backward_bulk_size=None, backend=None, backend_opts=None,
                  **kwargs):
        self._active = active
        self._flags = {'static_alloc': static_alloc, 'static_shape': static_shape, 'inline_limit': inline_limit,
                       'forward_bulk_size': forward_bulk_size, 'backward_bulk_size': backward_bulk_size}
        self._backend = backend
        self._backend_opts = backend_opts or {}
        self._clear_cached_op()
        # children run inside the parent's cached graph; they stay inactive themselves
        super().hybridize(False, **kwargs)

    def optimize_for(self, x, *args, backend=None, clear=False, partition_if_dynamic=True, static_alloc=False,
                     static_shape=False, inline_limit=2, forward_bulk_size=None, backward_bulk_size=None,
                     backend_opts=None, **kwargs):
        self.hybridize(True, partition_if_dynamic, static_alloc, static_shape, inline_limit, forward_bulk_size,
                       backward_bulk_size, backend, backend_opts or kwargs)
        return self(x, *args)

    def cast(self, dtype):
        self._clear_cached_op()
        super().cast(dtype)

    def infer_shape(self, *args):
        """Set parameter shapes from the inputs.  Layers with deferred-shape parameters override this."""
        raise NotImplementedError('%s has parameters with unknown shape; implement infer_shape' % type(self).__name__)

    def infer_type(self, *args):
        pass

    def _deferred_infer_shape(self, *args):
        try:
            self.infer_shape(*args)
        except Exception as e:
            raise ValueError('Deferred initialization failed because shape cannot be inferred. {}'.format(e))

    def _call_forward(self, *args, **kwargs):
        try:
            return self.forward(*args, **kwargs)
        except DeferredInitializationError:
            self._deferred_infer_shape(*args)
            for p in self._reg_params.values():
                p._finish_deferred_init()
            return self.forward(*args, **kwargs)

    def __call__(self, *args, **kwargs):
        for hook in self._forward_pre_hooks.values():
            hook(self, args)
        if self._active and not kwargs and _state.state.tracer is None:
            out = self._call_cached_op(*args)
        else:
            out = self._call_forward(*args, **kwargs)
        for hook in self._forward_hooks.values():
            hook(self, args, out)
        return out

    # ------------------------------------------------------------------ tracing / caching
    def _trace(self, *args):
        """Run ``forward`` once under deferred compute (inference mode, nothing is mutated) and keep
        (input symbols, output symbol).  Deferred parameter shapes must be resolved before."""
        from .. import _deferred_compute as dc
        from .. import symbol as sym
        flat_args, self._in_format = _flatten(args, 'input')
        params = self.collect_params()
        arrays = [a for a in flat_args if isinstance(a, NDArray)]
        names = ['data'] if len(arrays) == 1 else ['data%d' % i for i in range(len(arrays))]
        inputs = [sym.var(n) for n in names]
        with dc.context() as tracer:
            for a, v in zip(arrays, inputs):
                tracer.set_variable(a, v)
            ctx = arrays[0]._ctx if arrays else current_device()
            for name, p in params.items():
                if p._data is None:
                    continue
                arr = p._data.get(ctx)
                if arr is None:
                    arr = next(iter(p._data.values()))
                tracer.set_variable(arr, sym.var(name))
            with autograd.pause(train_mode=False):
                out = self.forward(*args)
            flat_out, self._out_format = _flatten(out, 'output')
            out_sym = tracer.get_symbol([o for o in flat_out if isinstance(o, NDArray)])
        self._cached_graph = (inputs, out_sym)
        # arrays the forward made itself (a zero begin state, a lookup table): leaves of the graph that are neither inputs
        # nor parameters; export writes them beside the parameters
        self._trace_constants = dict(tracer.constants)
        return out

    def _call_cached_op(self, *args):
        from .cached_op import CachedOp
        self._last_args = args
        if self._cached_op is None:
            # first call: finish deferred initialisation eagerly, then build the executor
            out = self._call_forward(*args)
            self._cached_op = CachedOp(self, self._flags)
            return out
        if self._backend not in (None, '', 'default'):
            return self._call_partitioned(*args)
        from ..symbol import layout as _layout
        if _layout.get_optimize_layout():
            # layout management is on (amp.init(layout_optimization=True) / set_optimize_layout): run the traced graph after
            # the pass that moves its convolutional trunk to NHWC (src/imperative/cached_op.h:213 in the reference)
            return self._cached_op(*args, graph_forward=self._layout_forward, graph_tag='optimize_layout')
        return self._cached_op(*args)

    def _layout_forward(self, *args):
        return self._call_partitioned(*args, backend='optimize_layout')

    def _call_partitioned(self, *args, backend=None):
        """``hybridize(backend=...)`` / ``optimize_for``: run the traced graph after the backend's graph pass
        (``HybridBlock._build_cache`` with ``MXOptimizeForBackend`` in the reference, ``python/mxnet/gluon/block.py``)."""
        flat, in_format = _flatten(args, 'input')
        if self._cached_graph is None or in_format != self._in_format:
            self._trace(*args)
            self._partitioned = None
        if backend is not None and getattr(self, '_partitioned_by', None) != backend:
            self._partitioned = None
        if getattr(self, '_partitioned', None) is None:
            if backend is not None:
                self._partitioned = self._cached_graph[1].optimize_for(backend)
                self._partitioned_by = backend
            else:
                self._partitioned = self._cached_graph[1].optimize_for(self._backend, **self._backend_opts)
                self._partitioned_by = None
        inputs, _ = self._cached_graph
        arrays = [a for a in flat if isinstance(a, NDArray)]
        ctx = arrays[0]._ctx
        feed = {v.name: a._data for v, a in zip(inputs, arrays)}
        needed = set(self._partitioned.list_inputs())
        for name, p in self.collect_params().items():
            if name in needed:
                feed[name] = p.data(ctx)._data
        for name, value in (getattr(self, '_trace_constants', None) or {}).items():
            if name in needed:
                feed[name] = value._data.to(arrays[0]._data.device)
        if _state.state.recording:
            with torch.enable_grad():
                outs = self._partitioned._run(feed)
        else:
            with torch.no_grad():
                outs = self._partitioned._run(feed)
        res = [arrays[0].__class__._from_tensor(o, ctx) for o in outs]
        return _regroup(res, self._out_format)[0]

    def export(self, path, epoch=0, remove_amp_cast=True):
        """Write ``path-symbol.json`` and ``path-%04d.params`` (``arg:``/``aux:`` prefixes)."""
        if self._cached_graph is None:
            if self._last_args is None:
                raise RuntimeError('Please first call block.hybridize() and then run forward with this block at '
                                   'least once before calling export.')
            self._trace(*self._last_args)
        _, sym = self._cached_graph
        if remove_amp_cast:
            sym = sym.remove_amp_cast()
        sym_file = '%s-symbol.json' % path
        sym.save(sym_file)
        arg_names = set(sym.list_arguments())
        aux_names = set(sym.list_auxiliary_states())
        arg_dict = {}
        for name, p in self.collect_params().items():
            if name in arg_names:
                arg_dict['arg:%s' % name] = p._reduce().as_nd_ndarray()
            elif name in aux_names:
                arg_dict['aux:%s' % name] = p._reduce().as_nd_ndarray()
        for name, value in (getattr(self, '_trace_constants', None) or {}).items():
            if name in arg_names:
                arg_dict['arg:%s' % name] = value.as_nd_ndarray()
        params_file = None
        if arg_dict:
            params_file = '%s-%04d.params' % (path, epoch)
            from ..ndarray.utils import save
            prev = _state.state.np_shape
            _state.state.np_shape = False
            try:
                save(params_file, arg_dict)
            finally:
                _state.state.np_shape = prev
        return sym_file, params_file

    def forward(self, x, *args):
        raise NotImplementedError

    def register_op_hook(self, callback, monitor_all=False):
        self._monitor = (callback, monitor_all)
        super().register_op_hook(callback, monitor_all)


def _remember_args(block, args):
    block._last_args = args


class SymbolBlock(HybridBlock):
    """Run a Symbol as a Block (``block.py:1600-1800``)."""

    @staticmethod
    def imports(symbol_file, input_names, param_file=None, device=None, allow_missing=False, ignore_extra=False,
                ctx=None):
        from .. import symbol as sym_mod
        device = device if device is not None else ctx
        sym = sym_mod.load(symbol_file)
        if isinstance(input_names, str):
            input_names = [input_names]
        if param_file is None:
            inputs = [sym_mod.var(i, dtype='float32') for i in input_names]
        else:
            inputs = [sym_mod.var(i).as_np_ndarray() if is_np_array() else sym_mod.var(i) for i in input_names]
        ret = SymbolBlock(sym, inputs)
        if param_file is not None:
            ret.load_parameters(param_file, device, allow_missing, ignore_extra, True, 'saved')
        return ret

    def __init__(self, outputs, inputs, params=None):
        super().__init__()
        from .. import symbol as sym_mod
        if isinstance(inputs, sym_mod.Symbol) and len(inputs.list_outputs()) == 1:
            inputs = [inputs]
        if isinstance(outputs, (list, tuple)):
            outputs = outputs[0] if len(outputs) == 1 else sym_mod.Group(outputs)
        self._symbol = outputs
        self._input_names = [i.name for i in inputs]
        arg_names = outputs.list_arguments()
        aux_names = outputs.list_auxiliary_states()
        known = set(self._input_names)
        attrs = outputs.attr_dict()
        for name in arg_names + aux_names:
            if name in known:
                continue
            is_aux = name in aux_names
            if params is not None and name in params:
                p = params[name]
            else:
                p = Parameter(name, grad_req='null' if is_aux else 'write', allow_deferred_init=True,
                              differentiable=not is_aux)
                a = attrs.get(name, {})
                if '__shape__' in a:
                    from ..symbol.symbol import _parse_attr
                    shp = _parse_attr(a['__shape__'])
                    if shp:
                        p._shape = tuple(shp)
            p._structure_name = name
            self._reg_params[name] = p
        self._cached_graph = (inputs, outputs)

    def _collect_params_with_prefix(self, prefix='', select=None):
        return OrderedDict(self._reg_params)

    def infer_shape(self, *args):
        shapes = {n: a.shape for n, a in zip(self._input_names, args)}
        arg_shapes, _, aux_shapes = self._symbol.infer_shape(**shapes)
        if arg_shapes is None:
            raise MXNetError('cannot infer parameter shapes of SymbolBlock')
        sdict = dict(zip(self._symbol.list_arguments(), arg_shapes))
        sdict.update(zip(self._symbol.list_auxiliary_states(), aux_shapes))
        for name, p in self._reg_params.items():
            if name in sdict and sdict[name] is not None:
                p._shape = tuple(sdict[name])

    def forward(self, x, *args):
        arrays = [x] + list(args)
        ctx = x._ctx
        feed = {n: a._data for n, a in zip(self._input_names, arrays)}
        for name, p in self._reg_params.items():
            feed[name] = p.data(ctx)._data
        rec = _state.state.recording
        if rec:
            with torch.enable_grad():
                outs = self._symbol._run(feed)
        else:
            with torch.no_grad():
                outs = self._symbol._run(feed)
        res = [x.__class__._from_tensor(o, ctx) for o in outs]
        return res[0] if len(res) == 1 else res

    def __call__(self, *args, **kwargs):
        for hook in self._forward_pre_hooks.values():
            hook(self, args)
        out = self._call_forward(*args)
        for hook in self._forward_hooks.values():
            hook(self, args, out)
        return out

    def _clear_cached_op(self):
        tmp = self._cached_graph
        super()._clear_cached_op()
        self._cached_graph = tmp

    def cast(self, dtype):
        self._clear_cached_op()
        super().cast(dtype)

    def reset_ctx(self, ctx):
        for p in self._reg_params.values():
            p.reset_ctx(ctx)


# ---- optimisation constraints (HybridBlock.OptConstraint, python/mxnet/gluon/block.py:1048): a scope in which
# graph-level optimisations are held back; the one flag that exists switches the AMP casts off.
import enum as _enum


class _OptConstraint(object):
    class Flag(_enum.Flag):
        DisableAMP = _enum.auto()

    def __init__(self, flag):
        self.flag = flag
        self.enter_state = None

    def __enter__(self):
        self.enter_state = get_optimization_constraints()
        set_optimization_constraints(self.enter_state | self.flag)

    def __exit__(self, ptype, value, trace):
        set_optimization_constraints(self.enter_state)

    @staticmethod
    def disable_all():
        flag = _OptConstraint.Flag(0)
        for f in _OptConstraint.Flag:
            flag |= f
        return _OptConstraint(flag)

    @staticmethod
    def disable_amp():
        return _OptConstraint(_OptConstraint.Flag.DisableAMP)


HybridBlock.OptConstraint = _OptConstraint


def set_optimization_constraints(state):
    """Set the current thread's optimisation constraints; returns the previous ones."""
    prev = _OptConstraint.Flag(_state.state.opt_constraints)
    _state.state.opt_constraints = int(state.value)
    return prev


def get_optimization_constraints():
    return _OptConstraint.Flag(_state.state.opt_constraints)


# ---- Block.save / Block.load (python/mxnet/gluon/block.py:579-700): configuration + parameters of a constructed model
def _block_save(self, prefix):
    """Write ``<prefix>-model.json`` (per block, in construction order: its parameter names, and for hybridized blocks the
    traced graph with its input / output formats) and ``<prefix>-model.params``."""
    import json
    model = {}

    def visit(blk, structure, index=0):
        mdl = {}
        structure[type(blk).__name__.lower() + str(index)] = mdl
        index += 1
        if isinstance(blk, HybridBlock):
            graph = getattr(blk, '_cached_graph', None)
            if not graph and blk._active and getattr(blk, '_last_args', None) is not None:
                blk._trace(*blk._last_args)          # hybridized and called, but not traced yet
                graph = blk._cached_graph
            if graph:
                inputs, out = graph
                mdl.update(in_format=blk._in_format, out_format=blk._out_format, inputs=[s.tojson() for s in inputs],
                           symbol=out.tojson(), hybridized=True)
            else:
                mdl['hybridized'] = False
        mdl['params'] = {name: name for name in blk._reg_params}
        for child in blk._children.values():
            index = visit(child, mdl, index)
        return index
    visit(self, model)
    with open(prefix + '-model.json', 'w') as fp:
        json.dump(model, fp)
    self.save_parameters(prefix + '-model.params')


def _block_load(self, prefix):
    """Restore what :meth:`save` wrote into a model that was constructed the same way (same blocks in the same order):
    traced graphs and hybridization state per block, then the parameters."""
    import json
    from ..symbol import fromjson
    with open(prefix + '-model.json') as fp:
        model = json.load(fp)

    def visit(blk, structure, index=0):
        key = type(blk).__name__.lower() + str(index)
        if key not in structure:
            raise ValueError('the saved model has no block %s here: the model must be constructed exactly as when it was saved' % key)
        mdl = structure[key]
        index += 1
        if isinstance(blk, HybridBlock) and mdl.get('hybridized'):
            blk._in_format, blk._out_format = mdl['in_format'], mdl['out_format']
            blk._cached_graph = ([fromjson(s) for s in mdl['inputs']], fromjson(mdl['symbol']))
            blk._active = True
        missing = [p for p in mdl.get('params', {}) if p not in blk._reg_params]
        if missing:
            raise ValueError('block %s lacks the saved parameters %s' % (key, missing))
        for child in blk._children.values():
            index = visit(child, mdl, index)
        return index
    visit(self, model)
    self.load_parameters(prefix + '-model.params')


Block.save = _block_save
Block.load = _block_load


def _generate_arg_names(self, arg_num):
    """Names of the traced graph's data inputs: ``data`` for one argument, else ``data0``, ``data1`` ..."""
    return ['data'] if arg_num == 1 else ['data%d' % i for i in range(arg_num)]


HybridBlock.generate_arg_names = _generate_arg_names

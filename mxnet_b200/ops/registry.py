"""Operator registry and the single imperative entry point :func:`invoke`.

The reference registers ~950 operator names with nnvm (``NNVM_REGISTER_OP`` …
``include/mxnet/op_attr_types.h:215-382``) and funnels every call through
``Imperative::Invoke`` (``src/imperative/imperative.cc:107-139``).  Here an operator is a Python
callable over ``torch.Tensor`` arguments: array inputs first (by declared name), attributes as
keyword arguments.  :func:`invoke` is the one place where

* array wrappers are unwrapped / results wrapped (``mx.nd.NDArray`` or ``mx.np.ndarray``),
* the autograd recording flag is mapped onto torch's grad mode,
* the AMP cast policy, the profiler and op monitors hook in,
* deferred-compute tracing records a graph node (``Imperative::RecordDeferredCompute``,
  ``imperative.cc:336-382``) so ``HybridBlock.export`` can emit ``-symbol.json``.

Attribute values are kept as Python objects at run time and are stringified with the reference's
formatting only when a Symbol is serialised (``"(3, 3)"``, ``"True"``, ``"None"``).
"""
from __future__ import annotations

import torch

from .. import _state
from ..base import MXNetError

__all__ = ['OpDef', 'register', 'get', 'has', 'list_ops', 'invoke', 'alias']

_OPS = {}


class OpDef(object):
    """Description of one operator.

    inputs   : tuple of array-argument names in positional order; a trailing name starting with
               ``*`` makes the operator variadic (``Concat(*data, dim=1)``).
    fn       : callable(*tensors, **attrs) -> Tensor | tuple[Tensor]
    nout     : number of visible outputs (int) or callable(attrs) -> int
    defaults : attribute defaults (used for JSON round trips and ``list_attr``).
    """
    __slots__ = ('name', 'fn', 'inputs', 'variadic', 'nout', 'defaults', 'aliases', 'aux', 'doc',
                 'mutate', 'hidden_outputs')

    def __init__(self, name, fn, inputs, nout=1, defaults=None, aux=(), mutate=(), doc=None):
        self.name = name
        self.fn = fn
        inputs = tuple(inputs)
        self.variadic = bool(inputs) and inputs[-1].startswith('*')
        self.inputs = tuple(i.lstrip('*') for i in inputs)
        self.nout = nout
        self.defaults = dict(defaults or {})
        self.aliases = []
        self.aux = tuple(aux)          # names of inputs that are auxiliary states (BatchNorm moving stats)
        self.mutate = tuple(mutate)    # names of inputs updated in place (optimizer ops)
        self.doc = doc or (fn.__doc__ if fn is not None else None)

    def num_outputs(self, attrs):
        return self.nout(attrs) if callable(self.nout) else self.nout

    def __repr__(self):
        return '<OpDef %s%s>' % (self.name, self.inputs)


def register(name, *aliases, inputs=('data',), nout=1, defaults=None, aux=(), mutate=()):
    """Decorator: ``@register('FullyConnected', inputs=('data','weight','bias'))``."""
    def deco(fn):
        op = OpDef(name, fn, inputs, nout=nout, defaults=defaults, aux=aux, mutate=mutate)
        _OPS[name] = op
        for a in aliases:
            _OPS[a] = op
            op.aliases.append(a)
        return fn
    return deco


def alias(name, *aliases):
    op = _OPS[name]
    for a in aliases:
        _OPS[a] = op
        op.aliases.append(a)


def get(name):
    try:
        return _OPS[name]
    except KeyError:
        raise MXNetError('Operator %s is not registered' % name)


def has(name):
    return name in _OPS


def list_ops():
    return sorted(_OPS)


# --------------------------------------------------------------------------------------------
# array class plumbing (filled in by ndarray/ndarray.py and numpy/multiarray.py at import)
# --------------------------------------------------------------------------------------------
_array_classes = {}   # 'nd' -> NDArray, 'np' -> ndarray


_set_grad_enabled = torch._C._set_grad_enabled


def _set_array_class(kind, cls):
    _array_classes[kind] = cls


def _wrap(t, kind, ctx=None):
    return _array_classes[kind]._from_tensor(t, ctx)


def invoke(op, args, attrs, out=None, kind=None):
    """Run operator ``op`` (OpDef or name) on array wrappers ``args`` with attribute dict ``attrs``.

    ``args`` may contain array wrappers, raw tensors, python scalars or ``None`` (optional
    inputs).  Returns a wrapper, or a list of wrappers for multi-output operators.
    """
    if isinstance(op, str):
        op = get(op)
    st = _state.state
    tensors = []
    ctx = None
    base = _array_classes['nd']
    for a in args:
        if isinstance(a, base):
            if kind is None:
                kind = a._kind
            if ctx is None:
                ctx = a._ctx
            tensors.append(a._data)
        else:
            tensors.append(a)
    if kind is None:
        kind = 'np' if st.np_array else 'nd'
    if ctx is None and attrs:
        c = attrs.get('ctx')
        if c is not None and hasattr(c, 'device_typeid'):
            ctx = c                       # a creation operator: the result carries the device it was asked for (cpu(1) stays cpu(1))
    hook = _state.amp_hook
    if hook is not None and not st.opt_constraints & 1:
        tensors = hook(op.name, tensors)
    prof = _state.profiler_hook
    pctx = prof(op.name) if prof is not None else None
    if pctx is not None:
        pctx.__enter__()
    try:
        # the tensor library's gradient mode follows the recording state; switched with the two C calls directly (the
        # context-manager objects cost more host time than a small operator)
        if st.recording == torch.is_grad_enabled():
            res = op.fn(*tensors, **attrs)
        else:
            _set_grad_enabled(st.recording)
            try:
                res = op.fn(*tensors, **attrs)
            finally:
                _set_grad_enabled(not st.recording)
        if _state.naive_engine and ctx is not None and ctx.device_typeid == 2 and not torch.cuda.is_current_stream_capturing():
            # MXNET_ENGINE_TYPE=NaiveEngine: every operator has finished (or failed) before its call returns, so a device
            # error is raised by the operator that caused it (src/engine/naive_engine.cc runs each op inline)
            torch.cuda.current_stream(ctx.torch_device).synchronize()
    except MXNetError:
        raise
    except RuntimeError as e:
        # operator failures (shape mismatch, bad arguments caught by the tensor library) surface as
        # MXNetError like the reference's dmlc::Error -> MXNetError path (python/mxnet/base.py:246)
        raise MXNetError('%s: %s' % (op.name, e)) from e
    finally:
        if pctx is not None:
            pctx.__exit__(None, None, None)
    multi = isinstance(res, (tuple, list))
    if out is not None:
        outs = out if isinstance(out, (list, tuple)) else [out]
        ress = res if multi else [res]
        for o, r in zip(outs, ress):
            if o._data is not r:
                with torch.no_grad():
                    o._data.copy_(r)
        result = out
        wrapped = list(outs)
    elif multi:
        wrapped = [_wrap(r, kind, ctx) if isinstance(r, torch.Tensor) else r for r in res]
        result = wrapped
    else:
        result = _wrap(res, kind, ctx) if isinstance(res, torch.Tensor) else res
        wrapped = [result]
    tracer = st.tracer
    if tracer is not None:
        tracer.record(op, args, attrs, wrapped)
    elif st.recording:
        # provenance for autograd.get_symbol: which operator call produced each recorded output
        for i, o in enumerate(wrapped):
            if isinstance(o, base):
                o._prov = (op, args, attrs, i, len(wrapped))
    mon = _state.op_monitor
    if mon is not None:
        mon(op.name, wrapped)
    return result


def make_frontend(op, kind):
    """Build the user-facing function of an operator for one namespace (``mx.nd`` or ``mx.npx``).

    Mirrors the code generation of ``python/mxnet/ndarray/register.py:116-270``: array arguments
    may be given positionally or by keyword, attributes by keyword (or positionally after the
    arrays), ``out=`` receives the result, ``name=`` is accepted and ignored imperatively.
    """
    if isinstance(op, str):
        op = get(op)
    in_names = op.inputs
    attr_names = [k for k in op.defaults]

    if op.variadic:
        def frontend(*args, out=None, name=None, **kwargs):
            arrays = []
            for a in args:
                if isinstance(a, (list, tuple)):
                    arrays.extend(a)
                else:
                    arrays.append(a)
            kwargs.pop('num_args', None)
            return invoke(op, arrays, kwargs, out=out, kind=kind)
    else:
        n_in = len(in_names)

        def frontend(*args, out=None, name=None, **kwargs):
            arrays = list(args[:n_in])
            extra = args[n_in:]
            if len(arrays) < n_in:
                arrays.extend([None] * (n_in - len(arrays)))
            for i, nm in enumerate(in_names):
                if nm in kwargs:
                    arrays[i] = kwargs.pop(nm)
            while arrays and arrays[-1] is None:
                arrays.pop()
            for k, v in zip(attr_names, extra):
                kwargs[k] = v
            return invoke(op, arrays, kwargs, out=out, kind=kind)
    frontend.__name__ = op.name
    frontend.__doc__ = op.doc
    frontend._op = op
    return frontend

"""Autograd: ``record/pause/train_mode/predict_mode``, ``mark_variables``, ``backward``, ``grad``, ``Function``.

Reference: ``python/mxnet/autograd.py`` over ``Imperative::RecordOp/MarkVariables/Backward``
(``src/imperative/imperative.cc:143-172,237-334,445-757``).  The tape is the tensor library's
autograd graph; the recording flag decides whether operators run with graph construction on.

Gradient buffers are owned by the array (``attach_grad``) and installed as the leaf's ``.grad``
so accumulation happens *in place* into memory whose address never changes; that is what lets
the fused KVStore kernels read gradients directly from flat buckets.  ``grad_req='write'`` is
implemented by clearing buffers that were written by an earlier pass right before the next
backward accumulates into them; ``'add'`` never clears.
"""
from __future__ import annotations

import weakref

import torch

from . import _state
from .base import MXNetError
from .ndarray.ndarray import NDArray

__all__ = ['set_recording', 'set_training', 'is_recording', 'is_training', 'record', 'pause', 'train_mode',
           'predict_mode', 'mark_variables', 'backward', 'grad', 'get_symbol', 'Function']


def set_recording(is_recording):
    prev = _state.state.recording
    _state.state.recording = bool(is_recording)
    return prev


def set_training(train_mode):
    prev = _state.state.training
    _state.state.training = bool(train_mode)
    return prev


def is_recording():
    return _state.state.recording


def is_training():
    return _state.state.training


class _RecordingStateScope(object):
    def __init__(self, is_record, train_mode):
        self._enter_is_record = is_record
        self._enter_train_mode = train_mode
        self._prev_is_record = None
        self._prev_train_mode = None

    def __enter__(self):
        if self._enter_is_record is not None:
            self._prev_is_record = set_recording(self._enter_is_record)
        if self._enter_train_mode is not None:
            self._prev_train_mode = set_training(self._enter_train_mode)
        return self

    def __exit__(self, ptype, value, trace):
        if self._enter_is_record is not None and self._prev_is_record != self._enter_is_record:
            set_recording(self._prev_is_record)
        if self._enter_train_mode is not None and self._prev_train_mode != self._enter_train_mode:
            set_training(self._prev_train_mode)


def record(train_mode=True):
    """Scope in which executed operators are recorded for differentiation."""
    return _RecordingStateScope(True, train_mode)


def pause(train_mode=False):
    return _RecordingStateScope(False, train_mode)


def train_mode():
    return _RecordingStateScope(None, True)


def predict_mode():
    return _RecordingStateScope(None, False)


_pass_id = [0]


def _make_hook(ref):
    """Pre-accumulation hook of a marked leaf.  ``grad_req='write'``: the first gradient that reaches
    the leaf in a new backward pass must replace what an earlier pass left in the buffer, so the
    buffer is cleared right before the in-place accumulation.  Leaves that do not take part in a
    pass keep their gradients, like in the reference where only the variables of the differentiated
    graph are written."""
    def hook(g):
        var = ref()
        if var is None:
            return None
        cur = _pass_id[0]
        if var._grad_req == 'write' and var._fresh_grad and var._grad_pass != cur:
            var._grad._data.zero_()
        var._fresh_grad = True
        var._grad_pass = cur
        return None
    return hook


def mark_variables(variables, gradients, grad_reqs='write'):
    """Attach gradient buffers to arrays (``MXAutogradMarkVariables``)."""
    if isinstance(variables, NDArray):
        variables, gradients = [variables], [gradients]
    if isinstance(grad_reqs, str):
        grad_reqs = [grad_reqs] * len(variables)
    for var, g, req in zip(variables, gradients, grad_reqs):
        t = var._data
        old = getattr(var, '_hook', None)
        if old is not None:
            old.remove()
            var._hook = None
        if t.grad_fn is not None and req != 'null' and g is not None:
            # An array produced by a recorded operator stays in its graph and keeps the gradient that flows through it
            # (``Imperative::MarkVariables`` on an array that already has autograd information, src/imperative/imperative.cc):
            # the hook copies (or adds) that gradient into the attached buffer in every backward pass.
            var._grad_req = req
            var._grad = g
            var._fresh_grad = False
            var._grad_pass = -1
            var._hook = t.register_hook(_make_retain_hook(weakref.ref(var)))
            continue
        if t.grad_fn is not None and req == 'null':
            var._grad_req, var._grad = 'null', None      # drop_grad of an intermediate: it stays part of its graph
            continue
        if t.grad_fn is not None or (t.requires_grad and not t.is_leaf):
            t = t.detach()
            var._data = t
        var._grad_req = req
        if req == 'null':
            var._grad = None
            if t.is_leaf:
                t.requires_grad_(False)
                t.grad = None
            continue
        if not (t.dtype.is_floating_point or t.dtype.is_complex):
            # integer arrays may be marked too (the reference allows it); nothing differentiable flows into them, so the
            # attached buffer simply stays zero
            var._grad = g
            var._fresh_grad = False
            continue
        var._grad = g
        var._fresh_grad = False
        t.requires_grad_(True)
        t.grad = g._data
        var._grad_pass = -1
        var._hook = t.register_hook(_make_hook(weakref.ref(var)))


def _make_retain_hook(ref):
    def hook(g):
        var = ref()
        if var is None or var._grad is None:
            return None
        with torch.no_grad():
            if var._grad_req == 'add':
                var._grad._data.add_(g)
            else:
                var._grad._data.copy_(g)
        var._fresh_grad = True
        return None
    return hook


def mark_grads_consumed(arrays):
    """Tell autograd that the gradient buffers attached to the variables ``arrays`` were consumed and
    already cleared by the caller (the fused optimizer kernels zero them in the same pass)."""
    for a in arrays:
        a._fresh_grad = False


def _head_grads(heads, head_grads):
    out = []
    for i, h in enumerate(heads):
        hg = head_grads[i] if head_grads is not None else None
        if hg is None:
            out.append(torch.ones_like(h._data))
        else:
            out.append(hg._data if isinstance(hg, NDArray) else torch.as_tensor(hg, device=h._data.device))
    return out


def backward(heads, head_grads=None, retain_graph=False, train_mode=True):  # pylint: disable=redefined-outer-name
    """Compute gradients of ``heads`` w.r.t. every marked variable (``MXAutogradBackwardEx``)."""
    if isinstance(heads, NDArray):
        heads = [heads]
        if head_grads is not None and not isinstance(head_grads, (list, tuple)):
            head_grads = [head_grads]
    tensors = [h._data for h in heads]
    for t in tensors:
        if not t.requires_grad:
            raise MXNetError('Cannot differentiate node because it is not in a computational graph. '
                             'You need to set is_recording to true or use autograd.record() to save '
                             'computational graphs for backward.')
    for h in heads:
        if getattr(h, '_freed', False):
            raise MXNetError('The computational graph of this array was freed by an earlier backward pass; '
                             'pass retain_graph=True to differentiate it more than once.')
    _pass_id[0] += 1
    grads = _head_grads(heads, head_grads)
    prev = set_training(train_mode)
    try:
        torch.autograd.backward(tensors, grads, retain_graph=retain_graph)
    finally:
        set_training(prev)
    if not retain_graph:
        for h in heads:
            if h._data.grad_fn is not None:
                h._freed = True                  # the reference frees the recorded graph here (MXAutogradBackwardEx); the mark
                                                 # lives on this array object, not on the tensor a graph replay hands out again


def grad(heads, variables, head_grads=None, retain_graph=None, create_graph=False, train_mode=True):  # pylint: disable=redefined-outer-name
    """Gradients of heads w.r.t. variables, returned as new arrays (supports higher order)."""
    single = isinstance(variables, NDArray)
    if isinstance(heads, NDArray):
        heads = [heads]
        if head_grads is not None and not isinstance(head_grads, (list, tuple)):
            head_grads = [head_grads]
    if single:
        variables = [variables]
    if retain_graph is None:
        retain_graph = create_graph
    prev = set_training(train_mode)
    try:
        with torch.enable_grad():
            res = torch.autograd.grad([h._data for h in heads], [v._data for v in variables],
                                      _head_grads(heads, head_grads), retain_graph=retain_graph,
                                      create_graph=create_graph, allow_unused=True)
    finally:
        set_training(prev)
    outs = []
    for r, v in zip(res, variables):
        if r is None:
            r = torch.zeros_like(v._data)
        outs.append(v.__class__._from_tensor(r, v._ctx))
    return outs[0] if single else outs


def get_symbol(x):
    """Retrieve the recorded computation history of ``x`` as a Symbol
    (python/mxnet/autograd.py:330-347, ``MXAutogradGetSymbol``).  Arrays that were not produced by a
    recorded operator become variables ``var0, var1, ...`` in order of first use."""
    from .symbol.symbol import Symbol, _Node, var
    from .name import NameManager
    from .ndarray.ndarray import NDArray
    if x._sym is not None:
        return Symbol([x._sym])
    names = NameManager()
    entries, nodes, leaves = {}, {}, []

    def entry(a):
        hit = entries.get(id(a))
        if hit is not None:
            return hit
        prov = getattr(a, '_prov', None)
        if prov is None:
            v = var('var%d' % len(leaves))
            leaves.append(a)
            entries[id(a)] = v._outputs[0]
            return entries[id(a)]
        op, args, attrs, idx, nout = prov
        key = id(prov[1])
        node = nodes.get(key)
        if node is None:
            ins = [entry(i) for i in args if isinstance(i, NDArray)]
            node = nodes[key] = _Node(op, names.get(None, op.name.lower().lstrip('_')), dict(attrs), ins, max(nout, 1))
        entries[id(a)] = (node, idx)
        return entries[id(a)]

    if getattr(x, '_prov', None) is None:
        raise MXNetError('array was not produced by a recorded operator')
    return Symbol([entry(x)])


class Function(object):
    """User-defined differentiable function (``python/mxnet/autograd.py`` ``Function``).

    Subclass and implement ``forward`` and ``backward`` over arrays; ``save_for_backward`` keeps
    tensors for the backward pass.  An instance may be called once.
    """

    def __init__(self):
        self._used = False
        self.saved_tensors = ()

    def save_for_backward(self, *args):
        self.saved_tensors = args

    def forward(self, *inputs):
        raise NotImplementedError()

    def backward(self, *output_grads):
        raise NotImplementedError()

    def __call__(self, *inputs):
        assert not self._used, 'Each Function instance can only be called once. Please create another instance.'
        self._used = True
        func = self
        cls = inputs[0].__class__ if inputs else NDArray
        ctxs = [i._ctx for i in inputs]

        class _Bridge(torch.autograd.Function):
            @staticmethod
            def forward(ctx, *tensors):
                with pause():
                    outs = func.forward(*[cls._from_tensor(t.detach(), c) for t, c in zip(tensors, ctxs)])
                ctx.single = not isinstance(outs, (list, tuple))
                outs = [outs] if ctx.single else list(outs)
                res = tuple(o._data for o in outs)
                return res[0] if ctx.single else res

            @staticmethod
            def backward(ctx, *gouts):
                with pause():
                    gin = func.backward(*[cls._from_tensor(g, None) for g in gouts])
                gin = [gin] if not isinstance(gin, (list, tuple)) else list(gin)
                return tuple(g._data if g is not None else None for g in gin)

        if _state.state.recording:
            with torch.enable_grad():
                res = _Bridge.apply(*[i._data for i in inputs])
        else:
            with torch.no_grad():
                res = _Bridge.apply(*[i._data for i in inputs])
        if isinstance(res, tuple):
            return [cls._from_tensor(r, ctxs[0] if ctxs else None) for r in res]
        return cls._from_tensor(res, ctxs[0] if ctxs else None)

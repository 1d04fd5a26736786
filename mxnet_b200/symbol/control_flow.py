"""Symbolic control flow: ``mx.sym.contrib.foreach / while_loop / cond`` (``python/mxnet/symbol/contrib.py``; operators
``_foreach``, ``_while_loop``, ``_cond`` of ``src/operator/control_flow.cc``).

The loop body (or branch) is traced once into a sub-graph on placeholder variables.  The outer graph gets one node whose
inputs are the loop data, the initial states and every variable the sub-graph reads from its surroundings; the node's
operator evaluates the sub-graph once per step (or once for the taken branch).  Sub-graphs travel in the ``subgraphs``
entry of the node in ``-symbol.json``, as in the reference's files.  Gradients flow through the unrolled evaluation.
"""
import torch

from ..base import MXNetError
from ..name import NameManager
from ..ops import registry as _reg
from .symbol import Symbol, _Node, _topo, var, Group

__all__ = ['foreach', 'while_loop', 'cond']

_uid = [0]


def _fresh(prefix):
    _uid[0] += 1
    return '%s%d' % (prefix, _uid[0])


def _as_list(x):
    if x is None:
        return [], False
    if isinstance(x, (list, tuple)):
        return list(x), True
    return [x], False


def _entries(symbols):
    out = []
    for s in symbols:
        if not isinstance(s, Symbol):
            raise MXNetError('control flow bodies must return Symbols, got %s' % type(s).__name__)
        out.extend(s._outputs)
    return out


def _free_variables(sub, placeholders):
    """Variables of the sub-graph that are not loop placeholders, in graph order, as Symbols of the same nodes."""
    own = set(placeholders)
    free = []
    for n in _topo(sub._outputs):
        if n.op is None and n.name not in own:
            free.append(Symbol([(n, 0)]))
    return free


def _node(op_name, inputs, attrs, nout, name):
    op = _reg.get(op_name)
    name = NameManager.current().get(name, op_name.lstrip('_'))
    node = _Node(op, name, attrs, [s._outputs[0] for s in inputs], nout)
    return [Symbol([(node, i)]) for i in range(nout)]


def foreach(body, data, init_states, name='foreach'):
    """Run ``body(data_slice, states) -> (outputs, new_states)`` over axis 0 of ``data``; returns the stacked outputs and
    the final states, with the nesting (single Symbol or list) of what ``body`` returned."""
    data_l, data_is_list = _as_list(data)
    state_l, state_is_list = _as_list(init_states)
    tag = _fresh('foreach')
    d_names = ['%s_data%d' % (tag, i) for i in range(len(data_l))]
    s_names = ['%s_state%d' % (tag, i) for i in range(len(state_l))]
    d_vars, s_vars = [var(n) for n in d_names], [var(n) for n in s_names]
    outs, new_states = body(d_vars if data_is_list else d_vars[0], s_vars if state_is_list else (s_vars[0] if s_vars else []))
    outs_l, outs_is_list = _as_list(outs)
    new_l, _ = _as_list(new_states)
    if len(new_l) != len(state_l):
        raise MXNetError('foreach: body returned %d states for %d initial states' % (len(new_l), len(state_l)))
    sub = Symbol(_entries(outs_l) + _entries(new_l))
    free = _free_variables(sub, d_names + s_names)
    attrs = {'num_data': len(data_l), 'num_states': len(state_l), 'num_outs': len(outs_l), 'data_names': ','.join(d_names),
             'state_names': ','.join(s_names), 'free_names': ','.join(f.name for f in free), '__subgraph__0': sub}
    res = _node('_foreach', data_l + state_l + free, attrs, len(outs_l) + len(state_l), name)
    out_syms, state_syms = res[:len(outs_l)], res[len(outs_l):]
    return (out_syms if outs_is_list else (out_syms[0] if out_syms else [])), \
        (state_syms if state_is_list else (state_syms[0] if state_syms else []))


def while_loop(cond, func, loop_vars, max_iterations=None, name='while_loop'):    # pylint: disable=redefined-outer-name
    """``while cond(*vars): outputs, vars = func(*vars)`` for at most ``max_iterations`` steps.  Returns the step outputs
    stacked along a new axis 0 of length ``max_iterations`` (rows of steps that did not run are zero) and the final
    loop variables."""
    if max_iterations is None:
        raise ValueError('max_iterations should be specified')
    vars_l, vars_is_list = _as_list(loop_vars)
    tag = _fresh('while')
    v_names = ['%s_var%d' % (tag, i) for i in range(len(vars_l))]
    v_vars = [var(n) for n in v_names]
    c = cond(*v_vars)
    step_out, new_vars = func(*v_vars)
    outs_l, outs_is_list = _as_list(step_out)
    new_l, _ = _as_list(new_vars)
    if len(new_l) != len(vars_l):
        raise MXNetError('while_loop: func returned %d loop variables for %d' % (len(new_l), len(vars_l)))
    cond_sub, func_sub = Symbol(_entries([c])), Symbol(_entries(outs_l) + _entries(new_l))
    free = _free_variables(Group([cond_sub, func_sub]), v_names)
    attrs = {'num_vars': len(vars_l), 'num_outs': len(outs_l), 'max_iterations': int(max_iterations), 'var_names': ','.join(v_names),
             'free_names': ','.join(f.name for f in free), '__subgraph__0': cond_sub, '__subgraph__1': func_sub}
    res = _node('_while_loop', vars_l + free, attrs, len(outs_l) + len(vars_l), name)
    out_syms, var_syms = res[:len(outs_l)], res[len(outs_l):]
    return (out_syms if outs_is_list else (out_syms[0] if out_syms else [])), (var_syms if vars_is_list else var_syms[0])


def cond(pred, then_func, else_func, name='cond'):
    """``then_func()`` when the scalar ``pred`` is non-zero, else ``else_func()``; both must give the same number of
    outputs."""
    then_l, is_list = _as_list(then_func())
    else_l, _ = _as_list(else_func())
    if len(then_l) != len(else_l):
        raise MXNetError('cond: the branches return %d and %d outputs' % (len(then_l), len(else_l)))
    then_sub, else_sub = Symbol(_entries(then_l)), Symbol(_entries(else_l))
    free = _free_variables(Group([then_sub, else_sub]), [])
    attrs = {'num_outs': len(then_l), 'free_names': ','.join(f.name for f in free), '__subgraph__0': then_sub, '__subgraph__1': else_sub}
    res = _node('_cond', [pred] + free, attrs, len(then_l), name)
    return res if is_list else res[0]


# ---------------------------------------------------------------------------------------- the operators
def _names(v):
    """Name lists are stored as one comma-separated string so that they survive the text form of graph attributes."""
    if isinstance(v, str):
        return tuple(n for n in v.split(',') if n)
    return tuple(v or ())


def _foreach_op(*tensors, num_data=1, num_states=0, num_outs=1, data_names=(), state_names=(), free_names=(), **subgraphs):
    sub = subgraphs['__subgraph__0']
    data_names, state_names, free_names = _names(data_names), _names(state_names), _names(free_names)
    data, states, free = tensors[:num_data], list(tensors[num_data:num_data + num_states]), tensors[num_data + num_states:]
    feed_free = dict(zip(free_names, free))
    steps = data[0].shape[0]
    outs = [[] for _ in range(num_outs)]
    for t in range(steps):
        feed = dict(feed_free)
        feed.update({n: d[t] for n, d in zip(data_names, data)})
        feed.update(dict(zip(state_names, states)))
        res = sub._run(feed)
        for j in range(num_outs):
            outs[j].append(res[j])
        states = list(res[num_outs:])
    if steps == 0:
        raise MXNetError('foreach over an empty axis')
    return tuple(torch.stack(o, 0) for o in outs) + tuple(states)


def _while_loop_op(*tensors, num_vars=1, num_outs=0, max_iterations=1, var_names=(), free_names=(), **subgraphs):
    cond_sub, func_sub = subgraphs['__subgraph__0'], subgraphs['__subgraph__1']
    var_names, free_names = _names(var_names), _names(free_names)
    loop_vars, free = list(tensors[:num_vars]), tensors[num_vars:]
    feed_free = dict(zip(free_names, free))
    meta = any(t.device.type == 'meta' for t in tensors)
    outs = [[] for _ in range(num_outs)]
    steps = 0
    while steps < max_iterations:
        feed = dict(feed_free)
        feed.update(dict(zip(var_names, loop_vars)))
        if not meta and not bool(cond_sub._run(feed)[0]):
            break
        res = func_sub._run(feed)
        for j in range(num_outs):
            outs[j].append(res[j])
        loop_vars = list(res[num_outs:])
        steps += 1
        if meta:
            break                                 # shapes only: one step tells them all
    stacked = []
    for o in outs:
        if not o:
            raise MXNetError('while_loop: the condition is false before the first step, so the shape of the outputs is unknown')
        s = torch.stack(o, 0)
        if s.shape[0] < max_iterations:
            pad = torch.zeros((max_iterations - s.shape[0],) + tuple(s.shape[1:]), dtype=s.dtype, device=s.device)
            s = torch.cat([s, pad], 0)
        stacked.append(s)
    return tuple(stacked) + tuple(loop_vars)


def _cond_op(pred, *free, num_outs=1, free_names=(), **subgraphs):
    free_names = _names(free_names)
    feed = dict(zip(free_names, free))
    take_then = True if pred.device.type == 'meta' else bool(pred.reshape(-1)[0] != 0)
    res = subgraphs['__subgraph__0' if take_then else '__subgraph__1']._run(feed)
    return tuple(res) if num_outs > 1 else res[0]


_reg.register('_foreach', inputs=('*data',), nout=lambda a: int(a.get('num_outs', 1)) + int(a.get('num_states', 0)))(_foreach_op)
_reg.register('_while_loop', inputs=('*data',), nout=lambda a: int(a.get('num_outs', 0)) + int(a.get('num_vars', 1)))(_while_loop_op)
_reg.register('_cond', inputs=('pred', '*data'), nout=lambda a: int(a.get('num_outs', 1)))(_cond_op)
for _old, _new in (('_foreach', '_npx_foreach'), ('_while_loop', '_npx_while_loop'), ('_cond', '_npx_cond')):
    _reg.alias(_old, _new)

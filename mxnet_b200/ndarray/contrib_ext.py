"""Control-flow helpers attached to ``mx.nd.contrib`` (``python/mxnet/ndarray/contrib.py``):
``foreach``, ``while_loop``, ``cond`` run eagerly over arrays; under autograd they unroll onto the
tape, which is also how the reference's imperative versions behave."""
import sys as _sys

from .ndarray import NDArray
from ..ops import registry as _reg


def _flatten(x):
    return list(x) if isinstance(x, (list, tuple)) else [x]


def foreach(body, data, init_states):
    single_data = isinstance(data, NDArray)
    seqs = [data] if single_data else list(data)
    states = init_states
    outs = []
    for i in range(seqs[0].shape[0]):
        eles = seqs[0][i] if single_data else [s[i] for s in seqs]
        out, states = body(eles, states)
        outs.append(out)
    if not outs:
        return [], states
    if isinstance(outs[0], (list, tuple)):
        stacked = [_reg.invoke('stack', [o[j] for o in outs], {'axis': 0}) for j in range(len(outs[0]))]
    else:
        stacked = _reg.invoke('stack', outs, {'axis': 0})
    return stacked, states


def while_loop(cond, func, loop_vars, max_iterations=None):
    if max_iterations is None:
        raise ValueError('max_iterations should be specified')
    loop_vars = _flatten(loop_vars)
    steps, outputs = 0, []
    while steps < max_iterations and bool(cond(*loop_vars)):
        step_out, loop_vars = func(*loop_vars)
        loop_vars = _flatten(loop_vars)
        outputs.append(_flatten(step_out))
        steps += 1
    stacked = []
    if outputs:
        for j in range(len(outputs[0])):
            s = _reg.invoke('stack', [o[j] for o in outputs], {'axis': 0})
            if steps < max_iterations:
                pad = [(0, max_iterations - steps)] + [(0, 0)] * (s.ndim - 1)
                import torch
                flat = []
                for lo, hi in reversed(pad):
                    flat.extend([lo, hi])
                s = s.__class__._from_tensor(torch.nn.functional.pad(s._data, flat), s._ctx)
            stacked.append(s)
    return stacked, loop_vars


def cond(pred, then_func, else_func):
    return then_func() if bool(pred) else else_func()


def isinf(data): return _reg.invoke('isinf', [data], {})
def isnan(data): return _reg.invoke('isnan', [data], {})
def isfinite(data): return _reg.invoke('isfinite', [data], {})


_contrib = _sys.modules[__name__.rsplit('.', 1)[0] + '.contrib']
for _n in ('foreach', 'while_loop', 'cond', 'isinf', 'isnan', 'isfinite'):
    setattr(_contrib, _n, globals()[_n])

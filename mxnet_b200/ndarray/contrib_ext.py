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


def rand_zipfian(true_classes, num_sampled, range_max, ctx=None):
    """Draw ``num_sampled`` candidates from [0, range_max) with P(class) = log((class + 2) / (class + 1)) / log(range_max + 1)
    (an approximately Zipfian law, for classes sorted by decreasing frequency; ``python/mxnet/ndarray/contrib.py:39``).
    Returns (samples int64 [num_sampled], expected count of each true class float64, expected count of each sample float64)."""
    import math
    import torch
    ctx = ctx or true_classes._ctx
    dev = ctx.torch_device
    log_range = math.log(range_max + 1)
    u = torch.rand(num_sampled, dtype=torch.float64, device=dev) * log_range       # the device's global stream (mx.random.seed)
    samples = (torch.exp(u).to(torch.int64) - 1) % range_max

    def expected(classes):
        c = classes.to(torch.float64)
        return torch.log((c + 2.0) / (c + 1.0)) / log_range * num_sampled
    true = true_classes._data.to(dev)
    return (NDArray._from_tensor(samples, ctx), NDArray._from_tensor(expected(true), ctx),
            NDArray._from_tensor(expected(samples), ctx))


def _multi_update(op_name, per_tensor, step_count, lrs, wds, out, num_tensors, kwargs):
    flat = [a for group in zip(*per_tensor) for a in group]
    n = num_tensors or len(per_tensor[0])
    attrs = dict(kwargs, step_count=tuple(step_count), learning_rates=tuple(lrs), wds=tuple(wds), num_tensors=n)
    return _reg.invoke(op_name, flat, attrs, out=out)


def multi_lamb_update(weights, grads, mean, var, step_count, lrs, wds, out=None, num_tensors=0, **kwargs):
    """LAMB update of several tensors in one call (``_multi_lamb_update``; lists of weights, gradients, means, variances)."""
    return _multi_update('_multi_lamb_update', (weights, grads, mean, var), step_count, lrs, wds, out or list(weights), num_tensors, kwargs)


def multi_mp_lamb_update(weights, grads, mean, var, weights32, step_count, lrs, wds, out=None, num_tensors=0, **kwargs):
    """Multi-precision form: fp32 master weights are updated and cast back."""
    return _multi_update('_multi_mp_lamb_update', (weights, grads, mean, var, weights32), step_count, lrs, wds, out or list(weights),
                         num_tensors, kwargs)


def multi_lans_update(weights, grads, mean, var, step_count, lrs, wds, out=None, num_tensors=0, **kwargs):
    """LANS update of several tensors in one call."""
    return _multi_update('_multi_lans_update', (weights, grads, mean, var), step_count, lrs, wds, out or list(weights), num_tensors, kwargs)


def multi_mp_lans_update(weights, grads, mean, var, weights32, step_count, lrs, wds, out=None, num_tensors=0, **kwargs):
    return _multi_update('_multi_mp_lans_update', (weights, grads, mean, var, weights32), step_count, lrs, wds, out or list(weights),
                         num_tensors, kwargs)


_contrib = _sys.modules[__name__.rsplit('.', 1)[0] + '.contrib']
for _n in ('foreach', 'while_loop', 'cond', 'isinf', 'isnan', 'isfinite', 'rand_zipfian', 'multi_lamb_update', 'multi_mp_lamb_update',
           'multi_lans_update', 'multi_mp_lans_update'):
    setattr(_contrib, _n, globals()[_n])

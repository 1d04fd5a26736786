"""``mx.nd.random``: sampling front ends that accept scalars or arrays as distribution parameters
(``python/mxnet/ndarray/random.py``)."""
from ..ops import registry as _reg
from ..ops.random import seed  # noqa: F401
from .ndarray import NDArray

__all__ = ['uniform', 'normal', 'randn', 'poisson', 'exponential', 'gamma', 'multinomial', 'negative_binomial',
           'generalized_negative_binomial', 'shuffle', 'randint', 'seed', 'binomial', 'categorical']


def _helper(scalar_op, sample_op, params, shape, dtype, ctx, out, kwargs):
    if isinstance(params[0][1], NDArray):
        return _reg.invoke(sample_op, [p for _, p in params], {'shape': shape or (), 'dtype': dtype}, out=out, kind='nd')
    attrs = {k: v for k, v in params}
    attrs.update(shape=shape if shape is not None else (1,), ctx=ctx, dtype=dtype or 'float32')
    return _reg.invoke(scalar_op, [], attrs, out=out, kind='nd')


def uniform(low=0, high=1, shape=None, dtype=None, ctx=None, out=None, **kwargs):
    return _helper('_random_uniform', '_sample_uniform', [('low', low), ('high', high)], shape, dtype, ctx, out, kwargs)


def normal(loc=0, scale=1, shape=None, dtype=None, ctx=None, out=None, **kwargs):
    return _helper('_random_normal', '_sample_normal', [('loc', loc), ('scale', scale)], shape, dtype, ctx, out, kwargs)


def randn(*shape, **kwargs):
    loc, scale = kwargs.pop('loc', 0), kwargs.pop('scale', 1)
    return normal(loc, scale, shape=shape or (1,), **kwargs)


def poisson(lam=1, shape=None, dtype=None, ctx=None, out=None, **kwargs):
    return _helper('_random_poisson', '_sample_poisson', [('lam', lam)], shape, dtype, ctx, out, kwargs)


def exponential(scale=1, shape=None, dtype=None, ctx=None, out=None, **kwargs):
    lam = 1.0 / scale if not isinstance(scale, NDArray) else 1.0 / scale
    return _helper('_random_exponential', '_sample_exponential', [('lam', lam)], shape, dtype, ctx, out, kwargs)


def gamma(alpha=1, beta=1, shape=None, dtype=None, ctx=None, out=None, **kwargs):
    return _helper('_random_gamma', '_sample_gamma', [('alpha', alpha), ('beta', beta)], shape, dtype, ctx, out, kwargs)


def negative_binomial(k=1, p=1, shape=None, dtype=None, ctx=None, out=None, **kwargs):
    return _helper('_random_negative_binomial', '_sample_negative_binomial', [('k', k), ('p', p)], shape, dtype, ctx, out, kwargs)


def generalized_negative_binomial(mu=1, alpha=1, shape=None, dtype=None, ctx=None, out=None, **kwargs):
    return _helper('_random_generalized_negative_binomial', '_sample_generalized_negative_binomial',
                   [('mu', mu), ('alpha', alpha)], shape, dtype, ctx, out, kwargs)


def multinomial(data, shape=None, get_prob=False, out=None, dtype='int32', **kwargs):
    return _reg.invoke('_sample_multinomial', [data], {'shape': shape or (), 'get_prob': get_prob, 'dtype': dtype}, out=out)


def binomial(n=1, p=0.5, shape=None, dtype=None, ctx=None, out=None, **kwargs):
    """Samples of a binomial distribution with ``n`` trials and success probability ``p`` (scalars, or arrays that give one
    distribution per element: ``python/mxnet/ndarray/random.py:386``)."""
    return _helper('_random_binomial', '_sample_binomial', [('n', n), ('p', p)], shape, dtype, ctx, out, kwargs)


def categorical(data, shape=None, get_prob=False, out=None, dtype='int32', **kwargs):
    """Concurrent sampling from the categorical distributions in the rows of ``data`` (probabilities that sum to one along
    the last axis); with ``get_prob`` also the log-likelihood of the samples (``python/mxnet/ndarray/random.py:552``)."""
    return _reg.invoke('_sample_categorical', [data], {'shape': shape or (), 'get_prob': get_prob, 'dtype': dtype}, out=out)


def shuffle(data, **kwargs):
    return _reg.invoke('_shuffle', [data], {})


def randint(low, high, shape=None, dtype=None, ctx=None, out=None, **kwargs):
    return _reg.invoke('_random_randint', [], {'low': low, 'high': high, 'shape': shape if shape is not None else (1,),
                                               'ctx': ctx, 'dtype': dtype or 'int32'}, out=out, kind='nd')

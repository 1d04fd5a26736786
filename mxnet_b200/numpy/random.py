"""``mx.np.random`` (``python/mxnet/numpy/random.py``)."""
from ..ops import registry as _reg
from ..ops.random import seed  # noqa: F401
from ..ndarray.ndarray import NDArray
from ..device import current_device

__all__ = ['uniform', 'normal', 'randn', 'rand', 'randint', 'choice', 'shuffle', 'permutation', 'gamma', 'beta',
           'exponential', 'bernoulli', 'multinomial', 'laplace', 'gumbel', 'logistic', 'rayleigh', 'weibull',
           'pareto', 'power', 'lognormal', 'chisquare', 'f', 'multivariate_normal', 'seed', 'random', 'random_sample']


def _arr(x):
    return isinstance(x, NDArray)


def _two(op, a, b, size, ctx, dtype, out=None, device=None):
    ctx = ctx or device
    arrays = [x for x in (a, b) if _arr(x)]
    if arrays:
        a = a if _arr(a) else float(a)
        b = b if _arr(b) else float(b)
        return _reg.invoke(op, [a, b], {'size': size, 'ctx': ctx, 'dtype': dtype or 'float32'}, out=out, kind='np')
    return _reg.invoke(op, [a, b], {'size': size, 'ctx': ctx or current_device(), 'dtype': dtype or 'float32'}, out=out, kind='np')


def uniform(low=0.0, high=1.0, size=None, dtype=None, ctx=None, out=None, device=None):
    return _two('_npi_uniform', low, high, size, ctx, dtype, out, device)


def normal(loc=0.0, scale=1.0, size=None, dtype=None, ctx=None, out=None, device=None):
    return _two('_npi_normal', loc, scale, size, ctx, dtype, out, device)


def lognormal(mean=0.0, sigma=1.0, size=None, dtype=None, ctx=None, out=None, device=None):
    from . import multiarray as mnp
    return mnp.exp(normal(mean, sigma, size, dtype, ctx, None, device))


def randn(*size, **kwargs): return normal(0.0, 1.0, size=size or None, **kwargs)
def rand(*size, **kwargs): return uniform(0.0, 1.0, size=size or None, **kwargs)
def random(size=None, **kwargs): return uniform(0.0, 1.0, size=size, **kwargs)
random_sample = random


def randint(low, high=None, size=None, dtype=None, ctx=None, out=None, device=None):
    return _reg.invoke('_npi_randint', [], {'low': low, 'high': high, 'size': size, 'ctx': ctx or device or current_device(),
                                            'dtype': dtype or 'int64'}, out=out, kind='np')


def choice(a, size=None, replace=True, p=None, ctx=None, out=None, device=None):
    args = [a] if _arr(a) else []
    attrs = {'size': size, 'replace': replace, 'ctx': ctx or device or current_device()}
    if not _arr(a):
        return _reg.invoke('_npi_choice', [a, p], attrs, out=out, kind='np')
    return _reg.invoke('_npi_choice', [a, p], attrs, out=out, kind='np')


def shuffle(x):
    r = _reg.invoke('_npi_shuffle', [x], {}, kind='np')
    x._data.copy_(r._data)


def permutation(x):
    from . import multiarray as mnp
    if isinstance(x, int):
        x = mnp.arange(x, dtype='int64')
    return _reg.invoke('_npi_shuffle', [x], {}, kind='np')


def gamma(shape, scale=1.0, size=None, dtype=None, ctx=None, out=None, device=None):
    return _two('_npi_gamma', shape, scale, size, ctx, dtype, out, device)


def beta(a, b, size=None, dtype=None, ctx=None, device=None):
    x = gamma(a, 1.0, size, dtype, ctx, None, device)
    y = gamma(b, 1.0, size, dtype, ctx, None, device)
    return x / (x + y)


def chisquare(df, size=None, dtype=None, ctx=None, device=None): return gamma(df / 2.0, 2.0, size, dtype, ctx, None, device)
def f(dfnum, dfden, size=None, ctx=None, device=None):
    return (chisquare(dfnum, size, None, ctx, device) / dfnum) / (chisquare(dfden, size, None, ctx, device) / dfden)


def exponential(scale=1.0, size=None, ctx=None, out=None, device=None):
    return _reg.invoke('_npi_exponential', [scale], {'size': size, 'ctx': ctx or device or current_device()}, out=out, kind='np')


def bernoulli(prob=None, logit=None, size=None, dtype=None, ctx=None, out=None, device=None):
    p = prob if prob is not None else logit
    return _reg.invoke('_npi_bernoulli', [p], {'size': size, 'ctx': ctx or device or current_device(), 'dtype': dtype or 'float32',
                                               'is_logit': prob is None}, out=out, kind='np')


def multinomial(n, pvals, size=None):
    from . import multiarray as mnp
    return _reg.invoke('_npi_multinomial', [pvals if _arr(pvals) else mnp.array(pvals)], {'n': n, 'size': size}, kind='np')


def multivariate_normal(mean, cov, size=None, check_valid=None, tol=None):
    from . import multiarray as mnp
    from . import linalg
    L = linalg.cholesky(cov)
    shape = (() if size is None else ((size,) if isinstance(size, int) else tuple(size))) + mean.shape
    z = normal(0.0, 1.0, size=shape, ctx=mean.ctx)
    return mean + mnp.matmul(z[..., None, :], mnp.swapaxes(L, -1, -2))[..., 0, :]


def _dist(op):
    def fn(*params, size=None, ctx=None, out=None, device=None):
        return _reg.invoke('_npi_' + op, list(params), {'size': size, 'ctx': ctx or device or current_device()}, out=out, kind='np')
    return fn


laplace = lambda loc=0.0, scale=1.0, size=None, dtype=None, ctx=None, out=None, device=None: _dist('laplace')(loc, scale, size=size, ctx=ctx, out=out, device=device)
gumbel = lambda loc=0.0, scale=1.0, size=None, ctx=None, out=None, device=None: _dist('gumbel')(loc, scale, size=size, ctx=ctx, out=out, device=device)
logistic = lambda loc=0.0, scale=1.0, size=None, ctx=None, out=None, device=None: _dist('logistic')(loc, scale, size=size, ctx=ctx, out=out, device=device)
rayleigh = lambda scale=1.0, size=None, ctx=None, out=None, device=None: _dist('rayleigh')(scale, size=size, ctx=ctx, out=out, device=device)
weibull = lambda a, size=None, ctx=None, out=None, device=None: _dist('weibull')(a, size=size, ctx=ctx, out=out, device=device)
pareto = lambda a, size=None, ctx=None, out=None, device=None: _dist('pareto')(a, size=size, ctx=ctx, out=out, device=device)
power = lambda a, size=None, ctx=None, out=None, device=None: _dist('powerd')(a, size=size, ctx=ctx, out=out, device=device)

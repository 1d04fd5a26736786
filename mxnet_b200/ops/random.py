"""Random sampling operators and the global seed.

Reference: ``src/operator/random/*`` and ``src/operator/numpy/random/*`` (per-thread Philox-style
states from the resource manager, ``src/common/random_generator.{h,cu}``).  The streams differ
from the reference's, so tests compare distributions, not bit patterns; determinism under a fixed
seed is kept per device through the tensor library's Philox generator.
"""
from __future__ import annotations

import torch

from .registry import register
from .tensor import _dev
from ..base import to_torch_dtype


def seed(seed_state, ctx='all'):
    """``mx.random.seed``: seed every device generator (or one device when ``ctx`` is given)."""
    seed_state = int(seed_state)
    if ctx == 'all' or ctx is None:
        torch.manual_seed(seed_state)
        if torch.cuda.is_available():
            torch.cuda.manual_seed_all(seed_state)
    elif ctx.device_type == 'gpu':
        with torch.cuda.device(ctx.device_id):
            torch.cuda.manual_seed(seed_state)
    else:
        torch.manual_seed(seed_state)
    import numpy as np
    import random as pyrandom
    np.random.seed(seed_state % (2 ** 32))
    pyrandom.seed(seed_state)


def _shape(shape):
    if shape is None:
        return ()
    if isinstance(shape, int):
        return (shape,)
    return tuple(shape)


def _dt(dtype):
    return to_torch_dtype(dtype if dtype not in (None, 'None') else 'float32')


_D = {'shape': (), 'ctx': None, 'dtype': 'float32'}


@register('_random_uniform', 'random_uniform', 'uniform', inputs=(), defaults=dict(_D, low=0.0, high=1.0))
def random_uniform(low=0.0, high=1.0, shape=(), ctx=None, dtype='float32'):
    return torch.empty(_shape(shape), dtype=_dt(dtype), device=_dev(ctx)).uniform_(low, high)


@register('_random_normal', 'random_normal', 'normal', inputs=(), defaults=dict(_D, loc=0.0, scale=1.0))
def random_normal(loc=0.0, scale=1.0, shape=(), ctx=None, dtype='float32'):
    return torch.empty(_shape(shape), dtype=_dt(dtype), device=_dev(ctx)).normal_(loc, scale)


@register('_random_gamma', 'random_gamma', inputs=(), defaults=dict(_D, alpha=1.0, beta=1.0))
def random_gamma(alpha=1.0, beta=1.0, shape=(), ctx=None, dtype='float32'):
    a = torch.full(_shape(shape), float(alpha), dtype=torch.float32, device=_dev(ctx))
    return (torch._standard_gamma(a) * beta).to(_dt(dtype))


@register('_random_exponential', 'random_exponential', inputs=(), defaults=dict(_D, lam=1.0))
def random_exponential(lam=1.0, shape=(), ctx=None, dtype='float32'):
    return torch.empty(_shape(shape), dtype=_dt(dtype), device=_dev(ctx)).exponential_(lam)


@register('_random_poisson', 'random_poisson', inputs=(), defaults=dict(_D, lam=1.0))
def random_poisson(lam=1.0, shape=(), ctx=None, dtype='float32'):
    return torch.poisson(torch.full(_shape(shape), float(lam), device=_dev(ctx))).to(_dt(dtype))


@register('_random_negative_binomial', 'random_negative_binomial', inputs=(), defaults=dict(_D, k=1, p=1.0))
def random_negative_binomial(k=1, p=1.0, shape=(), ctx=None, dtype='float32'):
    a = torch.full(_shape(shape), float(k), device=_dev(ctx))
    lam = torch._standard_gamma(a) * ((1 - p) / p)
    return torch.poisson(lam).to(_dt(dtype))


@register('_random_generalized_negative_binomial', 'random_generalized_negative_binomial', inputs=(),
          defaults=dict(_D, mu=1.0, alpha=1.0))
def random_gen_neg_binomial(mu=1.0, alpha=1.0, shape=(), ctx=None, dtype='float32'):
    if alpha == 0:
        return random_poisson(mu, shape, ctx, dtype)
    a = torch.full(_shape(shape), 1.0 / alpha, device=_dev(ctx))
    lam = torch._standard_gamma(a) * (alpha * mu)
    return torch.poisson(lam).to(_dt(dtype))


@register('_random_randint', 'random_randint', inputs=(), defaults={'low': 0, 'high': 1, 'shape': (), 'ctx': None, 'dtype': 'int32'})
def random_randint(low=0, high=1, shape=(), ctx=None, dtype='int32'):
    return torch.randint(int(low), int(high), _shape(shape), device=_dev(ctx)).to(to_torch_dtype(dtype or 'int32'))


def _like(fn):
    def op(data, **kw):
        kw.pop('shape', None)
        return fn(shape=tuple(data.shape), ctx=None, dtype=data.dtype, **kw).to(data.device)
    return op


for _n, _f in (('uniform', random_uniform), ('normal', random_normal), ('gamma', random_gamma),
               ('exponential', random_exponential), ('poisson', random_poisson),
               ('negative_binomial', random_negative_binomial),
               ('generalized_negative_binomial', random_gen_neg_binomial)):
    register('_random_%s_like' % _n, inputs=('data',))(_like(_f))


def _bshape(p, shape):
    return tuple(p.shape) + _shape(shape)


def _expand(p, shape):
    s = _shape(shape)
    return p.reshape(tuple(p.shape) + (1,) * len(s)).expand(tuple(p.shape) + s)


@register('_sample_uniform', 'sample_uniform', inputs=('low', 'high'), defaults={'shape': (), 'dtype': None})
def sample_uniform(low, high, shape=(), dtype=None):
    lo, hi = _expand(low, shape), _expand(high, shape)
    return lo + (hi - lo) * torch.rand_like(lo)


@register('_sample_normal', 'sample_normal', inputs=('mu', 'sigma'), defaults={'shape': (), 'dtype': None})
def sample_normal(mu, sigma, shape=(), dtype=None):
    m, s = _expand(mu, shape), _expand(sigma, shape)
    return m + s * torch.randn_like(m)


@register('_sample_gamma', 'sample_gamma', inputs=('alpha', 'beta'), defaults={'shape': (), 'dtype': None})
def sample_gamma(alpha, beta, shape=(), dtype=None):
    a, b = _expand(alpha, shape), _expand(beta, shape)
    return torch._standard_gamma(a.contiguous().float()).to(alpha.dtype) * b


@register('_sample_exponential', 'sample_exponential', inputs=('lam',), defaults={'shape': (), 'dtype': None})
def sample_exponential(lam, shape=(), dtype=None):
    l = _expand(lam, shape)
    return -torch.log1p(-torch.rand_like(l)) / l


@register('_sample_poisson', 'sample_poisson', inputs=('lam',), defaults={'shape': (), 'dtype': None})
def sample_poisson(lam, shape=(), dtype=None):
    return torch.poisson(_expand(lam, shape).contiguous().float()).to(lam.dtype)


@register('_sample_negative_binomial', 'sample_negative_binomial', inputs=('k', 'p'), defaults={'shape': (), 'dtype': None})
def sample_negative_binomial(k, p, shape=(), dtype=None):
    kk, pp = _expand(k, shape).float(), _expand(p, shape).float()
    lam = torch._standard_gamma(kk.contiguous()) * ((1 - pp) / pp)
    return torch.poisson(lam).to(p.dtype)


@register('_sample_generalized_negative_binomial', 'sample_generalized_negative_binomial', inputs=('mu', 'alpha'),
          defaults={'shape': (), 'dtype': None})
def sample_gen_neg_binomial(mu, alpha, shape=(), dtype=None):
    m, a = _expand(mu, shape).float(), _expand(alpha, shape).float()
    lam = torch.where(a == 0, m, torch._standard_gamma((1.0 / a.clamp(min=1e-12)).contiguous()) * (a * m))
    return torch.poisson(lam).to(mu.dtype)


def _multinomial_nout(attrs):
    return 2 if attrs.get('get_prob') in (True, 'True', 1) else 1


@register('_sample_multinomial', 'sample_multinomial', inputs=('data',), nout=_multinomial_nout,
          defaults={'shape': (), 'get_prob': False, 'dtype': 'int32'})
def sample_multinomial(data, shape=(), get_prob=False, dtype='int32'):
    s = _shape(shape)
    n = 1
    for v in s:
        n *= v
    p2 = data.reshape(-1, data.shape[-1]).float()
    idx = torch.multinomial(p2, max(n, 1), replacement=True)
    out = idx.reshape(tuple(data.shape[:-1]) + s) if s else idx.reshape(tuple(data.shape[:-1]))
    res = out.to(to_torch_dtype(dtype))
    if get_prob:
        logp = torch.log(torch.gather(p2, 1, idx)).reshape(out.shape)
        return res, logp
    return res


@register('_shuffle', 'shuffle', '_npi_shuffle', inputs=('data',))
def shuffle(data):
    return data[torch.randperm(data.shape[0], device=data.device)]


@register('_sample_unique_zipfian', inputs=(), nout=2, defaults={'range_max': 1, 'shape': ()})
def sample_unique_zipfian(range_max=1, shape=()):
    import math
    import numpy as np
    n = _shape(shape)[-1]
    out, tries = [], 0
    seen = set()
    log_range = math.log(range_max + 1)
    while len(out) < n:
        v = int(math.exp(np.random.rand() * log_range)) - 1
        tries += 1
        if v not in seen and 0 <= v < range_max:
            seen.add(v)
            out.append(v)
    return torch.tensor([out], dtype=torch.int64), torch.tensor([tries], dtype=torch.int64)


# ---- numpy-style (mx.np.random) -----------------------------------------------------------------
def _np_shape(size):
    return () if size is None else _shape(size)


def _param(v, dev):
    return v if isinstance(v, torch.Tensor) else torch.as_tensor(float(v), device=dev)


@register('_npi_uniform', inputs=('low', 'high'), defaults={'size': None, 'ctx': None, 'dtype': 'float32'})
def npi_uniform(low=0.0, high=1.0, size=None, ctx=None, dtype='float32'):
    dev = low.device if isinstance(low, torch.Tensor) else high.device if isinstance(high, torch.Tensor) else _dev(ctx)
    lo, hi = _param(low, dev), _param(high, dev)
    shape = _np_shape(size) if size is not None else torch.broadcast_shapes(lo.shape, hi.shape)
    u = torch.rand(shape, device=dev, dtype=_dt(dtype))
    return lo.to(u.dtype) + (hi - lo).to(u.dtype) * u


@register('_npi_normal', inputs=('loc', 'scale'), defaults={'size': None, 'ctx': None, 'dtype': 'float32'})
def npi_normal(loc=0.0, scale=1.0, size=None, ctx=None, dtype='float32'):
    dev = loc.device if isinstance(loc, torch.Tensor) else scale.device if isinstance(scale, torch.Tensor) else _dev(ctx)
    m, s = _param(loc, dev), _param(scale, dev)
    shape = _np_shape(size) if size is not None else torch.broadcast_shapes(m.shape, s.shape)
    z = torch.randn(shape, device=dev, dtype=_dt(dtype))
    return m.to(z.dtype) + s.to(z.dtype) * z


@register('_npi_gamma', inputs=('shape_', 'scale'), defaults={'size': None, 'ctx': None, 'dtype': 'float32'})
def npi_gamma(shape_=1.0, scale=1.0, size=None, ctx=None, dtype='float32'):
    dev = shape_.device if isinstance(shape_, torch.Tensor) else _dev(ctx)
    a, b = _param(shape_, dev).float(), _param(scale, dev).float()
    shape = _np_shape(size) if size is not None else torch.broadcast_shapes(a.shape, b.shape)
    return (torch._standard_gamma(a.expand(shape).contiguous()) * b).to(_dt(dtype))


@register('_npi_exponential', inputs=('scale',), defaults={'size': None, 'ctx': None})
def npi_exponential(scale=1.0, size=None, ctx=None, dtype='float32'):
    dev = scale.device if isinstance(scale, torch.Tensor) else _dev(ctx)
    s = _param(scale, dev)
    shape = _np_shape(size) if size is not None else s.shape
    return -torch.log1p(-torch.rand(shape, device=dev)) * s


@register('_npi_bernoulli', inputs=('prob',), defaults={'logit': None, 'size': None, 'ctx': None, 'dtype': 'float32', 'is_logit': False})
def npi_bernoulli(prob=None, logit=None, size=None, ctx=None, dtype='float32', is_logit=False):
    p = prob if prob is not None else logit
    dev = p.device if isinstance(p, torch.Tensor) else _dev(ctx)
    p = _param(p, dev)
    if is_logit or (prob is None and logit is not None):
        p = torch.sigmoid(p)
    shape = _np_shape(size) if size is not None else p.shape
    return torch.bernoulli(p.expand(shape)).to(_dt(dtype))


@register('_npi_choice', inputs=('a', 'p'), defaults={'size': None, 'replace': True, 'ctx': None, 'weighted': False})
def npi_choice(a, p=None, size=None, replace=True, ctx=None, weighted=False):
    n = a if isinstance(a, int) else a.shape[0]
    shape = _np_shape(size)
    cnt = 1
    for s in shape:
        cnt *= s
    dev = p.device if p is not None else (a.device if isinstance(a, torch.Tensor) else _dev(ctx))
    if p is not None:
        idx = torch.multinomial(p.float(), cnt, replacement=replace)
    elif replace:
        idx = torch.randint(0, n, (cnt,), device=dev)
    else:
        idx = torch.randperm(n, device=dev)[:cnt]
    idx = idx.reshape(shape)
    return idx if isinstance(a, int) else a[idx]


@register('_npi_multinomial', inputs=('pvals',), defaults={'n': 1, 'size': None})
def npi_multinomial(pvals, n=1, size=None):
    import numpy as np
    p = pvals.detach().cpu().numpy().astype('float64')
    p = p / p.sum()
    return torch.from_numpy(np.random.multinomial(n, p, size=size)).to(pvals.device)


@register('_npi_randint', inputs=(), defaults={'low': 0, 'high': None, 'size': None, 'ctx': None, 'dtype': 'int64'})
def npi_randint(low=0, high=None, size=None, ctx=None, dtype='int64'):
    if high is None:
        low, high = 0, low
    return torch.randint(int(low), int(high), _np_shape(size), device=_dev(ctx)).to(to_torch_dtype(dtype or 'int64'))


def _np_dist(name, sampler):
    def op(*params, size=None, ctx=None, dtype='float32'):
        dev = next((p.device for p in params if isinstance(p, torch.Tensor)), _dev(ctx))
        ps = [_param(p, dev).float() for p in params]
        shape = _np_shape(size) if size is not None else torch.broadcast_shapes(*[p.shape for p in ps])
        u = torch.rand(shape, device=dev).clamp_(1e-12, 1 - 1e-7)
        return sampler(u, *ps)
    register('_npi_' + name, inputs=('*params',), defaults={'size': None, 'ctx': None})(op)


_np_dist('laplace', lambda u, loc, scale: loc - scale * torch.sign(u - 0.5) * torch.log1p(-2 * (u - 0.5).abs()))
_np_dist('gumbel', lambda u, loc, scale: loc - scale * torch.log(-torch.log(u)))
_np_dist('logistic', lambda u, loc, scale: loc + scale * (torch.log(u) - torch.log1p(-u)))
_np_dist('rayleigh', lambda u, scale: scale * torch.sqrt(-2 * torch.log1p(-u)))
_np_dist('weibull', lambda u, a: torch.pow(-torch.log1p(-u), 1.0 / a))
_np_dist('pareto', lambda u, a: torch.exp(-torch.log1p(-u) / a) - 1)
_np_dist('powerd', lambda u, a: torch.pow(u, 1.0 / a))      # _npi_powerd: `_npi_power` is the arithmetic operator


# ---- pdf ops (src/operator/random/pdf_op.cc) --------------------------------------------------
def _pdf(name, fn, nparam):
    def op(sample, *params, is_log=False):
        ps = [p.reshape(tuple(p.shape) + (1,) * (sample.dim() - p.dim())) for p in params]
        logp = fn(sample, *ps)
        return logp if is_log else torch.exp(logp)
    register('_random_pdf_' + name, 'random_pdf_' + name, inputs=('sample',) + tuple('p%d' % i for i in range(nparam)),
             defaults={'is_log': False})(op)


_pdf('uniform', lambda x, lo, hi: torch.where((x >= lo) & (x <= hi), -torch.log(hi - lo), torch.full_like(x, float('-inf'))), 2)
_pdf('normal', lambda x, mu, s: -0.5 * ((x - mu) / s) ** 2 - torch.log(s) - 0.9189385332046727, 2)
_pdf('gamma', lambda x, a, b: a * torch.log(b) + (a - 1) * torch.log(x) - b * x - torch.lgamma(a), 2)
_pdf('exponential', lambda x, lam: torch.log(lam) - lam * x, 1)
_pdf('poisson', lambda x, lam: x * torch.log(lam) - lam - torch.lgamma(x + 1), 1)
_pdf('negative_binomial', lambda x, k, p: torch.lgamma(x + k) - torch.lgamma(x + 1) - torch.lgamma(k)
     + k * torch.log(p) + x * torch.log1p(-p), 2)
_pdf('generalized_negative_binomial', lambda x, mu, a: torch.lgamma(x + 1 / a) - torch.lgamma(x + 1) - torch.lgamma(1 / a)
     - (1 / a) * torch.log1p(a * mu) + x * (torch.log(a * mu) - torch.log1p(a * mu)), 2)
_pdf('dirichlet', lambda x, a: ((a - 1) * torch.log(x)).sum(-1) + torch.lgamma(a.sum(-1)) - torch.lgamma(a).sum(-1), 1)

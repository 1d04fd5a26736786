"""Probability distributions over framework arrays.  Sampling and densities are differentiable
through autograd (reparameterised where the family allows); the math is delegated to the tensor
library's distribution kernels, wrapped so inputs/outputs are ``mx.np`` / ``mx.nd`` arrays."""
import torch
import torch.distributions as D

from ... import _state
from ...ndarray.ndarray import NDArray

__all__ = ['Distribution', 'ExponentialFamily', 'Normal', 'Bernoulli', 'Categorical', 'OneHotCategorical', 'Uniform',
           'Exponential', 'Gamma', 'Beta', 'Dirichlet', 'Laplace', 'Cauchy', 'HalfCauchy', 'HalfNormal', 'Poisson',
           'Geometric', 'NegativeBinomial', 'Binomial', 'Multinomial', 'MultivariateNormal', 'StudentT', 'Chi2',
           'FisherSnedecor', 'Gumbel', 'Weibull', 'Pareto', 'RelaxedBernoulli', 'RelaxedOneHotCategorical',
           'Independent', 'TransformedDistribution', 'kl_divergence', 'register_kl', 'empirical_kl']


def _t(x, like=None):
    if isinstance(x, NDArray):
        return x._data
    if x is None:
        return None
    dev = like.device if like is not None else None
    return torch.as_tensor(x, dtype=torch.float32, device=dev)


def _wrap(t, cls=None, ctx=None):
    if cls is None:
        if _state.state.np_array:
            from ...numpy.multiarray import ndarray as cls
        else:
            cls = NDArray
    return cls._from_tensor(t, ctx)


def _grad_ctx():
    return torch.enable_grad() if _state.state.recording else torch.no_grad()


class Distribution(object):
    """Base class.  Subclasses set ``self._d`` (the backing distribution) in ``__init__``."""
    has_grad = False
    has_enumerate_support = False
    arg_constraints = {}
    support = None

    def __init__(self, F=None, event_dim=None, validate_args=None):
        self.F = F
        self.event_dim = event_dim
        self._validate_args = validate_args
        self._cls, self._ctx = None, None

    def _setup(self, *args):
        for a in args:
            if isinstance(a, NDArray):
                self._cls, self._ctx = a.__class__, a._ctx
                return

    def _out(self, t):
        return _wrap(t, self._cls, self._ctx)

    def log_prob(self, value):
        with _grad_ctx():
            return self._out(self._d.log_prob(_t(value)))

    def pdf(self, value):
        with _grad_ctx():
            return self._out(self._d.log_prob(_t(value)).exp())

    prob = pdf

    def cdf(self, value):
        with _grad_ctx():
            return self._out(self._d.cdf(_t(value)))

    def icdf(self, value):
        with _grad_ctx():
            return self._out(self._d.icdf(_t(value)))

    def sample(self, size=None):
        shape = () if size is None else ((size,) if isinstance(size, int) else tuple(size))
        # `size` is the full output shape in the reference; batch shape is already part of the distribution
        bs = tuple(self._d.batch_shape) + tuple(self._d.event_shape)
        if shape and bs and shape[-len(bs):] == bs:
            shape = shape[:-len(bs)]
        with _grad_ctx():
            s = self._d.rsample(shape) if self._d.has_rsample else self._d.sample(shape)
        return self._out(s)

    def sample_n(self, size=None):
        shape = () if size is None else ((size,) if isinstance(size, int) else tuple(size))
        with _grad_ctx():
            s = self._d.rsample(shape) if self._d.has_rsample else self._d.sample(shape)
        return self._out(s)

    def broadcast_to(self, batch_shape):
        new = self.__class__.__new__(self.__class__)
        new.__dict__.update(self.__dict__)
        new._d = self._d.expand(torch.Size(batch_shape))
        return new

    def enumerate_support(self):
        return self._out(self._d.enumerate_support())

    @property
    def mean(self):
        return self._out(self._d.mean)

    @property
    def variance(self):
        return self._out(self._d.variance)

    @property
    def stddev(self):
        return self._out(self._d.stddev)

    def entropy(self):
        with _grad_ctx():
            return self._out(self._d.entropy())

    def perplexity(self):
        with _grad_ctx():
            return self._out(self._d.entropy().exp())

    @property
    def batch_shape(self):
        return tuple(self._d.batch_shape)

    @property
    def event_shape(self):
        return tuple(self._d.event_shape)

    def __repr__(self):
        return self.__class__.__name__ + '(' + repr(self._d) + ')'


class ExponentialFamily(Distribution):
    pass


def _simple(name, torch_cls, params, base=Distribution, doc=None):
    """Build a wrapper class whose constructor takes ``params`` (name → default)."""
    names = list(params)

    def __init__(self, *args, F=None, validate_args=None, **kwargs):
        vals = dict(params)
        for k, v in zip(names, args):
            vals[k] = v
        vals.update({k: v for k, v in kwargs.items() if k in vals})
        Distribution.__init__(self, F, None, validate_args)
        self._setup(*vals.values())
        first = next((_t(v) for v in vals.values() if isinstance(v, NDArray)), None)
        tv = {k: _t(v, first) for k, v in vals.items() if v is not None}
        with _grad_ctx():
            self._d = torch_cls(**{self._rename.get(k, k): v for k, v in tv.items()})
        for k, v in vals.items():
            setattr(self, k, v)
    cls = type(name, (base,), {'__init__': __init__, '_rename': {}, '__doc__': doc})
    return cls


Normal = _simple('Normal', D.Normal, {'loc': 0.0, 'scale': 1.0}, ExponentialFamily)
Laplace = _simple('Laplace', D.Laplace, {'loc': 0.0, 'scale': 1.0})
Cauchy = _simple('Cauchy', D.Cauchy, {'loc': 0.0, 'scale': 1.0})
HalfCauchy = _simple('HalfCauchy', D.HalfCauchy, {'scale': 1.0})
HalfNormal = _simple('HalfNormal', D.HalfNormal, {'scale': 1.0})
Uniform = _simple('Uniform', D.Uniform, {'low': 0.0, 'high': 1.0})
Gumbel = _simple('Gumbel', D.Gumbel, {'loc': 0.0, 'scale': 1.0})
Poisson = _simple('Poisson', D.Poisson, {'rate': 1.0}, ExponentialFamily)
Dirichlet = _simple('Dirichlet', D.Dirichlet, {'alpha': None}, ExponentialFamily)
Dirichlet._rename = {'alpha': 'concentration'}
Beta = _simple('Beta', D.Beta, {'alpha': 1.0, 'beta': 1.0}, ExponentialFamily)
Beta._rename = {'alpha': 'concentration1', 'beta': 'concentration0'}
Chi2 = _simple('Chi2', D.Chi2, {'df': 1.0})
StudentT = _simple('StudentT', D.StudentT, {'df': 1.0, 'loc': 0.0, 'scale': 1.0})
FisherSnedecor = _simple('FisherSnedecor', D.FisherSnedecor, {'df1': 1.0, 'df2': 1.0})
Weibull = _simple('Weibull', D.Weibull, {'concentration': 1.0, 'scale': 1.0})
Pareto = _simple('Pareto', D.Pareto, {'alpha': 1.0, 'scale': 1.0})
Pareto._rename = {'alpha': 'alpha', 'scale': 'scale'}


class Exponential(ExponentialFamily):
    def __init__(self, scale=1.0, F=None, validate_args=None):
        super().__init__(F, None, validate_args)
        self._setup(scale)
        self.scale = scale
        with _grad_ctx():
            self._d = D.Exponential(1.0 / _t(scale))


class Gamma(ExponentialFamily):
    def __init__(self, shape, scale=1.0, F=None, validate_args=None):
        super().__init__(F, None, validate_args)
        self._setup(shape, scale)
        self.shape, self.scale = shape, scale
        with _grad_ctx():
            s = _t(shape)
            self._d = D.Gamma(s, 1.0 / _t(scale, s))


def _prob_logit(prob, logit):
    if (prob is None) == (logit is None):
        raise ValueError('Either `prob` or `logit` must be specified, but not both. Received prob={}, logit={}'.format(prob, logit))


class Bernoulli(ExponentialFamily):
    has_enumerate_support = True

    def __init__(self, prob=None, logit=None, F=None, validate_args=None):
        _prob_logit(prob, logit)
        super().__init__(F, None, validate_args)
        self._setup(prob, logit)
        with _grad_ctx():
            self._d = D.Bernoulli(probs=_t(prob), logits=_t(logit))

    prob = property(lambda self: self._out(self._d.probs))
    logit = property(lambda self: self._out(self._d.logits))


class Geometric(Distribution):
    def __init__(self, prob=None, logit=None, F=None, validate_args=None):
        _prob_logit(prob, logit)
        super().__init__(F, None, validate_args)
        self._setup(prob, logit)
        with _grad_ctx():
            self._d = D.Geometric(probs=_t(prob), logits=_t(logit))


class Binomial(Distribution):
    def __init__(self, n=1, prob=None, logit=None, F=None, validate_args=None):
        _prob_logit(prob, logit)
        super().__init__(F, None, validate_args)
        self._setup(prob, logit)
        with _grad_ctx():
            self._d = D.Binomial(total_count=n, probs=_t(prob), logits=_t(logit))


class NegativeBinomial(Distribution):
    def __init__(self, n, prob=None, logit=None, F=None, validate_args=None):
        _prob_logit(prob, logit)
        super().__init__(F, None, validate_args)
        self._setup(n, prob, logit)
        with _grad_ctx():
            self._d = D.NegativeBinomial(total_count=_t(n), probs=_t(prob), logits=_t(logit))


class Categorical(Distribution):
    has_enumerate_support = True

    def __init__(self, num_events, prob=None, logit=None, F=None, validate_args=None):
        _prob_logit(prob, logit)
        super().__init__(F, None, validate_args)
        self._setup(prob, logit)
        self.num_events = num_events
        with _grad_ctx():
            self._d = D.Categorical(probs=_t(prob), logits=_t(logit))

    prob = property(lambda self: self._out(self._d.probs))
    logit = property(lambda self: self._out(self._d.logits))


class OneHotCategorical(Distribution):
    has_enumerate_support = True

    def __init__(self, num_events=None, prob=None, logit=None, F=None, validate_args=None):
        _prob_logit(prob, logit)
        super().__init__(F, None, validate_args)
        self._setup(prob, logit)
        self.num_events = num_events
        with _grad_ctx():
            self._d = D.OneHotCategorical(probs=_t(prob), logits=_t(logit))


class Multinomial(Distribution):
    def __init__(self, num_events, prob=None, logit=None, total_count=1, F=None, validate_args=None):
        _prob_logit(prob, logit)
        super().__init__(F, None, validate_args)
        self._setup(prob, logit)
        with _grad_ctx():
            self._d = D.Multinomial(total_count=total_count, probs=_t(prob), logits=_t(logit))


class RelaxedBernoulli(Distribution):
    has_grad = True

    def __init__(self, T, prob=None, logit=None, F=None, validate_args=None):
        _prob_logit(prob, logit)
        super().__init__(F, None, validate_args)
        self._setup(prob, logit)
        with _grad_ctx():
            self._d = D.RelaxedBernoulli(torch.as_tensor(float(T)) if not isinstance(T, NDArray) else T._data,
                                         probs=_t(prob), logits=_t(logit))


class RelaxedOneHotCategorical(Distribution):
    has_grad = True

    def __init__(self, T, num_events=None, prob=None, logit=None, F=None, validate_args=None):
        _prob_logit(prob, logit)
        super().__init__(F, None, validate_args)
        self._setup(prob, logit)
        with _grad_ctx():
            self._d = D.RelaxedOneHotCategorical(torch.as_tensor(float(T)) if not isinstance(T, NDArray) else T._data,
                                                 probs=_t(prob), logits=_t(logit))


class MultivariateNormal(Distribution):
    has_grad = True

    def __init__(self, loc, cov=None, precision=None, scale_tril=None, F=None, validate_args=None):
        if (cov is not None) + (precision is not None) + (scale_tril is not None) != 1:
            raise ValueError('Exactly one onf `cov` or `precision` or `scale_tril` may be specified')
        super().__init__(F, 1, validate_args)
        self._setup(loc, cov, precision, scale_tril)
        with _grad_ctx():
            self._d = D.MultivariateNormal(_t(loc), covariance_matrix=_t(cov), precision_matrix=_t(precision),
                                           scale_tril=_t(scale_tril))


class Independent(Distribution):
    """Reinterpret the right-most batch dimensions as event dimensions."""

    def __init__(self, base_distribution, reinterpreted_batch_ndims, validate_args=None):
        super().__init__(None, None, validate_args)
        self._cls, self._ctx = base_distribution._cls, base_distribution._ctx
        self.base_dist = base_distribution
        self._d = D.Independent(base_distribution._d, reinterpreted_batch_ndims)


class TransformedDistribution(Distribution):
    def __init__(self, base_dist, transforms, validate_args=None):
        super().__init__(None, None, validate_args)
        self._cls, self._ctx = base_dist._cls, base_dist._ctx
        if not isinstance(transforms, (list, tuple)):
            transforms = [transforms]
        self._base_dist, self._transforms = base_dist, list(transforms)
        self._d = D.TransformedDistribution(base_dist._d, [t._t for t in transforms])


_KL = {}


def register_kl(typeP, typeQ):
    def deco(fn):
        _KL[(typeP, typeQ)] = fn
        return fn
    return deco


def kl_divergence(p, q):
    """KL(p || q): registered closed forms, else the tensor library's table of closed forms."""
    for (tp, tq), fn in _KL.items():
        if isinstance(p, tp) and isinstance(q, tq):
            return fn(p, q)
    with _grad_ctx():
        try:
            return p._out(D.kl_divergence(p._d, q._d))
        except NotImplementedError:
            raise NotImplementedError('KL divergence between {} and {} is not implemented.'.format(
                type(p).__name__, type(q).__name__))


def empirical_kl(p, q, n_samples=1):
    samples = p.sample_n((n_samples,))
    return (p.log_prob(samples) - q.log_prob(samples)).mean(0)

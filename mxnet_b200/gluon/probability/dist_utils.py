"""Helpers of the distribution classes (``python/mxnet/gluon/probability/distributions/utils.py``)."""
import numpy as _onp

__all__ = ['prob2logit', 'logit2prob', 'cached_property', 'sample_n_shape_converter', 'constraint_check', 'digamma', 'gammaln',
           'erfinv', 'erf']


def _np():
    from ... import numpy as mxnp
    return mxnp


def _npx():
    from ... import numpy_extension as npx
    return npx


def constraint_check():
    """The function used to validate a condition: ``f(condition, message)`` returns a true scalar or raises ValueError."""
    def check(condition, err_msg):
        return _npx().constraint_check(condition, err_msg)
    return check


def digamma():
    return lambda x: _npx().digamma(x)


def gammaln():
    return lambda x: _npx().gammaln(x)


def erf():
    return lambda x: _npx().erf(x)


def erfinv():
    return lambda x: _npx().erfinv(x)


def sample_n_shape_converter(size):
    """Shape argument of ``sample_n``: None -> (), an int -> (int,), (-2,)-style placeholders pass through."""
    if size is None:
        return ()
    if size == ():
        return ()
    if isinstance(size, int):
        size = (size,)
    return tuple(size)


def _clip_prob(prob):
    eps = _onp.finfo('float32').eps
    return _np().clip(prob, eps, 1 - eps)


def _clip_float_eps(value):
    eps = _onp.finfo('float32').eps
    return _np().maximum(value, eps)


def prob2logit(prob, binary=True):
    """Probabilities -> logits: log(p / (1 - p)) for binary variables, log(p) for categorical ones."""
    np_ = _np()
    clipped = _clip_prob(prob)
    if binary:
        return np_.log(clipped) - np_.log1p(-clipped)
    return np_.log(clipped)


def logit2prob(logit, binary=True):
    """Logits -> probabilities: sigmoid for binary variables, softmax over the last axis for categorical ones."""
    if binary:
        return _npx().sigmoid(logit)
    return _npx().softmax(logit)


class cached_property(object):   # pylint: disable=invalid-name
    """A property computed on first access and then stored on the instance."""

    def __init__(self, func):
        self._func = func
        self.__doc__ = func.__doc__

    def __get__(self, instance, cls=None):
        if instance is None:
            return self
        value = self._func(instance)
        setattr(instance, self._func.__name__, value)
        return value

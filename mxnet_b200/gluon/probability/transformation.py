"""Bijective transformations for ``TransformedDistribution`` (``gluon/probability/transformation``)."""
import torch
import torch.distributions.transforms as T

from ...ndarray.ndarray import NDArray
from .distributions import _t, _wrap, _grad_ctx

__all__ = ['Transformation', 'TransformBlock', 'ComposeTransform', 'ExpTransform', 'AffineTransform', 'PowerTransform',
           'AbsTransform', 'SigmoidTransform', 'SoftmaxTransform', 'domain_map', 'biject_to', 'transform_to']


class Transformation(object):
    bijective = False
    event_dim = 0

    def __init__(self, F=None):
        self._F = F
        self._inv = None

    def __call__(self, x):
        with _grad_ctx():
            return _wrap(self._t(_t(x)), x.__class__ if isinstance(x, NDArray) else None, getattr(x, '_ctx', None))

    def _inverse_compute(self, y):
        with _grad_ctx():
            return _wrap(self._t.inv(_t(y)), y.__class__ if isinstance(y, NDArray) else None, getattr(y, '_ctx', None))

    def log_det_jacobian(self, x, y):
        with _grad_ctx():
            return _wrap(self._t.log_abs_det_jacobian(_t(x), _t(y)), x.__class__ if isinstance(x, NDArray) else None,
                         getattr(x, '_ctx', None))

    @property
    def inv(self):
        if self._inv is None:
            self._inv = _Inverse(self)
        return self._inv

    @property
    def sign(self):
        return self._t.sign


class _Inverse(Transformation):
    def __init__(self, fwd):
        super().__init__()
        self._fwd = fwd
        self._t = fwd._t.inv

    @property
    def inv(self):
        return self._fwd


class TransformBlock(Transformation):
    pass


class ExpTransform(Transformation):
    bijective = True

    def __init__(self):
        super().__init__()
        self._t = T.ExpTransform()


class AffineTransform(Transformation):
    bijective = True

    def __init__(self, loc, scale, event_dim=0):
        super().__init__()
        self._t = T.AffineTransform(_t(loc), _t(scale), event_dim)


class PowerTransform(Transformation):
    bijective = True

    def __init__(self, exponent):
        super().__init__()
        self._t = T.PowerTransform(_t(exponent))


class AbsTransform(Transformation):
    def __init__(self):
        super().__init__()
        self._t = T.AbsTransform()


class SigmoidTransform(Transformation):
    bijective = True

    def __init__(self):
        super().__init__()
        self._t = T.SigmoidTransform()


class SoftmaxTransform(Transformation):
    event_dim = 1

    def __init__(self):
        super().__init__()
        self._t = T.SoftmaxTransform()


class ComposeTransform(Transformation):
    def __init__(self, parts):
        super().__init__()
        self._parts = parts
        self._t = T.ComposeTransform([p._t for p in parts])


class domain_map(object):   # pylint: disable=invalid-name
    def __init__(self):
        self._storage = {}

    def register(self, constraint, factory=None):
        if factory is None:
            return lambda f: self.register(constraint, f)
        self._storage[constraint] = factory
        return factory

    def __call__(self, constraint):
        return self._storage[type(constraint) if not isinstance(constraint, type) else constraint](constraint)


biject_to = domain_map()
transform_to = domain_map()

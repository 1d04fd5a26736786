"""Regions over which distribution parameters and samples are valid
(``python/mxnet/gluon/probability/distributions/constraint.py``).  ``check(value)`` returns the value when every element
lies in the region and raises ``ValueError`` otherwise."""
import numpy as _onp

__all__ = ['Constraint', 'Real', 'Boolean', 'Interval', 'OpenInterval', 'HalfOpenInterval', 'UnitInterval', 'IntegerInterval',
           'IntegerOpenInterval', 'IntegerHalfOpenInterval', 'GreaterThan', 'GreaterThanEq', 'IntegerGreaterThan',
           'IntegerGreaterThanEq', 'LessThan', 'LessThanEq', 'IntegerLessThan', 'IntegerLessThanEq', 'Positive', 'NonNegative',
           'PositiveInteger', 'NonNegativeInteger', 'Simplex', 'LowerTriangular', 'LowerCholesky', 'PositiveDefinite', 'Cat', 'Stack',
           'is_dependent', 'dependent', 'dependent_property']


def _np(value):
    return value.asnumpy() if hasattr(value, 'asnumpy') else _onp.asarray(value)


class Constraint(object):
    """Base class: a region over which a variable is valid."""

    def check(self, value):
        raise NotImplementedError

    def _verify(self, value, condition, message):
        if not bool(_onp.all(condition)):
            raise ValueError(message)
        return value


class _Dependent(Constraint):
    """Placeholder for variables whose support depends on other variables."""

    def check(self, value):
        raise ValueError('Cannot validate dependent constraint')


def is_dependent(constraint):
    return isinstance(constraint, _Dependent)


class _DependentProperty(property, _Dependent):
    """``@property`` that reads as a dependent constraint on the class and as the property on an instance."""


dependent = _Dependent()
dependent_property = _DependentProperty


class Real(Constraint):
    def check(self, value):
        v = _np(value)
        return self._verify(value, v == v, 'Constraint violated: {} should be a real tensor'.format(value))


class Boolean(Constraint):
    def check(self, value):
        v = _np(value)
        return self._verify(value, (v == 0) | (v == 1), 'Constraint violated: {} should be either 0 or 1.'.format(value))


class _Bounded(Constraint):
    _integer = False

    def _int_ok(self, v):
        return (v % 1 == 0) if self._integer else True

    def _kind(self):
        return 'integer ' if self._integer else ''


class Interval(_Bounded):
    """lower <= value <= upper"""

    def __init__(self, lower_bound, upper_bound):
        self._lower, self._upper = lower_bound, upper_bound

    def _inside(self, v):
        return (v >= self._lower) & (v <= self._upper)

    _text = 'be >= {lo} and <= {hi}'

    def check(self, value):
        v = _np(value)
        msg = 'Constraint violated: {} should be {}'.format(value, self._kind()) + self._text.format(lo=self._lower, hi=self._upper)
        return self._verify(value, self._inside(v) & self._int_ok(v), msg)


class OpenInterval(Interval):
    """lower < value < upper"""
    _text = 'be > {lo} and < {hi}'

    def _inside(self, v):
        return (v > self._lower) & (v < self._upper)


class HalfOpenInterval(Interval):
    """lower <= value < upper"""
    _text = 'be >= {lo} and < {hi}'

    def _inside(self, v):
        return (v >= self._lower) & (v < self._upper)


class UnitInterval(Interval):
    def __init__(self):
        super().__init__(0, 1)


class IntegerInterval(Interval):
    _integer = True


class IntegerOpenInterval(OpenInterval):
    _integer = True


class IntegerHalfOpenInterval(HalfOpenInterval):
    _integer = True


class GreaterThan(_Bounded):
    def __init__(self, lower_bound):
        self._lower = lower_bound

    def _inside(self, v):
        return v > self._lower

    _text = 'be greater than {b}'

    def check(self, value):
        v = _np(value)
        bound = getattr(self, '_lower', None) if hasattr(self, '_lower') else self._upper
        msg = 'Constraint violated: {} should {}'.format(value, self._kind()) + self._text.format(b=bound)
        return self._verify(value, self._inside(v) & self._int_ok(v), msg)


class GreaterThanEq(GreaterThan):
    _text = 'be greater than or equal to {b}'

    def _inside(self, v):
        return v >= self._lower


class IntegerGreaterThan(GreaterThan):
    _integer = True


class IntegerGreaterThanEq(GreaterThanEq):
    _integer = True


class LessThan(GreaterThan):
    _text = 'be less than {b}'

    def __init__(self, upper_bound):   # pylint: disable=super-init-not-called
        self._upper = upper_bound

    def _inside(self, v):
        return v < self._upper


class LessThanEq(LessThan):
    _text = 'be less than or equal to {b}'

    def _inside(self, v):
        return v <= self._upper


class IntegerLessThan(LessThan):
    _integer = True


class IntegerLessThanEq(LessThanEq):
    _integer = True


class Positive(GreaterThan):
    def __init__(self):
        super().__init__(0)


class NonNegative(GreaterThanEq):
    def __init__(self):
        super().__init__(0)


class PositiveInteger(IntegerGreaterThan):
    def __init__(self):
        super().__init__(0)


class NonNegativeInteger(IntegerGreaterThanEq):
    def __init__(self):
        super().__init__(0)


class Simplex(Constraint):
    """Non-negative entries whose last axis sums to one."""

    def check(self, value):
        v = _np(value)
        ok = (v >= 0).all() and (_onp.abs(v.sum(-1) - 1) < 1e-6).all()
        return self._verify(value, ok, 'Constraint violated: {} should be >= 0 and its rightmost dimension should sum up to 1'.format(value))


class LowerTriangular(Constraint):
    def check(self, value):
        v = _np(value)
        return self._verify(value, _onp.tril(v) == v, 'Constraint violated: {} should be square lower triangular matrices'.format(value))


class LowerCholesky(Constraint):
    """Lower triangular with a positive diagonal."""

    def check(self, value):
        v = _np(value)
        ok = (_onp.tril(v) == v).all() and (_onp.diagonal(v, axis1=-2, axis2=-1) > 0).all()
        return self._verify(value, ok, 'Constraint violated: {} should be square lower triangular matrices '
                                       'with real and positive diagonal entries'.format(value))


class PositiveDefinite(Constraint):
    def check(self, value):
        v = _np(value)
        sym = _onp.abs(v - _onp.swapaxes(v, -1, -2)) < 1e-6
        ok = sym.all() and (_onp.linalg.eigvalsh(v) > 0).all()
        return self._verify(value, ok, 'Constraint violated: {} should be positive definite matrices'.format(value))


class Cat(Constraint):
    """Apply a sequence of constraints to consecutive slices (of the given lengths) along ``axis``."""

    def __init__(self, constraint_seq, axis=0, lengths=None):
        assert all(isinstance(c, Constraint) for c in constraint_seq)
        self._constraints = list(constraint_seq)
        self._lengths = list(lengths) if lengths is not None else [1] * len(self._constraints)
        assert len(self._lengths) == len(self._constraints), 'The number of lengths {} should be equal to number of ' \
            'constraints {}'.format(len(self._lengths), len(self._constraints))
        self._axis = axis

    def check(self, value):
        start = 0
        for constraint, length in zip(self._constraints, self._lengths):
            index = [slice(None)] * value.ndim
            index[self._axis] = slice(start, start + length)
            constraint.check(value[tuple(index)])
            start += length
        return value


class Stack(Constraint):
    """Apply the i-th constraint to the i-th entry along ``axis``."""

    def __init__(self, constraint_seq, axis=0):
        assert all(isinstance(c, Constraint) for c in constraint_seq)
        self._constraints, self._axis = list(constraint_seq), axis

    def check(self, value):
        assert value.shape[self._axis] == len(self._constraints)
        for i, constraint in enumerate(self._constraints):
            index = [slice(None)] * value.ndim
            index[self._axis] = i
            constraint.check(value[tuple(index)])
        return value

"""``mx.random``: global seed plus the legacy sampling front ends (``python/mxnet/random.py``)."""
from .ops.random import seed
from .ndarray.random import (uniform, normal, randn, poisson, exponential, gamma, multinomial, negative_binomial,
                             generalized_negative_binomial, shuffle, randint)

from .ndarray import random as _ndr

binomial = getattr(_ndr, 'binomial', None)
categorical = getattr(_ndr, 'categorical', None)

__all__ = ['seed', 'uniform', 'normal', 'randn', 'poisson', 'exponential', 'gamma', 'multinomial',
           'negative_binomial', 'generalized_negative_binomial', 'shuffle', 'randint', 'binomial', 'categorical']

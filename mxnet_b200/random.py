"""``mx.random``: global seed plus the legacy sampling front ends (``python/mxnet/random.py``)."""
from .ops.random import seed
from .ndarray.random import (uniform, normal, randn, poisson, exponential, gamma, multinomial, negative_binomial,
                             generalized_negative_binomial, shuffle, randint)

__all__ = ['seed', 'uniform', 'normal', 'randn', 'poisson', 'exponential', 'gamma', 'multinomial',
           'negative_binomial', 'generalized_negative_binomial', 'shuffle', 'randint']

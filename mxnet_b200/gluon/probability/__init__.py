"""``gluon.probability``: distributions, transformations, KL divergence, ``StochasticBlock``
(``python/mxnet/gluon/probability``)."""
from .distributions import *     # noqa: F401,F403
from .transformation import *    # noqa: F401,F403
from .block import StochasticBlock, StochasticSequential
from . import distributions, transformation

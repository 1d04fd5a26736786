"""``gluon.probability``: distributions, transformations, KL divergence, ``StochasticBlock``
(``python/mxnet/gluon/probability``)."""
from .distributions import *     # noqa: F401,F403
from .transformation import *    # noqa: F401,F403
from .block import StochasticBlock, StochasticSequential
from . import distributions, transformation
from . import constraint, dist_utils as utils   # noqa: E402
import sys as _sys   # noqa: E402

# the reference keeps these as sub-modules of the distributions package
distributions.constraint, distributions.utils = constraint, utils
_sys.modules[distributions.__name__ + '.constraint'] = constraint
_sys.modules[distributions.__name__ + '.utils'] = utils

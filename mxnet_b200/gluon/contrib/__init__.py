"""``gluon.contrib``: the estimator API and contributed data loaders / transforms."""
from . import estimator   # noqa: F401
from . import data        # noqa: F401

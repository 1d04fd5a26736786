"""``gluon.contrib``."""
from . import estimator

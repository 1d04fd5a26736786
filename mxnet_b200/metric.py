"""``mx.metric``: legacy alias of ``mx.gluon.metric``."""
from .gluon.metric import *        # noqa: F401,F403
from .gluon.metric import create, register, alias, EvalMetric, CompositeEvalMetric

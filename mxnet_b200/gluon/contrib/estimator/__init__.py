"""Keras-like training loop (``python/mxnet/gluon/contrib/estimator``)."""
from .estimator import Estimator
from .event_handler import *   # noqa: F401,F403
from .batch_processor import BatchProcessor

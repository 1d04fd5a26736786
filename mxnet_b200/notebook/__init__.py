"""Helpers for interactive sessions (``python/mxnet/notebook``): training callbacks that collect metrics into pandas
tables and, where bokeh is installed, draw live charts."""
from . import callback   # noqa: F401

"""Deferred-compute tracing entry points (``python/mxnet/_deferred_compute.py:27-109``)."""
import contextlib

from . import _state
from .symbol import _trace


def is_deferred_compute():
    return _state.state.tracer is not None


@contextlib.contextmanager
def context(state=True):
    """Scope in which executed operators are also recorded into a graph."""
    prev = _state.state.tracer
    _state.state.tracer = _trace.Tracer() if state else None
    try:
        yield _state.state.tracer
    finally:
        _state.state.tracer = prev


def set_variable(arrays, variables):
    """Associate arrays with variable symbols so the traced graph treats them as inputs."""
    tr = _state.state.tracer
    if not isinstance(arrays, (list, tuple)):
        arrays, variables = [arrays], [variables]
    for a, v in zip(arrays, variables):
        tr.set_variable(a, v)


def get_symbol(output_arrays, *, sym_cls=None):
    tr = _state.state.tracer
    single = not isinstance(output_arrays, (list, tuple))
    outs = [output_arrays] if single else list(output_arrays)
    return tr.get_symbol(outs)

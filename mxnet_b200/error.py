"""Structured error classes (reference: ``python/mxnet/error.py``).

Native errors are turned into the most specific Python class by a "Kind: message" prefix
convention; :func:`register_error` lets extensions add their own kinds.
"""
from .base import MXNetError

__all__ = ['MXNetError', 'InternalError', 'register_error', 'register', 'translate']

_ERROR_TYPES = {}


def register_error(func_name=None, cls=None):
    """Register an error class so that it can be recognised by name in native messages."""
    if callable(func_name):
        cls, func_name = func_name, func_name.__name__

    def _do(mycls):
        _ERROR_TYPES[func_name if isinstance(func_name, str) else mycls.__name__] = mycls
        return mycls
    return _do(cls) if cls is not None else _do


register = register_error


@register_error
class InternalError(MXNetError):
    """Internal invariant violated; the message asks the user to file a report."""

    def __init__(self, msg):
        if 'hint:' not in msg:
            msg += ('\nhint: you hit an internal error; please report it with the stack trace.')
        super().__init__(msg)


for _n, _c in (('ValueError', ValueError), ('TypeError', TypeError), ('AttributeError', AttributeError),
               ('IndexError', IndexError), ('NotImplementedError', NotImplementedError),
               ('IOError', IOError), ('FloatingPointError', FloatingPointError),
               ('RuntimeError', RuntimeError)):
    register_error(_n, _c)


def translate(message):
    """Map a native "Kind: text" message onto a registered exception instance."""
    head, sep, tail = message.partition(':')
    cls = _ERROR_TYPES.get(head.strip()) if sep else None
    if cls is None:
        return MXNetError(message)
    return cls(tail.strip())

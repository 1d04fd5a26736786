"""Attribute scoping for symbols (``python/mxnet/attribute.py``)."""
import threading

__all__ = ['AttrScope']


class AttrScope(object):
    _current = threading.local()

    def __init__(self, **kwargs):
        self._old_scope = None
        for v in kwargs.values():
            if not isinstance(v, str):
                raise ValueError('Attributes need to be string')
        self._attr = kwargs

    def get(self, attr):
        if self._attr:
            ret = self._attr.copy()
            if attr:
                ret.update(attr)
            return ret
        return attr if attr else {}

    def __enter__(self):
        self._old_scope = AttrScope.current()
        attr = self._old_scope._attr.copy()
        attr.update(self._attr)
        self._attr = attr
        AttrScope._current.value = self
        return self

    def __exit__(self, ptype, value, trace):
        AttrScope._current.value = self._old_scope

    @staticmethod
    def current():
        v = getattr(AttrScope._current, 'value', None)
        if v is None:
            v = AttrScope._current.value = AttrScope()
        return v


def current():
    """The AttrScope in effect for the calling thread."""
    return AttrScope.current()

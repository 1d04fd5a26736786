"""Automatic symbol naming (``python/mxnet/name.py``)."""
import threading

__all__ = ['NameManager', 'Prefix']


class NameManager(object):
    _current = threading.local()

    def __init__(self):
        self._counter = {}
        self._old_manager = None

    def get(self, name, hint):
        if name:
            return name
        if hint not in self._counter:
            self._counter[hint] = 0
        name = '%s%d' % (hint, self._counter[hint])
        self._counter[hint] += 1
        return name

    def __enter__(self):
        self._old_manager = getattr(NameManager._current, 'value', None)
        NameManager._current.value = self
        return self

    def __exit__(self, ptype, value, trace):
        NameManager._current.value = self._old_manager

    @staticmethod
    def current():
        v = getattr(NameManager._current, 'value', None)
        if v is None:
            v = NameManager._current.value = NameManager()
        return v


class Prefix(NameManager):
    def __init__(self, prefix):
        super().__init__()
        self._prefix = prefix

    def get(self, name, hint):
        return self._prefix + super().get(name, hint)


def current():
    """The NameManager in effect for the calling thread."""
    return NameManager.current()

"""Tensor inspector: look into an array while debugging (reference: ``src/common/tensor_inspector.h``: ``print_string``,
``check_value`` with predefined checkers, ``dump_to_file``, visit counters per tag).

    from mxnet_b200.inspector import TensorInspector, CheckerType
    ti = TensorInspector(arr)
    print(ti.to_string())
    bad = ti.check_value(CheckerType.NaNChecker)        # list of coordinates
    ti.dump_to_file('conv1_out')                        # conv1_out_1.npy, conv1_out_2.npy, ...

Values are brought to the host for inspection (a debugging tool; it synchronises the device).
"""
import enum
import os
import threading

import numpy as np

__all__ = ['TensorInspector', 'CheckerType']


class CheckerType(enum.Enum):
    NegativeChecker = 'negative'
    PositiveChecker = 'positive'
    ZeroChecker = 'zero'
    NaNChecker = 'nan'
    InfChecker = 'inf'
    PositiveInfChecker = 'positive inf'
    NegativeInfChecker = 'negative inf'
    FiniteChecker = 'finite'
    NormalChecker = 'normal'
    AbnormalChecker = 'abnormal'


def _normal(v):
    """Finite, non-zero and not subnormal."""
    if not np.issubdtype(v.dtype, np.floating):
        return v != 0
    tiny = np.finfo(v.dtype).tiny
    return np.isfinite(v) & (np.abs(v) >= tiny)


_CHECKERS = {
    CheckerType.NegativeChecker: lambda v: v < 0,
    CheckerType.PositiveChecker: lambda v: v > 0,
    CheckerType.ZeroChecker: lambda v: v == 0,
    CheckerType.NaNChecker: np.isnan,
    CheckerType.InfChecker: np.isinf,
    CheckerType.PositiveInfChecker: np.isposinf,
    CheckerType.NegativeInfChecker: np.isneginf,
    CheckerType.FiniteChecker: np.isfinite,
    CheckerType.NormalChecker: _normal,
    CheckerType.AbnormalChecker: lambda v: ~_normal(v),
}

_visits = {}
_visits_lock = threading.Lock()


class TensorInspector(object):
    def __init__(self, array):
        self._array = array
        values = array.asnumpy() if hasattr(array, 'asnumpy') else np.asarray(array)
        self._values = values.astype('float32') if values.dtype.name == 'bfloat16' else values

    # ---- printing ---------------------------------------------------------------------------------------------
    def info_string(self):
        a = self._array
        ctx = getattr(a, 'context', 'cpu(0)')
        return '<%s Tensor %s on %s>' % (self._values.dtype.name, 'x'.join(str(d) for d in self._values.shape) or 'scalar', ctx)

    def to_string(self, max_items=1000):
        """The values (row by row, abbreviated beyond ``max_items``) followed by the type / shape / device line."""
        with np.printoptions(threshold=max_items, linewidth=120):
            return '%s\n%s' % (np.array2string(self._values, separator=', '), self.info_string())

    print_string = to_string

    # ---- checking ---------------------------------------------------------------------------------------------
    def check_value(self, checker, interactive=False, tag=None):
        """Coordinates of the entries for which ``checker`` holds: a :class:`CheckerType` or a function value -> bool
        applied elementwise.  ``interactive`` is accepted for parity; the coordinates are returned either way."""
        fn = _CHECKERS.get(checker) if isinstance(checker, CheckerType) else None
        if fn is None:
            if not callable(checker):
                raise TypeError('checker must be a CheckerType or a callable')
            fn = np.vectorize(checker, otypes=[bool])
        hits = np.argwhere(fn(self._values))
        coords = [tuple(int(i) for i in c) for c in hits]
        if interactive and coords:
            print('%s: %d entries flagged by %s, first at %s' % (tag or self.info_string(), len(coords),
                                                                 getattr(checker, 'name', 'the checker'), coords[0]))
        return coords

    # ---- dumping ----------------------------------------------------------------------------------------------
    def dump_to_file(self, tag, directory='.'):
        """Write the values as ``<tag>_<n>.npy`` where ``n`` counts the dumps made under this tag in this process; returns
        the file name."""
        with _visits_lock:
            n = _visits[tag] = _visits.get(tag, 0) + 1
        fname = os.path.join(directory, '%s_%d.npy' % (tag, n))
        np.save(fname, self._values)
        return fname

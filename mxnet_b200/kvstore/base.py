"""Plug-in interface of the key-value stores (API of ``python/mxnet/kvstore/base.py``): the abstract ``KVStoreBase``,
its class registry (``KVStoreBase.register`` -> ``kv_registry``, looked up by lower-cased class name in ``create``),
and ``TestStore``, an in-process store without optimizer capability that the Trainer tests use as a stand-in for
Horovod-like back ends.
"""
from ..ndarray.ndarray import NDArray

__all__ = ['KVStoreBase', 'TestStore', 'create']


def _listify(x):
    return list(x) if isinstance(x, (list, tuple)) else [x]


def _ctype_key_value(keys, vals):
    """``(keys, values)`` as two equally long lists (a single key with a single value becomes lists of one)."""
    if not isinstance(keys, (tuple, list)):
        return [keys], [vals]
    if len(keys) != len(vals):
        raise AssertionError('keys and values differ in length')
    return list(keys), list(vals)


def _abstract(*_args, **_kwargs):
    raise NotImplementedError()


class KVStoreBase(object):
    """What a store must offer to a Trainer: ``broadcast`` (initial values), ``pushpull`` (reduce over devices and
    workers, then deliver), and, when ``is_capable(OPTIMIZER)``, running the optimizer where the reduced value lives."""

    OPTIMIZER = 'optimizer'
    kv_registry = {}

    broadcast = _abstract            # (key, value, out, priority=0)
    pushpull = _abstract             # (key, value, out=None, priority=0)
    set_optimizer = _abstract        # (optimizer)
    save_optimizer_states = _abstract    # (fname, dump_optimizer=False)
    load_optimizer_states = _abstract    # (fname)
    is_capable = staticmethod(_abstract)     # (capability) -> bool
    type = property(_abstract)
    rank = property(_abstract)
    num_workers = property(_abstract)

    @staticmethod
    def register(klass):
        """Class decorator: make ``klass`` available to ``create`` under its lower-cased name."""
        if not isinstance(klass, type):
            raise AssertionError('register expects a class')
        KVStoreBase.kv_registry[klass.__name__.lower()] = klass
        return klass


@KVStoreBase.register
class TestStore(KVStoreBase):
    """Single-worker store for tests: ``pushpull`` sums the values of the devices; no optimizer on the store."""

    type = property(lambda self: 'teststore')
    rank = property(lambda self: 0)
    num_workers = property(lambda self: 1)

    @staticmethod
    def is_capable(capability):
        if capability.lower() != KVStoreBase.OPTIMIZER:
            raise ValueError('Unknown capability: {}'.format(capability))
        return False

    def broadcast(self, key, value, out, priority=0):
        src = _listify(value)[0]
        for dst in _listify(out):
            dst[:] = src

    def pushpull(self, key, value, out=None, priority=0):
        values = _listify(value)
        total = values[0]
        if len(values) > 1:
            total = values[0].copy()
            for v in values[1:]:
                total += v.as_in_context(total.context)
        for dst in (_listify(out) if out is not None else values):
            if dst is not total:
                dst[:] = total.as_in_context(dst.context)

    def set_optimizer(self, optimizer):
        raise NotImplementedError('TestStore does not support optimizer on the store')


def create(name='local'):
    """A store by name: ``local``, ``device``, ``nccl``, the ``dist_*`` family, ``horovod``, ``byteps``, or the
    lower-cased class name of any registered plug-in."""
    if not isinstance(name, str):
        raise TypeError('name must be a string')
    plugin = KVStoreBase.kv_registry.get(name.lower())
    if plugin is not None:
        return plugin()
    from .kvstore import KVStore
    return KVStore(name.lower())

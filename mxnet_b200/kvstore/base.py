"""KVStore plug-in base class, registry and the pure-Python ``TestStore``
(``python/mxnet/kvstore/base.py:243-459``)."""
from ..ndarray.ndarray import NDArray

__all__ = ['KVStoreBase', 'TestStore', 'create']


def _ctype_key_value(keys, vals):
    if isinstance(keys, (tuple, list)):
        assert len(keys) == len(vals)
        return list(keys), list(vals)
    return [keys], [vals]


class KVStoreBase(object):
    """Abstract key-value store for data-parallel parameter synchronisation."""
    kv_registry = {}
    OPTIMIZER = 'optimizer'

    def broadcast(self, key, value, out, priority=0):
        raise NotImplementedError()

    def pushpull(self, key, value, out=None, priority=0):
        raise NotImplementedError()

    def set_optimizer(self, optimizer):
        raise NotImplementedError()

    @staticmethod
    def is_capable(capability):
        raise NotImplementedError()

    def save_optimizer_states(self, fname, dump_optimizer=False):
        raise NotImplementedError()

    def load_optimizer_states(self, fname):
        raise NotImplementedError()

    @property
    def type(self):
        raise NotImplementedError()

    @property
    def rank(self):
        raise NotImplementedError()

    @property
    def num_workers(self):
        raise NotImplementedError()

    @staticmethod
    def register(klass):
        assert isinstance(klass, type)
        name = klass.__name__.lower()
        KVStoreBase.kv_registry[name] = klass
        return klass


@KVStoreBase.register
class TestStore(KVStoreBase):
    """In-process fake used to test Trainer logic: sums values, no optimizer capability."""

    def broadcast(self, key, value, out, priority=0):
        out = out if isinstance(out, list) else [out]
        v = value[0] if isinstance(value, (list, tuple)) else value
        for o in out:
            o[:] = v

    def pushpull(self, key, value, out=None, priority=0):
        values = value if isinstance(value, list) else [value]
        ctx = values[0].context
        reduced = sum([v.as_in_context(ctx) for v in values[1:]], values[0].copy()) if len(values) > 1 else values[0]
        if out is None:
            for v in values:
                if v is not reduced:
                    v[:] = reduced.as_in_context(v.context)
            return
        outs = out if isinstance(out, list) else [out]
        for o in outs:
            o[:] = reduced.as_in_context(o.context)

    @staticmethod
    def is_capable(capability):
        if capability.lower() == KVStoreBase.OPTIMIZER:
            return False
        raise ValueError('Unknown capability: {}'.format(capability))

    @property
    def type(self):
        return 'teststore'

    @property
    def rank(self):
        return 0

    @property
    def num_workers(self):
        return 1

    def set_optimizer(self, optimizer):
        raise NotImplementedError('TestStore does not support optimizer on the store')

    def save_optimizer_states(self, fname, dump_optimizer=False):
        raise NotImplementedError()

    def load_optimizer_states(self, fname):
        raise NotImplementedError()


def create(name='local'):
    """Create a store: 'local' | 'device' | 'nccl' | 'dist_sync' | 'dist_async' | 'dist_device_sync' |
    'dist_sync_device' | 'horovod' | 'byteps' | any registered plug-in class name."""
    if not isinstance(name, str):
        raise TypeError('name must be a string')
    name = name.lower()
    if name in KVStoreBase.kv_registry:
        return KVStoreBase.kv_registry[name]()
    from .kvstore import KVStore
    return KVStore(name)

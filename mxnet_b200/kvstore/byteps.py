"""BytePS adapter (``python/mxnet/kvstore/byteps.py:45-163``): push_pull of declared tensors.  Runs
over ``torch.distributed`` when the byteps package is absent."""
from .base import KVStoreBase
from .horovod import Horovod

__all__ = ['BytePS']


@KVStoreBase.register
class BytePS(Horovod):
    def __init__(self):
        super().__init__()
        self._declared = set()

    @property
    def type(self):
        return 'byteps'

    def broadcast(self, key, value, out, priority=0):
        self._declared.add(str(key))
        super().broadcast(key, value, out, priority)

    def pushpull(self, key, value, out=None, priority=0):
        self._declared.add(str(key))
        super().pushpull(key, value, out, priority)

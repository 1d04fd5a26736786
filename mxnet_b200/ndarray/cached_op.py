"""``mx.nd.CachedOp(sym, flags)``: the low-level callable over a symbolic graph (reference:
``python/mxnet/_ctypes/cached_op.py`` ``CachedOp.__call__`` over ``src/imperative/cached_op.cc``).  Arrays are given in the order of
``sym.list_inputs()``; the result is one array or a list.  Under ``autograd.record`` the call is differentiable.  Blocks use the
richer :class:`mxnet_b200.gluon.cached_op.CachedOp` (CUDA-graph capture, static allocation); this class is the plain form that
user code and exported graphs reach through ``mx.nd``."""
import torch

from .. import _state
from ..base import MXNetError
from ..device import current_device

__all__ = ['CachedOp']


class CachedOp(object):
    def __init__(self, sym, flags=(), thread_safe=False):
        self._sym = sym
        self.flags = dict(flags)
        self.is_np_sym = False
        self._names = sym.list_inputs()

    def __call__(self, *args, **kwargs):
        from .ndarray import NDArray
        out = kwargs.pop('out', None)
        ctx = kwargs.pop('default_device', None) or kwargs.pop('default_ctx', None)
        if kwargs:
            raise TypeError('CachedOp.__call__ got unexpected keyword argument(s): %s' % ', '.join(kwargs))
        arrays = [a for a in args if a is not None]
        if len(arrays) != len(self._names):
            raise MXNetError('CachedOp takes %d inputs (%s), got %d' % (len(self._names), ', '.join(self._names), len(arrays)))
        if arrays:
            ctx = arrays[0].context
        elif ctx is None:
            ctx = current_device()
        feed = {n: a._data for n, a in zip(self._names, arrays)}
        with ctx:
            if _state.state.recording:
                with torch.enable_grad():
                    outs = self._sym._run(feed)
            else:
                with torch.no_grad():
                    outs = self._sym._run(feed)
        cls = type(arrays[0]) if arrays else NDArray
        if not arrays and _state.state.np_array:
            from ..numpy import ndarray as cls           # noqa: F811
        res = [cls._from_tensor(o, ctx) for o in outs]
        if out is not None:
            dst = out if isinstance(out, (list, tuple)) else [out]
            for d, r in zip(dst, res):
                d._data.copy_(r._data)
            return out
        return res[0] if len(res) == 1 else res

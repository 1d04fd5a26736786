"""``mx.npx.random`` (bernoulli, *_n batch-shape samplers)."""
from ..numpy.random import bernoulli, seed   # noqa: F401
from ..numpy import random as _r


def uniform_n(low=0.0, high=1.0, batch_shape=None, dtype=None, ctx=None, device=None):
    import torch
    from ..ndarray.ndarray import NDArray
    shp = tuple(batch_shape or ()) if not isinstance(batch_shape, int) else (batch_shape,)
    base = [x.shape for x in (low, high) if isinstance(x, NDArray)]
    full = shp + tuple(torch.broadcast_shapes(*base)) if base else shp
    return _r.uniform(low, high, size=full or None, dtype=dtype, ctx=ctx, device=device)


def normal_n(loc=0.0, scale=1.0, batch_shape=None, dtype=None, ctx=None, device=None):
    import torch
    from ..ndarray.ndarray import NDArray
    shp = tuple(batch_shape or ()) if not isinstance(batch_shape, int) else (batch_shape,)
    base = [x.shape for x in (loc, scale) if isinstance(x, NDArray)]
    full = shp + tuple(torch.broadcast_shapes(*base)) if base else shp
    return _r.normal(loc, scale, size=full or None, dtype=dtype, ctx=ctx, device=device)

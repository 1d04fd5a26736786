"""``mx.nd``: legacy imperative namespace.  Operator functions are generated from the registry at
import time, like ``_init_op_module`` does in the reference (``python/mxnet/base.py:633``,
``python/mxnet/ndarray/register.py:116-270``)."""
import sys as _sys
import types as _types

from .. import ops as _ops
from ..ops import registry as _reg
from .ndarray import *        # noqa: F401,F403
from .ndarray import NDArray, _to_tensor
from . import sparse
from .sparse import CSRNDArray, RowSparseNDArray, BaseSparseNDArray, csr_matrix, row_sparse_array
from .utils import save, load, load_frombuffer, zeros_like_shape  # noqa: F401


def _populate():
    mod = _sys.modules[__name__]
    internal = _types.ModuleType(__name__ + '._internal')
    contrib = _types.ModuleType(__name__ + '.contrib')
    linalg = _types.ModuleType(__name__ + '.linalg')
    image = _types.ModuleType(__name__ + '.image')
    op = _types.ModuleType(__name__ + '.op')
    for name in _reg.list_ops():
        if name.startswith('_npi_') or name.startswith('_npx_') or name.startswith('_np_'):
            continue
        fn = _reg.make_frontend(_reg.get(name), 'nd')
        setattr(op, name, fn)
        if name.startswith('_contrib_'):
            setattr(contrib, name[len('_contrib_'):], fn)
            setattr(internal, name, fn)
        elif name.startswith('_linalg_'):
            setattr(linalg, name[len('_linalg_'):], fn)
            setattr(internal, name, fn)
        elif name.startswith('_image_'):
            setattr(image, name[len('_image_'):], fn)
            setattr(internal, name, fn)
        elif name.startswith('_'):
            setattr(internal, name, fn)
        else:
            if not hasattr(mod, name):
                setattr(mod, name, fn)
    for m in (internal, contrib, linalg, image, op):
        _sys.modules[m.__name__] = m
    mod._internal, mod.contrib, mod.linalg, mod.image, mod.op = internal, contrib, linalg, image, op


_populate()
from . import random      # noqa: E402
from .cached_op import CachedOp   # noqa: E402,F401
from . import contrib_ext as _contrib_ext  # noqa: E402,F401  (foreach/while_loop/cond on nd.contrib)


def add(lhs, rhs): return lhs + rhs
def subtract(lhs, rhs): return lhs - rhs
def multiply(lhs, rhs): return lhs * rhs
def divide(lhs, rhs): return lhs / rhs
def modulo(lhs, rhs): return lhs % rhs
def power(base, exp): return base ** exp if isinstance(base, NDArray) else exp.__rpow__(base)
def maximum(lhs, rhs): return _cmp2('maximum', lhs, rhs)
def minimum(lhs, rhs): return _cmp2('minimum', lhs, rhs)
def equal(lhs, rhs): return lhs == rhs
def not_equal(lhs, rhs): return lhs != rhs
def greater(lhs, rhs): return lhs > rhs
def greater_equal(lhs, rhs): return lhs >= rhs
def lesser(lhs, rhs): return lhs < rhs
def lesser_equal(lhs, rhs): return lhs <= rhs
def logical_and(lhs, rhs): return _cmp2('logical_and', lhs, rhs)
def logical_or(lhs, rhs): return _cmp2('logical_or', lhs, rhs)
def logical_xor(lhs, rhs): return _cmp2('logical_xor', lhs, rhs)
true_divide = divide


def _cmp2(name, lhs, rhs):
    if isinstance(lhs, NDArray):
        return lhs._binary(rhs, name)
    if isinstance(rhs, NDArray):
        return rhs._binary(lhs, name, True)
    import builtins
    return {'maximum': builtins.max, 'minimum': builtins.min}[name](lhs, rhs)


def eye(N, M=0, k=0, ctx=None, dtype=None, **kwargs):
    return _reg.invoke('_eye', [], {'N': N, 'M': M, 'k': k, 'ctx': ctx, 'dtype': dtype or 'float32'}, kind='nd')


def linspace(start, stop, num, endpoint=True, ctx=None, dtype=None):
    return _reg.invoke('_linspace', [], {'start': start, 'stop': stop, 'num': num, 'endpoint': endpoint, 'ctx': ctx,
                                         'dtype': dtype or 'float32'}, kind='nd')


def split_v2(ary, indices_or_sections, axis=0, squeeze_axis=False):
    """Split along ``axis`` into equal sections (an int) or at the given indices (``python/mxnet/ndarray/ndarray.py:split_v2``)."""
    from ..ops import registry as _r
    ios = indices_or_sections if isinstance(indices_or_sections, int) else tuple(indices_or_sections)
    return _r.invoke('_split_v2', [ary], {'indices_or_sections': ios, 'axis': axis, 'squeeze_axis': squeeze_axis})


def dtype_np_to_mx(dtype):
    """Type flag of a NumPy dtype (``include/mxnet/base.h`` type codes)."""
    from ..base import dtype_flag
    return dtype_flag(dtype)


def dtype_mx_to_np(flag):
    """NumPy type of a type flag."""
    from ..base import flag_to_torch, to_numpy_dtype
    d = to_numpy_dtype(flag_to_torch(int(flag)))
    return getattr(d, 'type', d)


def is_mx_dtype(dtype):
    """Whether arrays of this dtype can be created."""
    try:
        dtype_np_to_mx(dtype)
        return True
    except Exception:   # pylint: disable=broad-except
        return False


def get_dtype_name(dtype):
    import numpy as _np
    return _np.dtype(dtype).name if str(dtype) != 'bfloat16' else 'bfloat16'


def get_dtype_type(dtype):
    import numpy as _np
    return _np.dtype(dtype).type

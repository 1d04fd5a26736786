"""``mx.sym``: symbolic namespace; operator composition functions are generated from the registry
(``python/mxnet/symbol/register.py``)."""
import sys as _sys
import types as _types

from ..ops import registry as _reg
from .symbol import *      # noqa: F401,F403
from .symbol import Symbol, var, Variable, Group, load, load_json, fromjson, _op_frontend
from . import passes, _trace   # noqa: F401


def _populate():
    mod = _sys.modules[__name__]
    internal = _types.ModuleType(__name__ + '._internal')
    contrib = _types.ModuleType(__name__ + '.contrib')
    linalg = _types.ModuleType(__name__ + '.linalg')
    image = _types.ModuleType(__name__ + '.image')
    random = _types.ModuleType(__name__ + '.random')
    op = _types.ModuleType(__name__ + '.op')
    for name in _reg.list_ops():
        fn = _op_frontend(_reg.get(name))
        setattr(op, name, fn)
        if name.startswith('_contrib_'):
            setattr(contrib, name[len('_contrib_'):], fn)
        elif name.startswith('_linalg_'):
            setattr(linalg, name[len('_linalg_'):], fn)
        elif name.startswith('_image_'):
            setattr(image, name[len('_image_'):], fn)
        elif name.startswith('_random_') or name.startswith('_sample_'):
            setattr(random, name.split('_', 2)[2], fn)
        if name.startswith('_'):
            setattr(internal, name, fn)
        elif not hasattr(mod, name):
            setattr(mod, name, fn)
    for m in (internal, contrib, linalg, image, random, op):
        _sys.modules[m.__name__] = m
    mod._internal, mod.contrib, mod.linalg, mod.image, mod.random, mod.op = internal, contrib, linalg, image, random, op


_populate()

from . import control_flow, fusion   # noqa: E402,F401  (fusion registers _FusedOp)
for _n in control_flow.__all__:
    setattr(contrib, _n, getattr(control_flow, _n))   # noqa: F821  (contrib is set by _populate)
from . import numpy as np          # noqa: E402,F401
from . import numpy_extension as npx   # noqa: E402,F401


def _random_extras():
    from .symbol import _make_op_symbol

    def randn(*shape, loc=0.0, scale=1.0, dtype=None, name=None, **kwargs):
        """Normal samples of the given shape (positional extents), mean ``loc``, standard deviation ``scale``."""
        return _make_op_symbol(_reg.get('_random_normal'), [], {'loc': loc, 'scale': scale, 'shape': tuple(shape),
                                                                 'dtype': dtype or 'float32'}, name)

    def categorical(data, shape=(), get_prob=False, dtype='int32', name=None, **kwargs):
        """Draws from the categorical distributions in the last axis of ``data`` (alias of ``multinomial``)."""
        return _make_op_symbol(_reg.get('_sample_multinomial'), [data], {'shape': shape, 'get_prob': get_prob, 'dtype': dtype}, name)

    def shuffle(data, name=None, **kwargs):
        """Random permutation along the first axis."""
        return _make_op_symbol(_reg.get('_shuffle'), [data], {}, name)
    random.randn, random.categorical, random.shuffle = randn, categorical, shuffle   # noqa: F821


_random_extras()


def _legacy_helpers():
    """``eye``, ``linspace``, ``maximum``, ``minimum``, ``power`` / ``pow``, ``hypot``, ``split_v2`` and the ``sparse``
    namespace of ``python/mxnet/symbol/symbol.py``: the binary helpers accept symbols or scalars on either side."""
    from .symbol import _make_op_symbol

    def eye(N, M=0, k=0, dtype=None, **kwargs):
        return _make_op_symbol(_reg.get('_eye'), [], {'N': N, 'M': M, 'k': k, 'dtype': dtype or 'float32'}, kwargs.get('name'))

    def linspace(start, stop, num, endpoint=True, name=None, dtype=None):
        return _make_op_symbol(_reg.get('_linspace'), [], {'start': start, 'stop': stop, 'num': num, 'endpoint': endpoint,
                                                           'dtype': dtype or 'float32'}, name)

    def _binary(sym_op, scalar_op, rscalar_op, pyfn):
        def fn(left, right):
            ls, rs = isinstance(left, Symbol), isinstance(right, Symbol)
            if ls and rs:
                return _make_op_symbol(_reg.get(sym_op), [left, right], {}, None)
            if ls:
                return _make_op_symbol(_reg.get(scalar_op), [left], {'scalar': right}, None)
            if rs:
                return _make_op_symbol(_reg.get(rscalar_op), [right], {'scalar': left}, None)
            return pyfn(left, right)
        return fn
    import builtins
    import math
    maximum = _binary('broadcast_maximum', '_maximum_scalar', '_maximum_scalar', builtins.max)
    minimum = _binary('broadcast_minimum', '_minimum_scalar', '_minimum_scalar', builtins.min)
    power = _binary('broadcast_power', '_power_scalar', '_rpower_scalar', lambda a, b: a ** b)
    hypot = _binary('broadcast_hypot', '_hypot_scalar', '_hypot_scalar', math.hypot)

    def split_v2(ary, indices_or_sections, axis=0, squeeze_axis=False):
        """Split along ``axis`` into equal sections (an int) or at the given indices (a tuple), as ``mx.nd.split_v2``."""
        ios = indices_or_sections if isinstance(indices_or_sections, int) else tuple(indices_or_sections)
        return _make_op_symbol(_reg.get('_split_v2'), [ary], {'indices_or_sections': ios, 'axis': axis,
                                                              'squeeze_axis': squeeze_axis}, None)
    mod = _sys.modules[__name__]
    for name, fn in (('eye', eye), ('linspace', linspace), ('maximum', maximum), ('minimum', minimum), ('power', power),
                     ('pow', power), ('hypot', hypot), ('split_v2', split_v2)):
        setattr(mod, name, fn)
    sparse = _types.ModuleType(__name__ + '.sparse')
    sparse.__doc__ = 'Sparse operators on symbols (``python/mxnet/symbol/sparse.py``): the same operators; storage types are ' \
                     'decided when the graph runs.'
    for name in ('dot', 'cast_storage', 'add_n', 'elemwise_add', 'elemwise_sub', 'elemwise_mul', 'elemwise_div', 'zeros_like',
                 'retain', 'sum', 'mean', 'square_sum', 'where', 'slice', 'clip', 'abs', 'sign', 'sqrt', 'square', 'negative',
                 'relu', 'sigmoid', 'tanh', 'Embedding', 'sgd_update', 'sgd_mom_update', 'adam_update', 'ftrl_update',
                 'broadcast_add', 'broadcast_sub', 'broadcast_mul', 'broadcast_div', 'concat', 'stop_gradient', 'make_loss'):
        fn = getattr(mod, name, None) or getattr(mod._internal, '_sparse_' + name, None)
        if fn is not None:
            setattr(sparse, name, fn)
    _sys.modules[sparse.__name__] = sparse
    mod.sparse = sparse


_legacy_helpers()

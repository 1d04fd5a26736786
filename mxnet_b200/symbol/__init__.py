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

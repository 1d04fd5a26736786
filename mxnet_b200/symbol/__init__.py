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

    # Distribution samplers (``python/mxnet/symbol/random.py:_random_helper``): scalar parameters become attributes of the
    # ``_random_*`` operator, Symbol parameters become inputs of the ``_sample_*`` operator (one distribution per element).
    def sampler(pub, random_op, sample_op, params, defaults):
        def fn(*args, shape=None, dtype=None, name=None, **kwargs):
            values = dict(zip(params, defaults))
            values.update(dict(zip(params, args)))
            values.update({k: kwargs.pop(k) for k in list(kwargs) if k in params})
            given = [values[p] for p in params]
            if pub == 'exponential':                       # the operator is parametrised by the rate
                given = [1.0 / given[0]]
                values = {'lam': given[0]}
            if any(isinstance(v, Symbol) for v in given):
                if not all(isinstance(v, Symbol) for v in given):
                    raise ValueError('Distribution parameters must all have the same type, but got both Symbol and scalars')
                return _make_op_symbol(_reg.get(sample_op), given, {'shape': tuple(shape) if shape else (), 'dtype': dtype}, name)
            attrs = dict(values, shape=tuple(shape) if shape is not None and not isinstance(shape, int) else
                         ((shape,) if isinstance(shape, int) else (1,)), dtype=dtype or 'float32')
            return _make_op_symbol(_reg.get(random_op), [], attrs, name)
        fn.__name__ = pub
        return fn
    for pub, params, defaults in (('uniform', ('low', 'high'), (0.0, 1.0)), ('normal', ('loc', 'scale'), (0.0, 1.0)),
                                  ('poisson', ('lam',), (1.0,)), ('exponential', ('scale',), (1.0,)),
                                  ('gamma', ('alpha', 'beta'), (1.0, 1.0)), ('negative_binomial', ('k', 'p'), (1, 1.0)),
                                  ('generalized_negative_binomial', ('mu', 'alpha'), (1.0, 1.0)), ('binomial', ('n', 'p'), (1, 0.5))):
        if _reg.has('_random_' + pub) and _reg.has('_sample_' + pub):
            setattr(random, pub, sampler(pub, '_random_' + pub, '_sample_' + pub, params, defaults))   # noqa: F821


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


def _contrib_rand_zipfian():
    import math

    def rand_zipfian(true_classes, num_sampled, range_max):
        """Symbolic form of ``mx.nd.contrib.rand_zipfian`` (``python/mxnet/symbol/contrib.py``): (samples, expected count of the
        true classes, expected count of the samples) under P(class) = log((class + 2) / (class + 1)) / log(range_max + 1)."""
        mod = _sys.modules[__name__]
        log_range = math.log(range_max + 1)
        rand = mod.random.uniform(0, log_range, shape=(num_sampled,), dtype='float64')
        sampled = mod.cast(mod.exp(rand) - 1, dtype='int64') % range_max
        true_cls = mod.cast(true_classes, dtype='float64')
        expected_true = mod.log((true_cls + 2.0) / (true_cls + 1.0)) / log_range * num_sampled
        sampled64 = mod.cast(sampled, dtype='float64')
        expected_sampled = mod.log((sampled64 + 2.0) / (sampled64 + 1.0)) / log_range * num_sampled
        return sampled, expected_true, expected_sampled
    contrib.rand_zipfian = rand_zipfian   # noqa: F821  (contrib is set by _populate)


_contrib_rand_zipfian()

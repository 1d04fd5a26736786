"""Graph passes on Symbols: AMP cast removal, common-subexpression elimination, backend partitioning,
low-precision conversion (``src/nnvm/low_precision_pass.cc``, ``src/imperative/eliminate_common_expr_pass.cc``,
``src/operator/subgraph/build_subgraph.cc``)."""
from ..base import MXNetError
from ..ops import registry as _reg
from .symbol import Symbol, _Node, _topo, _fmt_attr

_BACKENDS = {}


def register_backend(name, fn):
    """Register a partitioning backend: ``fn(symbol, args, aux, **options) -> symbol``."""
    _BACKENDS[name] = fn


def optimize_for(sym, backend, args=None, aux=None, **kwargs):
    if backend in (None, '', 'default'):
        return sym
    if backend == 'pointwise_fusion':
        from .fusion import fuse_pointwise
        return fuse_pointwise(sym)
    if backend == 'optimize_layout':
        from .layout import optimize_layout
        return optimize_layout(sym)
    if backend not in _BACKENDS:
        raise MXNetError('subgraph backend %s is not registered (available: %s)' % (backend, sorted(_BACKENDS)))
    return _BACKENDS[backend](sym, args, aux, **kwargs)


def _rebuild(sym, transform):
    """Copy a graph, letting ``transform(node, new_inputs)`` return a replacement entry list or None."""
    mapping = {}
    for n in _topo(sym._outputs):
        new_inputs = [(mapping[id(i)][k]) for i, k in n.inputs]
        rep = transform(n, new_inputs)
        if rep is not None:
            mapping[id(n)] = rep
            continue
        if n.op is None:
            mapping[id(n)] = [(n, 0)]
            continue
        nn = _Node(n.op, n.name, dict(n.attrs), new_inputs, n.nout, dict(n.user_attrs))
        mapping[id(n)] = [(nn, i) for i in range(n.nout)]
    return Symbol([mapping[id(n)][k] for n, k in sym._outputs])


def remove_amp_cast(sym):
    def tf(n, ins):
        if n.op is not None and n.op.name in ('Cast',) and n.name.startswith('amp_cast'):
            return [ins[0]]
        if n.op is not None and n.op.name == 'amp_cast':
            return [ins[0]]
        if n.op is not None and n.op.name == 'amp_multicast':
            return list(ins)
        return None
    return _rebuild(sym, tf)


def eliminate_common_expr(sym):
    """Merge nodes with identical operator, attributes and inputs (random ops are left alone)."""
    seen = {}

    def tf(n, ins):
        if n.op is None or 'random' in n.op.name or 'sample' in n.op.name or n.op.name == 'Dropout':
            return None
        key = (n.op.name, tuple(sorted((k, _fmt_attr(v)) for k, v in n.attrs.items())), tuple((id(i), k) for i, k in ins))
        if key in seen:
            return seen[key]
        nn = _Node(n.op, n.name, dict(n.attrs), ins, n.nout, dict(n.user_attrs))
        seen[key] = [(nn, i) for i in range(n.nout)]
        return seen[key]
    return _rebuild(sym, tf)


def convert_precision(sym, target_dtype, fp16_ops, fp32_ops, widest_ops, cast_optional_params=False,
                      excluded_names=()):
    """``ReducePrecision`` pass: insert ``amp_cast`` before operators according to the lists."""
    cast = _reg.get('amp_cast')
    multicast = _reg.get('amp_multicast')
    counter = [0]

    def casted(entry, dtype):
        counter[0] += 1
        node = _Node(cast, 'amp_cast_%d' % counter[0], {'dtype': dtype}, [entry], 1)
        return (node, 0)

    def tf(n, ins):
        if n.op is None or n.name in excluded_names:
            return None
        name = n.op.name
        names = [name] + list(n.op.aliases)
        if any(x in fp16_ops for x in names):
            new_ins = [casted(e, target_dtype) if (e[0].op is not None or cast_optional_params or j == 0 or True) else e
                       for j, e in enumerate(ins)]
        elif any(x in fp32_ops for x in names):
            new_ins = [casted(e, 'float32') for e in ins]
        elif any(x in widest_ops for x in names) and len(ins) > 1:
            counter[0] += 1
            mc = _Node(multicast, 'amp_multicast_%d' % counter[0], {'num_outputs': len(ins)}, list(ins), len(ins))
            new_ins = [(mc, i) for i in range(len(ins))]
        else:
            return None
        nn = _Node(n.op, n.name, dict(n.attrs), new_ins, n.nout, dict(n.user_attrs))
        return [(nn, i) for i in range(n.nout)]
    return _rebuild(sym, tf)

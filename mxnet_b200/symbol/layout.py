"""Automatic layout management: run the convolutional part of an NCHW graph in NHWC.

Reference: ``src/common/alm.{h,cc}`` (``OptimizeLayout``, run on the forward graph of a CachedOp when
``MXSetOptimizeLayout`` is on, which ``amp.init(layout_optimization=True)`` does, ``python/mxnet/amp/amp.py:339``).  There
the target is the tensor-core friendly layout of cuDNN; here it is the layout of the tcgen05 convolution, normalisation and
pooling kernels, which take channel-last tensors only.

The pass walks the graph once.  A 2-D ``Convolution`` in NCHW becomes the same operator in NHWC: its data input is brought
to NHWC (one copying transpose where the producer is not already NHWC), its weight gets a (0, 2, 3, 1) transpose, and its
output is marked *pending*: the value now flowing through the graph is the NHWC permutation of what the original graph
held.  Operators that do not care about the position of the channel axis (activations, scalar arithmetic, casts,
elementwise binary operators whose operands are all pending) pass the mark on; ``BatchNorm`` (axis 1 -> 3), ``Pooling``
(layout) and ``Concat`` (dim 1 -> 3) are rewritten for the new position; every other consumer, and the graph outputs, get
the value back in NCHW through one transpose per pending value.  Transposes therefore appear only at the borders of the
convolutional trunk.
"""
from ..ops import registry as _reg
from .symbol import Symbol, _Node, _topo

__all__ = ['optimize_layout', 'set_optimize_layout', 'get_optimize_layout']

_TO_NHWC = (0, 2, 3, 1)
_TO_NCHW = (0, 3, 1, 2)
_enabled = [False]


def set_optimize_layout(flag):
    """Process-wide switch (``MXSetOptimizeLayout``): hybridized blocks run their traced graph through
    :func:`optimize_layout`."""
    _enabled[0] = bool(flag)


def get_optimize_layout():
    return _enabled[0]


def _canon(names):
    out = set()
    for n in names:
        if _reg.has(n):
            out.add(_reg.get(n).name)
    return out


_UNARY = None
_BINARY = None


def _tables():
    global _UNARY, _BINARY
    if _UNARY is None:
        _UNARY = _canon(['Activation', 'relu', 'sigmoid', 'tanh', 'softsign', 'mish', 'log_sigmoid', 'abs', 'sign', 'square', 'sqrt',
                         'rsqrt', 'cbrt', 'exp', 'expm1', 'log', 'log1p', 'negative', 'reciprocal', 'erf', 'clip', 'identity',
                         'stop_gradient', 'make_loss', '_copy', 'Cast', 'amp_cast', 'floor', 'ceil', 'round', 'rint', 'trunc',
                         '_add_scalar', '_sub_scalar', '_rsub_scalar', '_mul_scalar', '_div_scalar', '_rdiv_scalar',
                         '_power_scalar', '_rpower_scalar', '_maximum_scalar', '_minimum_scalar', '_npi_add_scalar',
                         '_npi_subtract_scalar', '_npi_rsubtract_scalar', '_npi_multiply_scalar', '_npi_true_divide_scalar',
                         '_npi_rtrue_divide_scalar', '_npi_power_scalar', '_npi_maximum_scalar', '_npi_minimum_scalar',
                         '_contrib_gelu', 'zeros_like', 'ones_like'])
        _BINARY = _canon(['broadcast_add', 'broadcast_sub', 'broadcast_mul', 'broadcast_div', 'broadcast_maximum',
                          'broadcast_minimum', 'broadcast_power', '_npi_add', '_npi_subtract', '_npi_multiply',
                          '_npi_true_divide', '_npi_maximum', '_npi_minimum', 'add_n'])
    return _UNARY, _BINARY


def _is_2d_nchw(node):
    lay = node.attrs.get('layout')
    if lay not in (None, 'NCHW', ''):
        return False
    kernel = node.attrs.get('kernel') or ()
    if isinstance(kernel, int):
        return False
    return len(tuple(kernel)) == 2


def optimize_layout(sym):
    """Return a graph that computes the same outputs with its 2-D convolutions, and what sits between them, in NHWC."""
    unary, binary = _tables()
    transpose = _reg.get('_layout_transpose')
    new_of = {}              # (id(old node), k) -> entry (new node, k) holding the value AS THE OLD GRAPH DEFINES IT, or None
    pending = {}             # (id(old node), k) -> entry holding the NHWC permutation of that value
    counter = [0]

    def make_transpose(entry, axes, tag):
        counter[0] += 1
        return (_Node(transpose, '%s_%s%d' % (entry[0].name, tag, counter[0]), {'axes': axes}, [entry], 1), 0)

    def plain(key):
        """The value in the original layout (a transpose back is made once per pending value)."""
        e = new_of.get(key)
        if e is None:
            e = new_of[key] = make_transpose(pending[key], _TO_NCHW, 'nchw')
        return e

    def nhwc(key):
        e = pending.get(key)
        if e is None:
            e = pending[key] = make_transpose(new_of[key], _TO_NHWC, 'nhwc')
        return e

    def is_pending(key):
        return key in pending and new_of.get(key) is None

    converted = 0
    for n in _topo(sym._outputs):
        if n.op is None:
            new_of[(id(n), 0)] = (n, 0)
            continue
        keys = [(id(i), k) for i, k in n.inputs]
        name = n.op.name
        attrs = dict(n.attrs)
        out_pending = False
        if name == 'Convolution' and _is_2d_nchw(n) and len(keys) >= 2:
            ins = [nhwc(keys[0]), make_transpose(plain(keys[1]), _TO_NHWC, 'ohwi')] + [plain(k) for k in keys[2:]]
            attrs['layout'] = 'NHWC'
            out_pending = True
            converted += 1
        elif name == 'BatchNorm' and attrs.get('axis', 1) == 1 and is_pending(keys[0]) and not attrs.get('output_mean_var', False):
            ins = [pending[keys[0]]] + [plain(k) for k in keys[1:5]] + [nhwc(k) for k in keys[5:]]      # residual input follows
            attrs['axis'] = 3
            out_pending = True
        elif name == 'Pooling' and is_pending(keys[0]) and (_is_2d_nchw(n) or (attrs.get('global_pool') and
                                                                               attrs.get('layout') in (None, 'NCHW', ''))):
            ins = [pending[keys[0]]]
            attrs['layout'] = 'NHWC'
            out_pending = True
        elif name == 'Concat' and attrs.get('dim', 1) == 1 and attrs.get('axis') is None and keys and \
                all(is_pending(k) for k in keys):
            ins = [pending[k] for k in keys]
            attrs['dim'] = 3
            out_pending = True
        elif name in unary and len(keys) == 1 and is_pending(keys[0]) and n.nout == 1 and \
                not (name == 'Activation' and attrs.get('act_type') == 'prelu'):
            ins = [pending[keys[0]]]
            out_pending = True
        elif name in binary and keys and all(is_pending(k) for k in keys) and n.nout == 1:
            ins = [pending[k] for k in keys]
            out_pending = True
        else:
            ins = [plain(k) for k in keys]
        nn = _Node(n.op, n.name, attrs, ins, n.nout, dict(n.user_attrs))
        if out_pending:
            pending[(id(n), 0)] = (nn, 0)
            new_of[(id(n), 0)] = None
            for k in range(1, n.nout):
                new_of[(id(n), k)] = (nn, k)
        else:
            for k in range(n.nout):
                new_of[(id(n), k)] = (nn, k)
    if not converted:
        return sym
    return Symbol([plain((id(n), k)) for n, k in sym._outputs])

"""Symbol + parameters -> ONNX model (``python/mxnet/onnx/mx2onnx``: ``export_model``, ``get_operator_support``).

The model file is written by the in-tree protobuf writer (``_proto.py``), so no ``onnx`` package is needed.  Every
operator converter receives the node (name, parsed attributes, number of outputs), the ONNX names of its inputs and an
:class:`Exporter` to emit nodes and constants; shapes inferred from ``in_shapes`` are available to converters that need
them (``Reshape`` special codes, ``FullyConnected`` without flattening).  Default opset: 13."""
import json

import numpy as np

from ..base import MXNetError
from . import _proto as P

_CONVERTERS = {}


def register(*op_names):
    def deco(fn):
        for n in op_names:
            _CONVERTERS[n] = fn
        return fn
    return deco


def get_operator_support(opset_version=None):
    """Names of the operators that can be exported."""
    return sorted(_CONVERTERS)


class Exporter(object):
    def __init__(self, opset, shapes, dtypes):
        self.opset = opset
        self.nodes, self.initializers = [], []
        self.shapes, self.dtypes = shapes, dtypes          # ONNX value name -> shape tuple / numpy dtype (when inferred)
        self._uid = 0

    def fresh(self, hint):
        self._uid += 1
        return '%s_%d' % (hint, self._uid)

    def node(self, op_type, inputs, outputs=None, name=None, **attrs):
        """Emit one node; returns its first output name (or the list when several were asked for)."""
        if outputs is None:
            outputs = [self.fresh(op_type.lower())]
        elif isinstance(outputs, str):
            outputs = [outputs]
        self.nodes.append(P.make_node(op_type, inputs, outputs, name or outputs[0], **attrs))
        return outputs[0] if len(outputs) == 1 else list(outputs)

    def const(self, value, hint='const', dtype=None):
        arr = np.asarray(value, dtype=dtype)
        name = self.fresh(hint)
        self.initializers.append(P.make_tensor(name, arr))
        self.shapes[name], self.dtypes[name] = tuple(arr.shape), arr.dtype
        return name

    def scalar_like(self, value, ref):
        """A scalar constant in the element type of the value `ref` (float32 when unknown)."""
        return self.const(value, 'scalar', self.dtypes.get(ref) or np.float32)

    def shape(self, name):
        return self.shapes.get(name)


def _t(v, n=None, default=None):
    """Attribute value -> tuple of ints (scalars are repeated n times)."""
    if v is None or v == ():
        return default
    if isinstance(v, (int, np.integer)):
        return (int(v),) * (n or 1)
    return tuple(int(x) for x in v)


# ---------------------------------------------------------------------------------------- layers
def _nhwc(layout):
    return layout is not None and str(layout).upper() in ('NHWC', 'NWC', 'NDHWC')


def _to_channels_first(ex, x, nd):
    return ex.node('Transpose', [x], perm=[0, nd + 1] + list(range(1, nd + 1)))


def _to_channels_last(ex, x, nd, out=None):
    return ex.node('Transpose', [x], out, perm=[0] + list(range(2, nd + 2)) + [1])


@register('Convolution', 'Deconvolution')
def _conv(node, ins, ex):
    a = node['attrs']
    k = _t(a['kernel'])
    nd = len(k)
    stride, dil, pad = _t(a.get('stride'), nd, (1,) * nd), _t(a.get('dilate'), nd, (1,) * nd), _t(a.get('pad'), nd, (0,) * nd)
    x, w = ins[0], ins[1]
    last = _nhwc(a.get('layout'))
    if last:                                   # data N..C and weights O..I -> channels first
        x, w = _to_channels_first(ex, x, nd), _to_channels_first(ex, w, nd)
    inputs = [x, w] + ([ins[2]] if len(ins) > 2 and not a.get('no_bias') else [])
    kw = dict(kernel_shape=list(k), strides=list(stride), dilations=list(dil), pads=list(pad) * 2, group=int(a.get('num_group', 1)))
    if node['op'] == 'Deconvolution':
        adj = _t(a.get('adj'), nd, (0,) * nd)
        if any(adj):
            kw['output_padding'] = list(adj)
        y = ex.node('ConvTranspose', inputs, None if last else node['name'], **kw)
    else:
        y = ex.node('Conv', inputs, None if last else node['name'], **kw)
    return [_to_channels_last(ex, y, nd, node['name'])] if last else [y]


@register('FullyConnected')
def _fc(node, ins, ex):
    a = node['attrs']
    bias = ins[2] if len(ins) > 2 and not a.get('no_bias') else None
    if a.get('flatten', True):
        x = ex.node('Flatten', [ins[0]], axis=1)
        return [ex.node('Gemm', [x, ins[1]] + ([bias] if bias else []), node['name'], alpha=1.0, beta=1.0, transA=0, transB=1)]
    wt = ex.node('Transpose', [ins[1]], perm=[1, 0])
    y = ex.node('MatMul', [ins[0], wt], None if bias else node['name'])
    return [ex.node('Add', [y, bias], node['name'])] if bias else [y]


@register('BatchNorm')
def _bn(node, ins, ex):
    a = node['attrs']
    axis = int(a.get('axis', 1))
    x, gamma = ins[0], ins[1]
    if a.get('fix_gamma', True):
        shp = ex.shape(ins[1])
        if shp is None:
            raise MXNetError('BatchNorm %s with fix_gamma needs known shapes (pass in_shapes)' % node['name'])
        gamma = ex.const(np.ones(shp, dtype=ex.dtypes.get(ins[1]) or np.float32), 'gamma_one')
    rank = len(ex.shape(ins[0])) if ex.shape(ins[0]) else None
    moved = axis not in (1,) and not (rank and axis % rank == 1)
    if moved:
        if rank is None:
            raise MXNetError('BatchNorm %s over axis %d needs known shapes (pass in_shapes)' % (node['name'], axis))
        ax = axis % rank
        perm = [0, ax] + [d for d in range(1, rank) if d != ax]
        x = ex.node('Transpose', [x], perm=perm)
    y = ex.node('BatchNormalization', [x, gamma, ins[2], ins[3], ins[4]], None if moved else node['name'],
                epsilon=float(a.get('eps', 1e-3)), momentum=float(a.get('momentum', 0.9)))
    if moved:
        inv = [perm.index(d) for d in range(rank)]
        y = ex.node('Transpose', [y], node['name'], perm=inv)
    return [y]


def _gelu(ex, x, out):
    h = ex.node('Div', [x, ex.scalar_like(np.sqrt(2.0), x)])
    e = ex.node('Add', [ex.node('Erf', [h]), ex.scalar_like(1.0, x)])
    return ex.node('Mul', [ex.node('Mul', [x, e]), ex.scalar_like(0.5, x)], out)


@register('Activation')
def _act(node, ins, ex):
    kind = node['attrs'].get('act_type', 'relu')
    simple = {'relu': 'Relu', 'sigmoid': 'Sigmoid', 'tanh': 'Tanh', 'softrelu': 'Softplus', 'softsign': 'Softsign'}
    if kind in simple:
        return [ex.node(simple[kind], [ins[0]], node['name'])]
    if kind == 'log_sigmoid':
        return [ex.node('Log', [ex.node('Sigmoid', [ins[0]])], node['name'])]
    if kind == 'mish':
        return [ex.node('Mul', [ins[0], ex.node('Tanh', [ex.node('Softplus', [ins[0]])])], node['name'])]
    if kind == 'gelu':
        return [_gelu(ex, ins[0], node['name'])]
    raise MXNetError('Activation type %s cannot be exported' % kind)


@register('LeakyReLU')
def _leaky(node, ins, ex):
    a = node['attrs']
    kind = a.get('act_type', 'leaky')
    if kind == 'leaky':
        return [ex.node('LeakyRelu', [ins[0]], node['name'], alpha=float(a.get('slope', 0.25)))]
    if kind == 'elu':
        return [ex.node('Elu', [ins[0]], node['name'], alpha=float(a.get('slope', 0.25)))]
    if kind == 'selu':
        return [ex.node('Selu', [ins[0]], node['name'], alpha=1.6732632423543772, gamma=1.0507009873554805)]
    if kind == 'gelu':
        return [_gelu(ex, ins[0], node['name'])]
    if kind == 'prelu':
        rank = len(ex.shape(ins[0])) if ex.shape(ins[0]) else 4
        slope = ex.node('Reshape', [ins[1], ex.const([-1] + [1] * (rank - 2), 'shape', np.int64)]) if rank > 2 else ins[1]
        return [ex.node('PRelu', [ins[0], slope], node['name'])]
    raise MXNetError('LeakyReLU type %s cannot be exported' % kind)


@register('Pooling')
def _pool(node, ins, ex):
    a = node['attrs']
    kind = a.get('pool_type', 'max')
    x = ins[0]
    last = _nhwc(a.get('layout'))
    rank = len(ex.shape(ins[0])) if ex.shape(ins[0]) else None
    k = _t(a.get('kernel'))
    nd = len(k) if k else (rank - 2 if rank else 2)
    if last:
        x = _to_channels_first(ex, x, nd)
    out = None if last else node['name']
    if a.get('global_pool'):
        if kind not in ('max', 'avg'):
            raise MXNetError('global %s pooling cannot be exported' % kind)
        y = ex.node('GlobalMaxPool' if kind == 'max' else 'GlobalAveragePool', [x], out)
    else:
        stride, pad = _t(a.get('stride'), nd, (1,) * nd), _t(a.get('pad'), nd, (0,) * nd)
        kw = dict(kernel_shape=list(k), strides=list(stride), pads=list(pad) * 2,
                  ceil_mode=int(a.get('pooling_convention', 'valid') == 'full'))
        if kind == 'max':
            y = ex.node('MaxPool', [x], out, **kw)
        elif kind == 'avg':
            y = ex.node('AveragePool', [x], out, count_include_pad=int(bool(a.get('count_include_pad', True))), **kw)
        else:
            raise MXNetError('%s pooling cannot be exported' % kind)
    return [_to_channels_last(ex, y, nd, node['name'])] if last else [y]


@register('Flatten')
def _flatten(node, ins, ex):
    return [ex.node('Flatten', [ins[0]], node['name'], axis=1)]


@register('softmax', 'log_softmax', 'SoftmaxOutput', 'SoftmaxActivation')
def _softmax(node, ins, ex):
    a = node['attrs']
    x = ins[0]
    if node['op'] == 'SoftmaxOutput':
        axis = 1 if not a.get('preserve_shape') else -1
    elif node['op'] == 'SoftmaxActivation':
        axis = 1
    else:
        axis = int(a.get('axis', -1))
    t = a.get('temperature')
    if t not in (None, 1, 1.0):
        x = ex.node('Div', [x, ex.scalar_like(float(t), x)])
    return [ex.node('LogSoftmax' if node['op'] == 'log_softmax' else 'Softmax', [x], node['name'], axis=axis)]


@register('Concat')
def _concat(node, ins, ex):
    return [ex.node('Concat', ins, node['name'], axis=int(node['attrs'].get('dim', 1)))]


@register('Dropout', '_copy', 'identity', 'BlockGrad', 'stop_gradient', 'make_loss', 'MakeLoss')
def _identity(node, ins, ex):
    return [ex.node('Identity', [ins[0]], node['name'])]


@register('LayerNorm')
def _ln(node, ins, ex):
    a = node['attrs']
    axis = int(a.get('axis', -1))
    x = ins[0]
    mean = ex.node('ReduceMean', [x], axes=[axis], keepdims=1)
    d = ex.node('Sub', [x, mean])
    var = ex.node('ReduceMean', [ex.node('Mul', [d, d])], axes=[axis], keepdims=1)
    inv = ex.node('Reciprocal', [ex.node('Sqrt', [ex.node('Add', [var, ex.scalar_like(float(a.get('eps', 1e-5)), x)])])])
    norm = ex.node('Mul', [d, inv])
    gamma, beta = ins[1], ins[2]
    rank = len(ex.shape(x)) if ex.shape(x) else None
    if axis != -1 and not (rank and axis % rank == rank - 1):
        if rank is None:
            raise MXNetError('LayerNorm %s over axis %d needs known shapes (pass in_shapes)' % (node['name'], axis))
        shp = ex.const([-1] + [1] * (rank - 1 - axis % rank), 'shape', np.int64)
        gamma, beta = ex.node('Reshape', [gamma, shp]), ex.node('Reshape', [beta, shp])
    return [ex.node('Add', [ex.node('Mul', [norm, gamma]), beta], node['name'])]


@register('InstanceNorm')
def _in(node, ins, ex):
    return [ex.node('InstanceNormalization', ins[:3], node['name'], epsilon=float(node['attrs'].get('eps', 1e-3)))]


@register('L2Normalization')
def _l2n(node, ins, ex):
    mode = node['attrs'].get('mode', 'instance')
    if mode != 'channel':
        raise MXNetError('L2Normalization mode %s cannot be exported (channel only)' % mode)
    return [ex.node('LpNormalization', [ins[0]], node['name'], axis=1, p=2)]


@register('LRN')
def _lrn(node, ins, ex):
    a = node['attrs']
    return [ex.node('LRN', [ins[0]], node['name'], size=int(a['nsize']), alpha=float(a.get('alpha', 1e-4)), beta=float(a.get('beta', 0.75)),
                    bias=float(a.get('knorm', 2.0)))]


@register('Embedding')
def _embedding(node, ins, ex):
    idx = ex.node('Cast', [ins[0]], to=P.INT64)
    return [ex.node('Gather', [ins[1], idx], node['name'], axis=0)]


@register('UpSampling')
def _upsampling(node, ins, ex):
    a = node['attrs']
    if a.get('sample_type', 'nearest') != 'nearest':
        raise MXNetError('UpSampling with sample_type %s cannot be exported' % a.get('sample_type'))
    s = float(a['scale'])
    return [ex.node('Resize', [ins[0], '', ex.const([1.0, 1.0, s, s], 'scales', np.float32)], node['name'], mode='nearest',
                    coordinate_transformation_mode='asymmetric', nearest_mode='floor')]


@register('_contrib_BilinearResize2D')
def _bilinear(node, ins, ex):
    a = node['attrs']
    shp = ex.shape(ins[0])
    if a.get('height') and a.get('width') and shp:
        sizes = ex.const([shp[0], shp[1], int(a['height']), int(a['width'])], 'sizes', np.int64)
        return [ex.node('Resize', [ins[0], '', '', sizes], node['name'], mode='linear', coordinate_transformation_mode='align_corners')]
    scales = ex.const([1.0, 1.0, float(a.get('scale_height', 1.0)), float(a.get('scale_width', 1.0))], 'scales', np.float32)
    return [ex.node('Resize', [ins[0], '', scales], node['name'], mode='linear', coordinate_transformation_mode='align_corners')]


@register('Pad', 'pad')
def _pad(node, ins, ex):
    a = node['attrs']
    w = _t(a['pad_width'])
    nd = len(w) // 2
    pads = [w[2 * i] for i in range(nd)] + [w[2 * i + 1] for i in range(nd)]
    mode = a.get('mode', 'constant')
    inputs = [ins[0], ex.const(pads, 'pads', np.int64)]
    if mode == 'constant':
        inputs.append(ex.scalar_like(float(a.get('constant_value', 0.0)), ins[0]))
    return [ex.node('Pad', inputs, node['name'], mode=mode)]


# ---------------------------------------------------------------------------------------- shape manipulation
@register('Reshape', 'reshape', '_npx_reshape')
def _reshape(node, ins, ex):
    a = node['attrs']
    target = list(_t(a.get('shape', a.get('newshape'))) or ())
    if any(s < -1 for s in target) or a.get('reverse'):
        out_shape = ex.shape(node['name'])
        if out_shape is None:
            raise MXNetError('Reshape %s uses special codes; pass in_shapes so that the result shape is known' % node['name'])
        target = list(out_shape)
    return [ex.node('Reshape', [ins[0], ex.const(target, 'shape', np.int64)], node['name'])]


@register('transpose', '_npi_transpose')
def _transpose(node, ins, ex):
    axes = _t(node['attrs'].get('axes'))
    return [ex.node('Transpose', [ins[0]], node['name'], **({'perm': list(axes)} if axes else {}))]


@register('expand_dims')
def _expand_dims(node, ins, ex):
    return [ex.node('Unsqueeze', [ins[0], ex.const([int(node['attrs']['axis'])], 'axes', np.int64)], node['name'])]


@register('squeeze')
def _squeeze(node, ins, ex):
    axes = _t(node['attrs'].get('axis'))
    return [ex.node('Squeeze', [ins[0]] + ([ex.const(list(axes), 'axes', np.int64)] if axes else []), node['name'])]


@register('slice_axis')
def _slice_axis(node, ins, ex):
    a = node['attrs']
    end = a.get('end')
    end = np.iinfo(np.int64).max if end is None else int(end)
    return [ex.node('Slice', [ins[0], ex.const([int(a['begin'])], 'starts', np.int64), ex.const([end], 'ends', np.int64),
                              ex.const([int(a['axis'])], 'axes', np.int64)], node['name'])]


@register('slice', 'crop')
def _slice(node, ins, ex):
    a = node['attrs']
    begin, end = list(a['begin']), list(a['end'])
    step = list(a.get('step') or [None] * len(begin))
    big = np.iinfo(np.int64).max
    starts = [0 if b is None else int(b) for b in begin]
    ends = [big if e is None else int(e) for e in end]
    steps = [1 if s is None else int(s) for s in step] + [1] * (len(begin) - len(step))
    if any(s < 0 for s in steps):
        raise MXNetError('slice with negative steps cannot be exported')
    return [ex.node('Slice', [ins[0], ex.const(starts, 'starts', np.int64), ex.const(ends, 'ends', np.int64),
                              ex.const(list(range(len(starts))), 'axes', np.int64), ex.const(steps, 'steps', np.int64)], node['name'])]


@register('SliceChannel', 'split')
def _split(node, ins, ex):
    a = node['attrs']
    n, axis = int(a['num_outputs']), int(a.get('axis', 1))
    names = [node['name']] + ['%s_output%d' % (node['name'], i) for i in range(1, n)]
    if a.get('squeeze_axis'):
        parts = ex.node('Split', [ins[0]], [ex.fresh('split') for _ in range(n)], axis=axis)
        parts = [parts] if isinstance(parts, str) else parts
        ax = ex.const([axis], 'axes', np.int64)
        return [ex.node('Squeeze', [p, ax], nm) for p, nm in zip(parts, names)]
    outs = ex.node('Split', [ins[0]], names, axis=axis)
    return [outs] if isinstance(outs, str) else outs


@register('Cast', 'amp_cast')
def _cast(node, ins, ex):
    dt = np.dtype(str(node['attrs'].get('dtype', 'float32')))
    return [ex.node('Cast', [ins[0]], node['name'], to=P.NP_TO_ONNX[dt])]


@register('clip')
def _clip(node, ins, ex):
    a = node['attrs']
    lo = ex.scalar_like(float(a['a_min']), ins[0]) if a.get('a_min') is not None else ''
    hi = ex.scalar_like(float(a['a_max']), ins[0]) if a.get('a_max') is not None else ''
    return [ex.node('Clip', [ins[0], lo, hi], node['name'])]


@register('tile')
def _tile(node, ins, ex):
    reps = list(_t(node['attrs']['reps']))
    rank = len(ex.shape(ins[0])) if ex.shape(ins[0]) else len(reps)
    reps = [1] * (rank - len(reps)) + reps
    return [ex.node('Tile', [ins[0], ex.const(reps, 'repeats', np.int64)], node['name'])]


@register('broadcast_to')
def _broadcast_to(node, ins, ex):
    shape = list(_t(node['attrs']['shape']))
    src = ex.shape(ins[0])
    if src:
        shape = [s if t == 0 else t for s, t in zip(src, shape)]
    return [ex.node('Expand', [ins[0], ex.const(shape, 'shape', np.int64)], node['name'])]


@register('zeros_like', 'ones_like')
def _fill_like(node, ins, ex):
    dt = ex.dtypes.get(ins[0]) or np.dtype('float32')
    value = P.make_tensor('value', np.full((1,), 0 if node['op'] == 'zeros_like' else 1, dtype=dt))
    return [ex.node('ConstantOfShape', [ex.node('Shape', [ins[0]])], node['name'], value=value)]


@register('where')
def _where(node, ins, ex):
    return [ex.node('Where', [ex.node('Cast', [ins[0]], to=P.BOOL), ins[1], ins[2]], node['name'])]


# ---------------------------------------------------------------------------------------- arithmetic
def _binary(onnx_op):
    def conv(node, ins, ex):
        return [ex.node(onnx_op, ins[:2], node['name'])]
    return conv


for _names, _op in ((('broadcast_add', '_npi_add'), 'Add'), (('broadcast_sub', '_npi_subtract'), 'Sub'),
                    (('broadcast_mul', '_npi_multiply'), 'Mul'), (('broadcast_div', '_npi_true_divide'), 'Div'),
                    (('broadcast_power', '_npi_power'), 'Pow'), (('broadcast_maximum', '_npi_maximum'), 'Max'),
                    (('broadcast_minimum', '_npi_minimum'), 'Min')):
    register(*_names)(_binary(_op))


def _scalar(onnx_op, reverse=False):
    def conv(node, ins, ex):
        s = ex.scalar_like(float(node['attrs'].get('scalar', 0.0)), ins[0])
        return [ex.node(onnx_op, [s, ins[0]] if reverse else [ins[0], s], node['name'])]
    return conv


for _names, _op, _rev in ((('_add_scalar', '_npi_add_scalar'), 'Add', False), (('_sub_scalar', '_npi_subtract_scalar'), 'Sub', False),
                          (('_rsub_scalar', '_npi_rsubtract_scalar'), 'Sub', True), (('_mul_scalar', '_npi_multiply_scalar'), 'Mul', False),
                          (('_div_scalar', '_npi_true_divide_scalar'), 'Div', False),
                          (('_rdiv_scalar', '_npi_rtrue_divide_scalar'), 'Div', True),
                          (('_power_scalar', '_npi_power_scalar'), 'Pow', False), (('_rpower_scalar', '_npi_rpower_scalar'), 'Pow', True),
                          (('_maximum_scalar', '_npi_maximum_scalar'), 'Max', False),
                          (('_minimum_scalar', '_npi_minimum_scalar'), 'Min', False)):
    register(*_names)(_scalar(_op, _rev))


def _unary(onnx_op):
    def conv(node, ins, ex):
        return [ex.node(onnx_op, [ins[0]], node['name'])]
    return conv


for _mx, _ox in (('relu', 'Relu'), ('sigmoid', 'Sigmoid'), ('tanh', 'Tanh'), ('exp', 'Exp'), ('log', 'Log'), ('sqrt', 'Sqrt'),
                 ('abs', 'Abs'), ('negative', 'Neg'), ('reciprocal', 'Reciprocal'), ('erf', 'Erf'), ('floor', 'Floor'),
                 ('ceil', 'Ceil'), ('round', 'Round'), ('sin', 'Sin'), ('cos', 'Cos'), ('tan', 'Tan'), ('arcsin', 'Asin'),
                 ('arccos', 'Acos'), ('arctan', 'Atan'), ('sinh', 'Sinh'), ('cosh', 'Cosh'), ('arcsinh', 'Asinh'),
                 ('arccosh', 'Acosh'), ('arctanh', 'Atanh'), ('sign', 'Sign'), ('softsign', 'Softsign')):
    register(_mx)(_unary(_ox))


@register('square')
def _square(node, ins, ex):
    return [ex.node('Mul', [ins[0], ins[0]], node['name'])]


@register('rsqrt')
def _rsqrt(node, ins, ex):
    return [ex.node('Reciprocal', [ex.node('Sqrt', [ins[0]])], node['name'])]


@register('log_sigmoid')
def _log_sigmoid(node, ins, ex):
    return [ex.node('Log', [ex.node('Sigmoid', [ins[0]])], node['name'])]


@register('add_n', 'ElementWiseSum')
def _add_n(node, ins, ex):
    return [ex.node('Sum', ins, node['name'])]


# ---------------------------------------------------------------------------------------- reductions, products
def _reduce_axes(node, ex, x):
    a = node['attrs']
    axes = _t(a.get('axis'))
    if a.get('exclude') and axes is not None:
        rank = len(ex.shape(x)) if ex.shape(x) else None
        if rank is None:
            raise MXNetError('%s with exclude=True needs known shapes (pass in_shapes)' % node['name'])
        axes = tuple(d for d in range(rank) if d not in [ax % rank for ax in axes])
    return axes, int(bool(a.get('keepdims', False)))


def _reduce(onnx_op):
    def conv(node, ins, ex):
        axes, keep = _reduce_axes(node, ex, ins[0])
        if onnx_op == 'ReduceSum':                     # axes moved to an input in opset 13
            inputs = [ins[0]] + ([ex.const(list(axes), 'axes', np.int64)] if axes else [])
            return [ex.node('ReduceSum', inputs, node['name'], keepdims=keep)]
        return [ex.node(onnx_op, [ins[0]], node['name'], keepdims=keep, **({'axes': list(axes)} if axes else {}))]
    return conv


for _mx, _ox in (('sum', 'ReduceSum'), ('mean', 'ReduceMean'), ('max', 'ReduceMax'), ('min', 'ReduceMin'), ('prod', 'ReduceProd')):
    register(_mx)(_reduce(_ox))


@register('norm')
def _norm(node, ins, ex):
    if int(node['attrs'].get('ord', 2)) != 2:
        raise MXNetError('norm with ord != 2 cannot be exported')
    axes, keep = _reduce_axes(node, ex, ins[0])
    return [ex.node('ReduceL2', [ins[0]], node['name'], keepdims=keep, **({'axes': list(axes)} if axes else {}))]


@register('argmax', 'argmin')
def _argmax(node, ins, ex):
    a = node['attrs']
    idx = ex.node('ArgMax' if node['op'] == 'argmax' else 'ArgMin', [ins[0]], axis=int(a.get('axis', 0) or 0),
                  keepdims=int(bool(a.get('keepdims', False))))
    return [ex.node('Cast', [idx], node['name'], to=P.FLOAT)]          # the operator returns floating indices


@register('dot')
def _dot(node, ins, ex):
    a = node['attrs']
    x = ex.node('Transpose', [ins[0]], perm=[1, 0]) if a.get('transpose_a') else ins[0]
    y = ex.node('Transpose', [ins[1]], perm=[1, 0]) if a.get('transpose_b') else ins[1]
    return [ex.node('MatMul', [x, y], node['name'])]


@register('batch_dot')
def _batch_dot(node, ins, ex):
    a = node['attrs']

    def tr(x):
        rank = len(ex.shape(x)) if ex.shape(x) else 3
        perm = list(range(rank - 2)) + [rank - 1, rank - 2]
        return ex.node('Transpose', [x], perm=perm)
    x = tr(ins[0]) if a.get('transpose_a') else ins[0]
    y = tr(ins[1]) if a.get('transpose_b') else ins[1]
    return [ex.node('MatMul', [x, y], node['name'])]


@register('_npi_matmul')
def _matmul(node, ins, ex):
    return [ex.node('MatMul', ins[:2], node['name'])]


# ---------------------------------------------------------------------------------------- comparisons, logic, indexing
def _compare(onnx_op, negate=False):
    """Comparison operators return 0/1 in the element type of their first input (not booleans)."""
    def conv(node, ins, ex):
        y = ins[1] if len(ins) > 1 else ex.scalar_like(float(node['attrs'].get('scalar', 0.0)), ins[0])
        b = ex.node(onnx_op, [ins[0], y])
        if negate:
            b = ex.node('Not', [b])
        return [ex.node('Cast', [b], node['name'], to=P.NP_TO_ONNX[np.dtype(ex.dtypes.get(ins[0]) or np.float32)])]
    return conv


for _names, _op, _neg in ((('broadcast_equal', '_equal_scalar', '_npi_equal'), 'Equal', False),
                          (('broadcast_not_equal', '_not_equal_scalar', '_npi_not_equal'), 'Equal', True),
                          (('broadcast_greater', '_greater_scalar', '_npi_greater'), 'Greater', False),
                          (('broadcast_lesser', '_lesser_scalar', '_npi_less'), 'Less', False),
                          (('broadcast_greater_equal', '_greater_equal_scalar', '_npi_greater_equal'), 'GreaterOrEqual', False),
                          (('broadcast_lesser_equal', '_lesser_equal_scalar', '_npi_less_equal'), 'LessOrEqual', False)):
    register(*_names)(_compare(_op, _neg))


def _logical(onnx_op):
    def conv(node, ins, ex):
        dt = P.NP_TO_ONNX[np.dtype(ex.dtypes.get(ins[0]) or np.float32)]
        zero = ex.scalar_like(0.0, ins[0])
        bools = [ex.node('Not', [ex.node('Equal', [i, zero])]) for i in ins[:2]]
        return [ex.node('Cast', [ex.node(onnx_op, bools)], node['name'], to=dt)]
    return conv


for _mx, _ox in (('broadcast_logical_and', 'And'), ('broadcast_logical_or', 'Or'), ('broadcast_logical_xor', 'Xor')):
    register(_mx)(_logical(_ox))


@register('logical_not')
def _logical_not(node, ins, ex):
    dt = P.NP_TO_ONNX[np.dtype(ex.dtypes.get(ins[0]) or np.float32)]
    return [ex.node('Cast', [ex.node('Equal', [ins[0], ex.scalar_like(0.0, ins[0])])], node['name'], to=dt)]


@register('take')
def _take(node, ins, ex):
    a = node['attrs']
    idx = ex.node('Cast', [ins[1]], to=P.INT64)
    if str(a.get('mode', 'clip')) == 'clip' and ex.shape(ins[0]):
        hi = ex.shape(ins[0])[int(a.get('axis', 0) or 0)] - 1
        idx = ex.node('Clip', [idx, ex.const(0, 'lo', np.int64), ex.const(hi, 'hi', np.int64)])
    return [ex.node('Gather', [ins[0], idx], node['name'], axis=int(a.get('axis', 0) or 0))]


@register('one_hot')
def _one_hot(node, ins, ex):
    a = node['attrs']
    depth = ex.const([int(a['depth'])], 'depth', np.int64)
    values = ex.const([float(a.get('off_value', 0.0)), float(a.get('on_value', 1.0))], 'values', np.float32)
    out = ex.node('OneHot', [ex.node('Cast', [ins[0]], to=P.INT64), depth, values], axis=-1)
    return [ex.node('Cast', [out], node['name'], to=P.NP_TO_ONNX[np.dtype(str(a.get('dtype', 'float32')))])]


@register('stack')
def _stack(node, ins, ex):
    axis = int(node['attrs'].get('axis', 0) or 0)
    parts = [ex.node('Unsqueeze', [i, ex.const([axis], 'axes', np.int64)]) for i in ins]
    return [ex.node('Concat', parts, node['name'], axis=axis)]


@register('repeat')
def _repeat(node, ins, ex):
    a = node['attrs']
    shp = ex.shape(ins[0])
    if shp is None or a.get('axis') is None:
        raise AttributeError('repeat needs an explicit axis and a known input shape to be exported')
    axis, r = int(a['axis']) % len(shp), int(a['repeats'])
    x = ex.node('Unsqueeze', [ins[0], ex.const([axis + 1], 'axes', np.int64)])
    reps = [1] * (len(shp) + 1)
    reps[axis + 1] = r
    x = ex.node('Tile', [x, ex.const(reps, 'reps', np.int64)])
    new_shape = list(shp)
    new_shape[axis] *= r
    return [ex.node('Reshape', [x, ex.const(new_shape, 'shape', np.int64)], node['name'])]


@register('reverse', 'flip')
def _reverse(node, ins, ex):
    shp = ex.shape(ins[0])
    axes = node['attrs'].get('axis', 0)
    axes = [axes] if isinstance(axes, int) else list(axes)
    if shp is None:
        raise AttributeError('reverse needs a known input shape to be exported')
    n = len(axes)
    return [ex.node('Slice', [ins[0], ex.const([-1] * n, 'starts', np.int64), ex.const([-(2 ** 62)] * n, 'ends', np.int64),
                              ex.const([ax % len(shp) for ax in axes], 'axes', np.int64), ex.const([-1] * n, 'steps', np.int64)],
                    node['name'])]


@register('swapaxes', 'SwapAxis')
def _swapaxes(node, ins, ex):
    shp = ex.shape(ins[0])
    if shp is None:
        raise AttributeError('swapaxes needs a known input shape to be exported')
    a = node['attrs']
    d1, d2 = int(a.get('dim1', 0)) % len(shp), int(a.get('dim2', 0)) % len(shp)
    perm = list(range(len(shp)))
    perm[d1], perm[d2] = perm[d2], perm[d1]
    return [ex.node('Transpose', [ins[0]], node['name'], perm=perm)]


@register('depth_to_space', 'space_to_depth')
def _d2s(node, ins, ex):
    bs = int(node['attrs']['block_size'])
    if node['op'] == 'depth_to_space':
        return [ex.node('DepthToSpace', [ins[0]], node['name'], blocksize=bs, mode='DCR')]
    return [ex.node('SpaceToDepth', [ins[0]], node['name'], blocksize=bs)]


@register('shape_array')
def _shape_array(node, ins, ex):
    return [ex.node('Shape', [ins[0]], node['name'])]


@register('size_array')
def _size_array(node, ins, ex):
    return [ex.node('Reshape', [ex.node('Size', [ins[0]]), ex.const([1], 'shape', np.int64)], node['name'])]      # one element, rank 1


@register('topk')
def _topk(node, ins, ex):
    a = node['attrs']
    k = ex.const([int(a.get('k', 1))], 'k', np.int64)
    vals, idx = ex.node('TopK', [ins[0], k], [ex.fresh('topk_values'), ex.fresh('topk_indices')], axis=int(a.get('axis', -1)),
                        largest=0 if a.get('is_ascend', False) else 1, sorted=1)
    ret = str(a.get('ret_typ', 'indices'))
    idx_f = ex.node('Cast', [idx], to=P.NP_TO_ONNX[np.dtype(str(a.get('dtype', 'float32')))])
    if ret == 'value':
        return [ex.node('Identity', [vals], node['name'])]
    if ret == 'both':
        return [ex.node('Identity', [vals], node['name'] + '_values'), ex.node('Identity', [idx_f], node['name'] + '_indices')]
    return [ex.node('Identity', [idx_f], node['name'])]


@register('hard_sigmoid')
def _hard_sigmoid(node, ins, ex):
    a = node['attrs']
    return [ex.node('HardSigmoid', [ins[0]], node['name'], alpha=float(a.get('alpha', 0.2)), beta=float(a.get('beta', 0.5)))]


@register('softmin')
def _softmin(node, ins, ex):
    return [ex.node('Softmax', [ex.node('Neg', [ins[0]])], node['name'], axis=int(node['attrs'].get('axis', -1)))]


@register('log2', 'log10', 'log1p', 'expm1', 'cbrt', 'rcbrt', 'degrees', 'radians')
def _derived_unary(node, ins, ex):
    op, x = node['op'], ins[0]
    c = lambda v: ex.scalar_like(v, x)       # noqa: E731
    if op in ('log2', 'log10'):
        return [ex.node('Div', [ex.node('Log', [x]), c(float(np.log(2.0 if op == 'log2' else 10.0)))], node['name'])]
    if op == 'log1p':
        return [ex.node('Log', [ex.node('Add', [x, c(1.0)])], node['name'])]
    if op == 'expm1':
        return [ex.node('Sub', [ex.node('Exp', [x]), c(1.0)], node['name'])]
    if op in ('cbrt', 'rcbrt'):
        mag = ex.node('Pow', [ex.node('Abs', [x]), c(1.0 / 3.0)])
        y = ex.node('Mul', [ex.node('Sign', [x]), mag])
        return [ex.node('Reciprocal', [y], node['name'])] if op == 'rcbrt' else [ex.node('Identity', [y], node['name'])]
    return [ex.node('Mul', [x, c(180.0 / np.pi if op == 'degrees' else np.pi / 180.0)], node['name'])]


@register('broadcast_like')
def _broadcast_like(node, ins, ex):
    return [ex.node('Expand', [ins[0], ex.node('Shape', [ins[1]])], node['name'])]


@register('reshape_like')
def _reshape_like(node, ins, ex):
    return [ex.node('Reshape', [ins[0], ex.node('Shape', [ins[1]])], node['name'])]


@register('SequenceMask')
def _sequence_mask(node, ins, ex):
    """(T, N, ...) data, positions t >= length[n] replaced by `value` (axis 0 is time, as in the operator's default)."""
    a = node['attrs']
    if not a.get('use_sequence_length', False) or len(ins) < 2:
        return [ex.node('Identity', [ins[0]], node['name'])]
    shp = ex.shape(ins[0])
    if shp is None or int(a.get('axis', 0)) != 0:
        raise AttributeError('SequenceMask is exported for axis 0 with a known input shape')
    steps = ex.const(np.arange(shp[0]).reshape([shp[0], 1] + [1] * (len(shp) - 2)), 'steps', np.float32)
    lens = ex.node('Reshape', [ex.node('Cast', [ins[1]], to=P.FLOAT), ex.const([1, shp[1]] + [1] * (len(shp) - 2), 'shape', np.int64)])
    keep = ex.node('Less', [steps, lens])
    return [ex.node('Where', [keep, ins[0], ex.scalar_like(float(a.get('value', 0.0)), ins[0])], node['name'])]


# ---------------------------------------------------------------------------------------- driver
def _canonical(op_name):
    """Operator names in a graph file may be aliases; converters are keyed by the registry's primary name too."""
    if op_name in _CONVERTERS:
        return op_name
    from ..ops import registry
    if registry.has(op_name):
        primary = registry.get(op_name).name
        if primary in _CONVERTERS:
            return primary
        for alias in registry.get(op_name).aliases:
            if alias in _CONVERTERS:
                return alias
    return None


def export_model(sym, params, in_shapes=None, in_types=np.float32, onnx_file_path='model.onnx', verbose=False,
                 dynamic=False, dynamic_input_shapes=None, run_shape_inference=False, input_type=None, input_shape=None,
                 opset_version=13):
    """Export a Symbol (object or ``-symbol.json`` path) with its parameters (dict or ``.params`` path) to
    ``onnx_file_path`` and return that path.  ``in_shapes`` / ``in_types`` describe the data inputs in the order of
    ``sym.list_inputs()`` minus the parameters; with ``dynamic=True`` the graph inputs are declared with
    ``dynamic_input_shapes`` (strings or None mark free dimensions) while ``in_shapes`` still drives shape inference."""
    from ..symbol import load as sym_load
    from ..symbol.symbol import _parse_attr
    from ..ndarray.utils import load as nd_load
    if isinstance(sym, str):
        sym = sym_load(sym)
    if isinstance(params, str):
        params = nd_load(params)
    if isinstance(params, (list, tuple)):                 # (arg_params, aux_params)
        merged = {}
        for p in params:
            merged.update(p)
        params = merged
    params = {(k[4:] if k.startswith(('arg:', 'aux:')) else k): v for k, v in params.items()}
    in_shapes = in_shapes if in_shapes is not None else input_shape
    in_types = in_types if input_type is None else input_type
    graph = json.loads(sym.tojson())
    nodes = graph['nodes']
    data_names = [n['name'] for n in nodes if n['op'] == 'null' and n['name'] not in params]
    if in_shapes is not None and len(in_shapes) != len(data_names):
        raise MXNetError('in_shapes has %d entries for the %d data inputs %s' % (len(in_shapes), len(data_names), data_names))
    if not isinstance(in_types, (list, tuple)):
        in_types = [in_types] * len(data_names)
    data_types = {n: np.dtype(t) for n, t in zip(data_names, in_types)}
    # shapes and element types of every value, where the inputs' shapes are known
    shapes, dtypes = {}, {}
    for name, p in params.items():
        arr = p.asnumpy() if hasattr(p, 'asnumpy') else np.asarray(p)
        shapes[name], dtypes[name] = tuple(arr.shape), arr.dtype
    for n in data_names:
        dtypes[n] = data_types[n]
    if in_shapes is not None:
        feed = {n: tuple(s) for n, s in zip(data_names, in_shapes)}
        shapes.update(feed)
        try:
            internals = sym.get_internals()
            feed.update({k: v for k, v in shapes.items() if k in set(sym.list_inputs())})
            _, out_shapes, _ = internals.infer_shape(**feed)
            for oname, shp in zip(internals.list_outputs(), out_shapes):
                if shp is not None:
                    base = oname[:-len('_output')] if oname.endswith('_output') else oname
                    shapes.setdefault(base, tuple(shp))
        except Exception as e:   # pylint: disable=broad-except
            if verbose:
                print('shape inference failed (%s); converters that need shapes will say so' % e)
    ex = Exporter(int(opset_version), shapes, dtypes)
    inputs, names = [], {}
    declared = dynamic_input_shapes if dynamic and dynamic_input_shapes is not None else in_shapes
    shape_of = dict(zip(data_names, declared)) if declared is not None else {}
    for i, n in enumerate(nodes):
        if n['op'] == 'null':
            names[(i, 0)] = n['name']
            if n['name'] in params:
                p = params[n['name']]
                ex.initializers.append(P.make_tensor(n['name'], p.asnumpy() if hasattr(p, 'asnumpy') else np.asarray(p)))
            else:
                shp = shape_of.get(n['name'])
                shp = [d if isinstance(d, (int, np.integer)) and d > 0 else (d if isinstance(d, str) else 'dim_%d' % k)
                       for k, d in enumerate(shp)] if shp is not None else None
                inputs.append(P.make_value_info(n['name'], P.NP_TO_ONNX[data_types[n['name']]], shp))
            continue
        key = _canonical(n['op'])
        if key is None:
            raise AttributeError('No conversion function registered for op type %s yet.' % n['op'])
        attrs = {k: _parse_attr(v) for k, v in n.get('attrs', {}).items()}
        node = {'name': n['name'], 'op': key, 'attrs': attrs}
        ins = [names[(j[0], j[1])] for j in n['inputs']]
        outs = _CONVERTERS[key](node, ins, ex)
        for k, o in enumerate(outs):
            names[(i, k)] = o
            if k == 0 and ins and ins[0] in ex.dtypes and o not in ex.dtypes and key not in ('Cast', 'amp_cast', 'argmax', 'argmin'):
                ex.dtypes[o] = ex.dtypes[ins[0]]
        if key in ('Cast', 'amp_cast'):
            ex.dtypes[outs[0]] = np.dtype(str(attrs.get('dtype', 'float32')))
        if verbose:
            print('converted %s (%s) -> %s' % (n['name'], n['op'], outs))
    outputs = []
    for h in graph['heads']:
        oname = names[(h[0], h[1])]
        dt = ex.dtypes.get(oname) or np.dtype('float32')
        shp = ex.shapes.get(oname) if not dynamic else None
        outputs.append(P.make_value_info(oname, P.NP_TO_ONNX.get(np.dtype(dt), P.FLOAT), list(shp) if shp else None))
    g = P.make_graph(ex.nodes, 'mxnet_b200_converted_model', inputs, outputs, initializer=ex.initializers)
    from ..libinfo import __version__
    data = P.encode_model(P.make_model(g, opset_version=opset_version, producer_version=__version__))
    with open(onnx_file_path, 'wb') as f:
        f.write(data)
    return onnx_file_path

"""A reference evaluator for ONNX graphs (opset 13 semantics of the operators the exporter emits), built on the tensor
library: ``run_model(path_or_bytes, {input name: array}) -> [outputs]``.  It exists so that an exported model can be
checked against the network it came from without any ONNX runtime installed; it is not a deployment runtime."""
import numpy as np
import torch
import torch.nn.functional as F

from . import _proto

_TORCH = {_proto.FLOAT: torch.float32, _proto.UINT8: torch.uint8, _proto.INT8: torch.int8, _proto.INT16: torch.int16,
          _proto.INT32: torch.int32, _proto.INT64: torch.int64, _proto.BOOL: torch.bool, _proto.FLOAT16: torch.float16,
          _proto.DOUBLE: torch.float64, _proto.BFLOAT16: torch.bfloat16}


def _pads(pads, nd):
    """ONNX pads (begin_0.., end_0..) -> (symmetric padding or None, explicit F.pad list)."""
    pads = list(pads) if pads else [0] * (2 * nd)
    begin, end = pads[:nd], pads[nd:]
    flat = []
    for b, e in zip(reversed(begin), reversed(end)):
        flat += [b, e]
    return (tuple(begin) if begin == end else None), flat


def _pool(x, a, kind):
    k = a['kernel_shape']
    nd = len(k)
    strides = a.get('strides', [1] * nd)
    sym, flat = _pads(a.get('pads'), nd)
    ceil = bool(a.get('ceil_mode', 0))
    fn_max = {1: F.max_pool1d, 2: F.max_pool2d, 3: F.max_pool3d}[nd]
    fn_avg = {1: F.avg_pool1d, 2: F.avg_pool2d, 3: F.avg_pool3d}[nd]
    if kind == 'max':
        if sym is None:
            x = F.pad(x, flat, value=float('-inf'))
            sym = (0,) * nd
        return fn_max(x, k, strides, sym, ceil_mode=ceil)
    include = bool(a.get('count_include_pad', 0))
    if sym is None:
        if not include:
            raise NotImplementedError('asymmetric padding with count_include_pad=0')
        x = F.pad(x, flat)
        sym = (0,) * nd
    return fn_avg(x, k, strides, sym, ceil_mode=ceil, count_include_pad=include)


def _conv(x, w, b, a, transpose=False):
    nd = w.dim() - 2
    strides, dil, group = a.get('strides', [1] * nd), a.get('dilations', [1] * nd), a.get('group', 1)
    sym, flat = _pads(a.get('pads'), nd)
    if transpose:
        if sym is None:
            raise NotImplementedError('asymmetric padding in ConvTranspose')
        fn = {1: F.conv_transpose1d, 2: F.conv_transpose2d, 3: F.conv_transpose3d}[nd]
        return fn(x, w, b, strides, sym, tuple(a.get('output_padding', [0] * nd)), group, dil)
    if sym is None:
        x = F.pad(x, flat)
        sym = (0,) * nd
    fn = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[nd]
    return fn(x, w, b, strides, sym, dil, group)


def _reduce(fn):
    def run(ins, a):
        x = ins[0]
        axes = a.get('axes')
        if axes is None and len(ins) > 1 and ins[1] is not None:
            axes = [int(v) for v in ins[1].tolist()]
        keep = bool(a.get('keepdims', 1))
        if not axes:
            if a.get('noop_with_empty_axes', 0):
                return x
            axes = list(range(x.dim()))
        return fn(x, axes, keep)
    return run


def _slice(ins, a):
    x, starts, ends = ins[0], ins[1].tolist(), ins[2].tolist()
    axes = ins[3].tolist() if len(ins) > 3 and ins[3] is not None else list(range(len(starts)))
    steps = ins[4].tolist() if len(ins) > 4 and ins[4] is not None else [1] * len(starts)
    idx = [slice(None)] * x.dim()
    for s, e, ax, st in zip(starts, ends, axes, steps):
        n = x.shape[ax]
        if st > 0:
            s = min(max(s + n if s < 0 else s, 0), n)
            e = min(max(e + n if e < 0 else e, 0), n)
            idx[ax] = slice(s, e, st)
        else:
            # negative step: start is clamped to [0, n-1], end to [-1, n-1] (ONNX Slice-13)
            s = min(max(s + n if s < 0 else s, 0), n - 1)
            e = min(max(e + n if e < 0 else e, -1), n - 1) if e >= -n else -1
            sel = torch.arange(s, e, st)
            x = x.index_select(ax, sel)
    return x[tuple(idx)]


def _resize(ins, a):
    x = ins[0]
    scales = ins[2] if len(ins) > 2 and ins[2] is not None and ins[2].numel() else None
    sizes = ins[3] if len(ins) > 3 and ins[3] is not None and ins[3].numel() else None
    mode = a.get('mode', 'nearest')
    if mode != 'nearest':
        align = a.get('coordinate_transformation_mode', 'half_pixel') == 'align_corners'
        mode = {1: 'linear', 2: 'bilinear', 3: 'trilinear'}[x.dim() - 2]
        if sizes is not None:
            return F.interpolate(x, size=[int(v) for v in sizes.tolist()[2:]], mode=mode, align_corners=align)
        return F.interpolate(x, scale_factor=[float(v) for v in scales.tolist()[2:]], mode=mode, align_corners=align)
    if sizes is not None:
        return F.interpolate(x, size=[int(v) for v in sizes.tolist()[2:]], mode='nearest')
    return F.interpolate(x, scale_factor=[float(v) for v in scales.tolist()[2:]], mode='nearest')


def _gemm(ins, a):
    x, w = ins[0], ins[1]
    if a.get('transA', 0):
        x = x.t()
    if a.get('transB', 0):
        w = w.t()
    y = a.get('alpha', 1.0) * (x @ w)
    if len(ins) > 2 and ins[2] is not None:
        y = y + a.get('beta', 1.0) * ins[2]
    return y


def _batchnorm(ins, a):
    x, g, b, m, v = ins
    shape = [1, -1] + [1] * (x.dim() - 2)
    return (x - m.reshape(shape)) / torch.sqrt(v.reshape(shape) + a.get('epsilon', 1e-5)) * g.reshape(shape) + b.reshape(shape)


def _instancenorm(ins, a):
    x, g, b = ins
    axes = list(range(2, x.dim()))
    mean, var = x.mean(axes, keepdim=True), x.var(axes, unbiased=False, keepdim=True)
    shape = [1, -1] + [1] * (x.dim() - 2)
    return (x - mean) / torch.sqrt(var + a.get('epsilon', 1e-5)) * g.reshape(shape) + b.reshape(shape)


def _lrn(ins, a):
    return F.local_response_norm(ins[0], a['size'], a.get('alpha', 1e-4), a.get('beta', 0.75), a.get('bias', 1.0))


def _split(ins, a):
    x = ins[0]
    axis = a.get('axis', 0)
    if len(ins) > 1 and ins[1] is not None:
        return list(torch.split(x, [int(v) for v in ins[1].tolist()], axis))
    return list(torch.chunk(x, a['_nout'], axis))


def _pad(ins, a):
    x, pads = ins[0], [int(v) for v in ins[1].tolist()]
    value = float(ins[2]) if len(ins) > 2 and ins[2] is not None else 0.0
    nd = x.dim()
    flat = []
    for d in reversed(range(nd)):
        flat += [pads[d], pads[d + nd]]
    mode = a.get('mode', 'constant')
    if mode == 'constant':
        return F.pad(x, flat, value=value)
    while len(flat) > 2 and flat[-1] == 0 and flat[-2] == 0 and len(flat) // 2 > nd - 2:
        flat = flat[:-2]                          # reflect / replicate pad the trailing spatial axes only
    return F.pad(x, flat, mode={'reflect': 'reflect', 'edge': 'replicate'}[mode])


_UNARY = {'Relu': torch.relu, 'Sigmoid': torch.sigmoid, 'Tanh': torch.tanh, 'Softplus': F.softplus, 'Softsign': F.softsign,
          'Erf': torch.erf, 'Exp': torch.exp, 'Log': torch.log, 'Sqrt': torch.sqrt, 'Abs': torch.abs, 'Neg': torch.neg,
          'Reciprocal': torch.reciprocal, 'Floor': torch.floor, 'Ceil': torch.ceil, 'Round': torch.round, 'Sin': torch.sin,
          'Cos': torch.cos, 'Tan': torch.tan, 'Asin': torch.asin, 'Acos': torch.acos, 'Atan': torch.atan, 'Sinh': torch.sinh,
          'Cosh': torch.cosh, 'Asinh': torch.asinh, 'Acosh': torch.acosh, 'Atanh': torch.atanh, 'Sign': torch.sign,
          'Identity': lambda x: x, 'Not': torch.logical_not}
_BINARY = {'Add': torch.add, 'Sub': torch.sub, 'Mul': torch.mul, 'Div': torch.div, 'Pow': torch.pow,
           'Equal': torch.eq, 'Greater': torch.gt, 'Less': torch.lt, 'GreaterOrEqual': torch.ge, 'LessOrEqual': torch.le,
           'And': torch.logical_and, 'Or': torch.logical_or, 'Xor': torch.logical_xor, 'MatMul': torch.matmul}


def _depth_to_space_dcr(x, b):
    n, c, h, w = x.shape
    return x.reshape(n, b, b, c // (b * b), h, w).permute(0, 3, 4, 1, 5, 2).reshape(n, c // (b * b), h * b, w * b)


def _run_node(op, ins, a):
    if op in _UNARY:
        return _UNARY[op](ins[0])
    if op in _BINARY:
        return _BINARY[op](ins[0], ins[1])
    if op in ('Max', 'Min', 'Sum'):
        out = ins[0]
        for t in ins[1:]:
            out = {'Max': torch.maximum, 'Min': torch.minimum, 'Sum': torch.add}[op](out, t)
        return out
    if op == 'Conv':
        return _conv(ins[0], ins[1], ins[2] if len(ins) > 2 else None, a)
    if op == 'ConvTranspose':
        return _conv(ins[0], ins[1], ins[2] if len(ins) > 2 else None, a, True)
    if op == 'Gemm':
        return _gemm(ins, a)
    if op == 'LeakyRelu':
        return F.leaky_relu(ins[0], a.get('alpha', 0.01))
    if op == 'Elu':
        return F.elu(ins[0], a.get('alpha', 1.0))
    if op == 'Selu':
        return a.get('gamma', 1.0507009873554805) * F.elu(ins[0], a.get('alpha', 1.6732632423543772))
    if op == 'PRelu':
        return torch.where(ins[0] > 0, ins[0], ins[0] * ins[1])
    if op == 'Flatten':
        ax = a.get('axis', 1)
        return ins[0].reshape(int(np.prod(ins[0].shape[:ax])) if ax else 1, -1)
    if op == 'Reshape':
        shape = [int(v) for v in ins[1].tolist()]
        shape = [ins[0].shape[i] if s == 0 and not a.get('allowzero', 0) else s for i, s in enumerate(shape)]
        return ins[0].reshape(shape)
    if op == 'Transpose':
        perm = a.get('perm') or list(reversed(range(ins[0].dim())))
        return ins[0].permute(perm)
    if op == 'Concat':
        return torch.cat(ins, a['axis'])
    if op == 'Split':
        return _split(ins, a)
    if op == 'Slice':
        return _slice(ins, a)
    if op == 'Squeeze':
        axes = ins[1].tolist() if len(ins) > 1 and ins[1] is not None else None
        if axes is None:
            return ins[0].squeeze()
        out = ins[0]
        for ax in sorted([ax % ins[0].dim() for ax in axes], reverse=True):
            out = out.squeeze(ax)
        return out
    if op == 'Unsqueeze':
        out = ins[0]
        for ax in sorted(int(v) % (ins[0].dim() + len(ins[1])) for v in ins[1].tolist()):
            out = out.unsqueeze(ax)
        return out
    if op == 'Gather':
        idx = ins[1].long()
        ax = a.get('axis', 0)
        idx = torch.where(idx < 0, idx + ins[0].shape[ax], idx)
        return torch.index_select(ins[0], ax, idx.reshape(-1)).reshape(ins[0].shape[:ax] + idx.shape + ins[0].shape[ax + 1:])
    if op == 'Cast':
        return ins[0].to(_TORCH[a['to']])
    if op == 'Clip':
        lo = ins[1] if len(ins) > 1 and ins[1] is not None else None
        hi = ins[2] if len(ins) > 2 and ins[2] is not None else None
        return torch.clamp(ins[0], lo, hi)
    if op == 'Softmax':
        return torch.softmax(ins[0], a.get('axis', -1))
    if op == 'LogSoftmax':
        return torch.log_softmax(ins[0], a.get('axis', -1))
    if op == 'BatchNormalization':
        return _batchnorm(ins, a)
    if op == 'InstanceNormalization':
        return _instancenorm(ins, a)
    if op == 'LpNormalization':
        return ins[0] / torch.linalg.vector_norm(ins[0], a.get('p', 2), a.get('axis', -1), keepdim=True)
    if op == 'LRN':
        return _lrn(ins, a)
    if op == 'MaxPool':
        return _pool(ins[0], a, 'max')
    if op == 'AveragePool':
        return _pool(ins[0], a, 'avg')
    if op == 'GlobalMaxPool':
        return ins[0].amax(list(range(2, ins[0].dim())), keepdim=True)
    if op == 'GlobalAveragePool':
        return ins[0].mean(list(range(2, ins[0].dim())), keepdim=True)
    if op == 'ReduceSum':
        return _reduce(lambda x, ax, k: x.sum(ax, keepdim=k))(ins, a)
    if op == 'ReduceMean':
        return _reduce(lambda x, ax, k: x.mean(ax, keepdim=k))(ins, a)
    if op == 'ReduceMax':
        return _reduce(lambda x, ax, k: x.amax(ax, keepdim=k))(ins, a)
    if op == 'ReduceMin':
        return _reduce(lambda x, ax, k: x.amin(ax, keepdim=k))(ins, a)
    if op == 'ReduceL2':
        return _reduce(lambda x, ax, k: torch.linalg.vector_norm(x, 2, ax, keepdim=k))(ins, a)
    if op == 'ReduceProd':
        def prod(x, ax, k):
            for d in sorted(ax, reverse=True):
                x = x.prod(d, keepdim=k)
            return x
        return _reduce(prod)(ins, a)
    if op in ('ArgMax', 'ArgMin'):
        fn = torch.argmax if op == 'ArgMax' else torch.argmin
        return fn(ins[0], a.get('axis', 0), keepdim=bool(a.get('keepdims', 1)))
    if op == 'Where':
        return torch.where(ins[0].bool(), ins[1], ins[2])
    if op == 'Pad':
        return _pad(ins, a)
    if op == 'Resize':
        return _resize(ins, a)
    if op == 'Tile':
        return ins[0].repeat([int(v) for v in ins[1].tolist()])
    if op == 'Expand':
        shape = [int(v) for v in ins[1].tolist()]
        return ins[0] * torch.ones(shape, dtype=ins[0].dtype)
    if op == 'Shape':
        return torch.tensor(list(ins[0].shape), dtype=torch.int64)
    if op == 'ConstantOfShape':
        value = a.get('value')
        fill = torch.from_numpy(np.asarray(value)) if value is not None else torch.zeros(1)
        return torch.full([int(v) for v in ins[0].tolist()], fill.reshape(-1)[0].item(), dtype=fill.dtype)
    if op == 'Constant':
        return torch.from_numpy(np.asarray(a['value']))
    if op == 'Dropout':
        return ins[0]
    if op == 'OneHot':
        depth = int(ins[1].reshape(-1)[0])
        idx = ins[0].long()
        idx = torch.where(idx < 0, idx + depth, idx)
        hot = F.one_hot(idx.clamp(0, depth - 1), depth).to(ins[2].dtype)
        hot = hot * (ins[2][1] - ins[2][0]) + ins[2][0]
        ax = a.get('axis', -1)
        return hot if ax in (-1, hot.dim() - 1) else hot.movedim(-1, ax)
    if op == 'DepthToSpace':
        return F.pixel_shuffle(ins[0], a['blocksize']) if a.get('mode', 'DCR') == 'CRD' else _depth_to_space_dcr(ins[0], a['blocksize'])
    if op == 'SpaceToDepth':
        b = a['blocksize']
        n, c, h, w = ins[0].shape
        return ins[0].reshape(n, c, h // b, b, w // b, b).permute(0, 3, 5, 1, 2, 4).reshape(n, c * b * b, h // b, w // b)
    if op == 'Size':
        return torch.tensor(ins[0].numel(), dtype=torch.int64)
    if op == 'TopK':
        k = int(ins[1].reshape(-1)[0])
        v, i = torch.topk(ins[0], k, dim=a.get('axis', -1), largest=bool(a.get('largest', 1)), sorted=True)
        return [v, i]
    if op == 'HardSigmoid':
        return torch.clamp(a.get('alpha', 0.2) * ins[0] + a.get('beta', 0.5), 0, 1)
    raise NotImplementedError('ONNX operator %s is not implemented by this evaluator' % op)


def load_model(model):
    """Path, bytes or an already decoded model dict -> model dict."""
    if isinstance(model, dict):
        return model
    if isinstance(model, (bytes, bytearray, memoryview)):
        return _proto.decode_model(bytes(model))
    with open(model, 'rb') as f:
        return _proto.decode_model(f.read())


def run_model(model, inputs):
    """Evaluate the graph.  ``inputs``: {graph input name: numpy array or NDArray}.  Returns a list of numpy arrays in
    the order of the graph's outputs."""
    m = load_model(model)
    g = m['graph']
    env = {'': None}
    for t in g['initializer']:
        env[t['name']] = torch.from_numpy(_proto.tensor_to_numpy(t))
    for vi in g['input']:
        if vi['name'] in env:
            continue
        if vi['name'] not in inputs:
            raise KeyError('missing graph input %s' % vi['name'])
        v = inputs[vi['name']]
        v = v.asnumpy() if hasattr(v, 'asnumpy') else np.asarray(v)
        env[vi['name']] = torch.from_numpy(np.ascontiguousarray(v))
    with torch.no_grad():
        for n in g['node']:
            attrs = {a['name']: _proto.attribute_value(a) for a in n['attribute']}
            attrs['_nout'] = len(n['output'])
            ins = [env[i] for i in n['input']]
            out = _run_node(n['op_type'], ins, attrs)
            outs = out if isinstance(out, (list, tuple)) else [out]
            for name, o in zip(n['output'], outs):
                if name:
                    env[name] = o
    return [env[o['name']].numpy() for o in g['output']]

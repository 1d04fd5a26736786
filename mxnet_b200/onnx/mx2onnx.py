"""Symbol → ONNX graph translation."""
import json

import numpy as np

_CONVERTERS = {}


def register(op_name):
    def deco(fn):
        _CONVERTERS[op_name] = fn
        return fn
    return deco


def get_operator_support(opset_version=None):
    return sorted(_CONVERTERS)


def _tuple(v, default):
    if v is None or v == ():
        return list(default)
    return [int(x) for x in (v if isinstance(v, (list, tuple)) else (v,))]


@register('Convolution')
def _conv(node, ins, helper):
    a = node['attrs']
    k = _tuple(a.get('kernel'), ())
    return [helper.make_node('Conv', ins, [node['name']], kernel_shape=k, strides=_tuple(a.get('stride'), [1] * len(k)),
                             dilations=_tuple(a.get('dilate'), [1] * len(k)), pads=_tuple(a.get('pad'), [0] * len(k)) * 2,
                             group=int(a.get('num_group', 1)), name=node['name'])]


@register('FullyConnected')
def _fc(node, ins, helper):
    flat = node['name'] + '_flatten'
    nodes = [helper.make_node('Flatten', [ins[0]], [flat], name=flat)] if node['attrs'].get('flatten', True) else []
    src = flat if nodes else ins[0]
    nodes.append(helper.make_node('Gemm', [src] + ins[1:], [node['name']], alpha=1.0, beta=1.0, transA=0, transB=1, name=node['name']))
    return nodes


@register('BatchNorm')
def _bn(node, ins, helper):
    a = node['attrs']
    return [helper.make_node('BatchNormalization', ins[:5], [node['name']], epsilon=float(a.get('eps', 1e-3)),
                             momentum=float(a.get('momentum', 0.9)), name=node['name'])]


@register('Activation')
def _act(node, ins, helper):
    t = {'relu': 'Relu', 'sigmoid': 'Sigmoid', 'tanh': 'Tanh', 'softrelu': 'Softplus', 'softsign': 'Softsign'}[node['attrs'].get('act_type', 'relu')]
    return [helper.make_node(t, ins, [node['name']], name=node['name'])]


@register('Pooling')
def _pool(node, ins, helper):
    a = node['attrs']
    pt = a.get('pool_type', 'max')
    if a.get('global_pool', False):
        return [helper.make_node('GlobalMaxPool' if pt == 'max' else 'GlobalAveragePool', ins, [node['name']], name=node['name'])]
    k = _tuple(a.get('kernel'), ())
    kw = dict(kernel_shape=k, strides=_tuple(a.get('stride'), [1] * len(k)), pads=_tuple(a.get('pad'), [0] * len(k)) * 2,
              ceil_mode=int(a.get('pooling_convention', 'valid') == 'full'))
    if pt == 'avg':
        kw['count_include_pad'] = int(a.get('count_include_pad', True) in (True, None))
    return [helper.make_node('MaxPool' if pt == 'max' else 'AveragePool', ins, [node['name']], name=node['name'], **kw)]


for _mx, _ox in (('Flatten', 'Flatten'), ('elemwise_add', 'Add'), ('broadcast_add', 'Add'), ('_npi_add', 'Add'),
                 ('elemwise_mul', 'Mul'), ('broadcast_mul', 'Mul'), ('elemwise_sub', 'Sub'), ('broadcast_sub', 'Sub'),
                 ('relu', 'Relu'), ('sigmoid', 'Sigmoid'), ('tanh', 'Tanh'), ('exp', 'Exp'), ('log', 'Log'), ('sqrt', 'Sqrt'),
                 ('identity', 'Identity'), ('_copy', 'Identity')):
    def _mk(ox):
        def conv(node, ins, helper):
            return [helper.make_node(ox, ins, [node['name']], name=node['name'])]
        return conv
    _CONVERTERS[_mx] = _mk(_ox)


@register('softmax')
def _softmax(node, ins, helper):
    return [helper.make_node('Softmax', ins[:1], [node['name']], axis=int(node['attrs'].get('axis', -1)), name=node['name'])]


@register('Concat')
def _concat(node, ins, helper):
    return [helper.make_node('Concat', ins, [node['name']], axis=int(node['attrs'].get('dim', 1)), name=node['name'])]


@register('Dropout')
def _dropout(node, ins, helper):
    return [helper.make_node('Identity', ins[:1], [node['name']], name=node['name'])]


@register('LayerNorm')
def _ln(node, ins, helper):
    a = node['attrs']
    return [helper.make_node('LayerNormalization', ins, [node['name']], axis=int(a.get('axis', -1)), epsilon=float(a.get('eps', 1e-5)), name=node['name'])]


@register('Reshape')
def _reshape(node, ins, helper):
    import onnx
    shape_name = node['name'] + '_shape'
    shp = np.asarray(node['attrs'].get('shape', ()), dtype=np.int64)
    const = helper.make_node('Constant', [], [shape_name], value=onnx.numpy_helper.from_array(shp, shape_name))
    return [const, helper.make_node('Reshape', [ins[0], shape_name], [node['name']], name=node['name'])]


@register('transpose')
def _transpose(node, ins, helper):
    axes = node['attrs'].get('axes')
    kw = {'perm': [int(a) for a in axes]} if axes else {}
    return [helper.make_node('Transpose', ins, [node['name']], name=node['name'], **kw)]


def export_model(sym, params, in_shapes=None, in_types=np.float32, onnx_file_path='model.onnx', verbose=False,
                 dynamic=False, dynamic_input_shapes=None, run_shape_inference=False, input_type=None, input_shape=None,
                 opset_version=13):
    """Export a Symbol (object or ``-symbol.json`` path) and its params (dict or ``.params`` path)."""
    try:
        import onnx
        from onnx import helper, TensorProto, numpy_helper
    except ImportError as e:
        raise ImportError('Onnx and protobuf need to be installed to export models: %s' % e)
    from ..symbol import load as sym_load, Symbol
    from ..symbol.symbol import _parse_attr
    from ..ndarray.utils import load as nd_load
    if isinstance(sym, str):
        sym = sym_load(sym)
    if isinstance(params, str):
        params = nd_load(params)
    params = {(k[4:] if k.startswith(('arg:', 'aux:')) else k): v for k, v in params.items()}
    in_shapes = in_shapes or input_shape
    graph = json.loads(sym.tojson())
    nodes = graph['nodes']
    onnx_nodes, initializers, inputs = [], [], []
    names = {}
    data_inputs = [n['name'] for i, n in enumerate(nodes) if n['op'] == 'null' and n['name'] not in params]
    shape_it = iter(in_shapes or [])
    for i, n in enumerate(nodes):
        names[i] = n['name']
        if n['op'] == 'null':
            if n['name'] in params:
                initializers.append(numpy_helper.from_array(params[n['name']].asnumpy(), n['name']))
            else:
                shp = next(shape_it, None)
                inputs.append(helper.make_tensor_value_info(n['name'], TensorProto.FLOAT, list(shp) if shp else None))
            continue
        if n['op'] not in _CONVERTERS:
            raise AttributeError('No conversion function registered for op type %s yet.' % n['op'])
        node = {'name': n['name'], 'attrs': {k: _parse_attr(v) for k, v in n.get('attrs', {}).items()}}
        onnx_nodes.extend(_CONVERTERS[n['op']](node, [names[j[0]] for j in n['inputs']], helper))
    outputs = [helper.make_tensor_value_info(names[h[0]], TensorProto.FLOAT, None) for h in graph['heads']]
    g = helper.make_graph(onnx_nodes, 'mxnet_b200_converted_model', inputs, outputs, initializer=initializers)
    model = helper.make_model(g, opset_imports=[helper.make_opsetid('', opset_version)])
    onnx.save(model, onnx_file_path)
    return onnx_file_path

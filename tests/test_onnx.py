"""ONNX export: the in-tree protobuf reader and evaluator are validated against a model written by the tensor library's
own (independent) ONNX serializer; exported networks are then evaluated and compared with the network they came from."""
import io
import os

import numpy as np
import pytest
import torch

import mxnet_b200 as mx
from mxnet_b200 import gluon, nd
from mxnet_b200.onnx import _proto, backend


def _rel(a, b):
    return float(np.abs(a - b).max() / (np.abs(b).max() + 1e-30))


def test_reader_and_evaluator_on_a_model_from_an_independent_writer():
    try:
        from torch.onnx._internal.torchscript_exporter import onnx_proto_utils
    except ImportError:
        pytest.skip('this version of the tensor library has no TorchScript ONNX serializer')

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.c = torch.nn.Conv2d(3, 8, 3, padding=1, stride=2)
            self.bn = torch.nn.BatchNorm2d(8)
            self.p = torch.nn.MaxPool2d(3, 2, 1)
            self.l = torch.nn.Linear(8, 5)
            self.ct = torch.nn.ConvTranspose2d(8, 4, 2, stride=2)
            self.ln = torch.nn.LayerNorm(5)

        def forward(self, x):
            h = self.p(torch.relu(self.bn(self.c(x))))
            u = self.ct(h).mean((2, 3))
            g = torch.nn.functional.gelu(h.mean((2, 3)))
            return torch.softmax(self.ln(self.l(g)), -1), torch.cat([u, g[:, 1:3] * 2 - 1], 1).clamp(-0.5, 0.5)
    keep = onnx_proto_utils._add_onnxscript_fn
    onnx_proto_utils._add_onnxscript_fn = lambda proto, custom_opsets: proto       # that step needs the onnx package
    try:
        net, x, f = Net().eval(), torch.randn(2, 3, 16, 16), io.BytesIO()
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter('ignore')
            torch.onnx.export(net, (x,), f, opset_version=13, dynamo=False)
    except Exception as e:   # pylint: disable=broad-except
        pytest.skip('the serializer is not usable here: %s' % e)
    finally:
        onnx_proto_utils._add_onnxscript_fn = keep
    model = backend.load_model(f.getvalue())
    assert model['opset_import'][0]['version'] == 13 and model['producer_name'] == 'pytorch'
    ops = {n['op_type'] for n in model['graph']['node']}
    assert {'Conv', 'ConvTranspose', 'Gemm', 'MaxPool', 'Softmax', 'Erf', 'Slice', 'Clip'} <= ops
    outs = backend.run_model(model, {model['graph']['input'][0]['name']: x.numpy()})
    for o, r in zip(outs, net(x)):
        np.testing.assert_allclose(o, r.detach().numpy(), rtol=1e-5, atol=1e-6)
    # what the writer produces from the decoded model decodes to the same graph again
    again = _proto.decode_model(_proto.encode_model(model))
    assert [n['op_type'] for n in again['graph']['node']] == [n['op_type'] for n in model['graph']['node']]
    assert [t['raw_data'] for t in again['graph']['initializer']] == [t['raw_data'] for t in model['graph']['initializer']]


@pytest.mark.parametrize('name,size', [('resnet18_v1', 32), ('mobilenet_v2_0_25', 32), ('squeezenet1_1', 64), ('vgg11_bn', 32)])
def test_model_zoo_networks_export_and_evaluate(tmp_path, name, size):
    net = gluon.model_zoo.vision.get_model(name, classes=7)
    net.initialize(mx.init.Normal(0.15))
    x = nd.array(np.random.RandomState(0).rand(2, 3, size, size).astype('float32'))
    net.hybridize()
    net(x)
    ref = net(x).asnumpy()
    sym_file, params_file = net.export(str(tmp_path / name))
    out = mx.onnx.export_model(sym_file, params_file, in_shapes=[(2, 3, size, size)], in_types=[np.float32],
                               onnx_file_path=str(tmp_path / (name + '.onnx')))
    model = backend.load_model(out)
    assert model['graph']['input'][0]['shape'] == [2, 3, size, size] and model['graph']['output'][0]['shape'] == [2, 7]
    assert _rel(backend.run_model(model, {'data': x.asnumpy()})[0], ref) < 1e-4


def test_transformer_style_graph_with_shape_codes(tmp_path):
    T, B, C, H = 6, 2, 16, 4
    tok, x = mx.sym.var('tokens'), mx.sym.var('x')
    emb = mx.sym.Embedding(tok, mx.sym.var('emb_weight'), input_dim=11, output_dim=C, name='emb')        # (B, T, C)
    h = mx.sym.LayerNorm(emb + x, mx.sym.var('ln_gamma'), mx.sym.var('ln_beta'), axis=-1, eps=1e-5, name='ln')
    qkv = mx.sym.FullyConnected(h, mx.sym.var('qkv_weight'), mx.sym.var('qkv_bias'), num_hidden=3 * C, flatten=False, name='qkv')
    q, k, v = mx.sym.split(qkv, num_outputs=3, axis=2, name='split')

    def heads(t, name):
        t = mx.sym.Reshape(t, shape=(0, 0, -4, H, -1), name=name + '_r')                                   # (B, T, H, C/H)
        return mx.sym.Reshape(mx.sym.transpose(t, axes=(0, 2, 1, 3), name=name + '_t'), shape=(-3, 0, 0), name=name + '_m')
    q, k, v = heads(q, 'q'), heads(k, 'k'), heads(v, 'v')
    att = mx.sym.softmax(mx.sym.batch_dot(q, k, transpose_b=True, name='qk') / 2.0, axis=-1, name='att')
    ctx = mx.sym.batch_dot(att, v, name='ctx')                                                             # (B*H, T, C/H)
    ctx = mx.sym.Reshape(mx.sym.transpose(mx.sym.Reshape(ctx, shape=(-4, -1, H, 0, 0), name='c_r'), axes=(0, 2, 1, 3), name='c_t'),
                         shape=(0, 0, -3), name='c_m')                                                    # (B, T, C)
    ff = mx.sym.LeakyReLU(mx.sym.FullyConnected(ctx, mx.sym.var('ff_weight'), None, num_hidden=C, no_bias=True, flatten=False,
                                                name='ff'), act_type='gelu', name='gelu')
    pooled = mx.sym.mean(mx.sym.slice_axis(ff, axis=1, begin=1, end=None, name='sl'), axis=1, name='pool')
    extra = mx.sym.clip(mx.sym.sum(mx.sym.square(ff), axis=(1, 2), keepdims=False, name='ssq'), a_min=0.0, a_max=50.0, name='clip')
    out = mx.sym.Concat(pooled * 2.0 - 1.0, mx.sym.expand_dims(mx.sym.sqrt(extra), axis=1), dim=1, name='cat')
    rng = np.random.RandomState(1)
    params = {'emb_weight': rng.randn(11, C), 'ln_gamma': rng.rand(C) + 0.5, 'ln_beta': rng.randn(C) * 0.1,
              'qkv_weight': rng.randn(3 * C, C) * 0.3, 'qkv_bias': rng.randn(3 * C) * 0.1, 'ff_weight': rng.randn(C, C) * 0.3}
    params = {k: nd.array(v.astype('float32')) for k, v in params.items()}
    tokens = rng.randint(0, 11, (B, T)).astype('float32')
    xv = rng.randn(B, T, C).astype('float32')
    feed = dict(params, tokens=nd.array(tokens), x=nd.array(xv))
    ref = out._bind(mx.cpu(), feed).forward()[0].asnumpy()
    assert ref.shape == (B, C + 1)
    path = mx.onnx.export_model(out, params, in_shapes=[(B, T), (B, T, C)], in_types=[np.float32, np.float32],
                                onnx_file_path=str(tmp_path / 'attn.onnx'))
    got = mx.onnx.run_model(path, {'tokens': tokens, 'x': xv})[0]
    np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-5)
    ops = [n['op_type'] for n in backend.load_model(path)['graph']['node']]
    assert 'Gather' in ops and 'Erf' in ops and 'Split' in ops and ops.count('MatMul') >= 4


def test_operator_table_and_unknown_operator(tmp_path):
    support = mx.onnx.get_operator_support()
    assert {'Convolution', 'FullyConnected', 'BatchNorm', 'Pooling', 'LayerNorm', 'Embedding', 'batch_dot', 'softmax'} <= set(support)
    s = mx.sym.sort(mx.sym.var('data'))
    with pytest.raises(AttributeError, match='No conversion function registered'):
        mx.onnx.export_model(s, {}, in_shapes=[(2, 5)], onnx_file_path=str(tmp_path / 'x.onnx'))


def test_dynamic_batch_declaration_and_nhwc_layers(tmp_path):
    data = mx.sym.var('data')
    c = mx.sym.Convolution(data, mx.sym.var('w'), mx.sym.var('b'), kernel=(3, 3), pad=(1, 1), num_filter=8, layout='NHWC', name='conv')
    c = mx.sym.BatchNorm(c, mx.sym.var('g'), mx.sym.var('be'), mx.sym.var('mm'), mx.sym.var('mv'), axis=3, fix_gamma=False, eps=1e-5,
                         name='bn')
    p = mx.sym.Pooling(mx.sym.relu(c), kernel=(2, 2), stride=(2, 2), pool_type='max', layout='NHWC', name='pool')
    out = mx.sym.Pooling(p, global_pool=True, pool_type='avg', kernel=(1, 1), layout='NHWC', name='gap')
    rng = np.random.RandomState(2)
    params = {'w': rng.randn(8, 3, 3, 4) * 0.3, 'b': rng.randn(8) * 0.1, 'g': rng.rand(8) + 0.5, 'be': rng.randn(8) * 0.1,
              'mm': rng.randn(8) * 0.1, 'mv': rng.rand(8) + 0.5}
    params = {k: nd.array(v.astype('float32')) for k, v in params.items()}
    path = mx.onnx.export_model(out, params, in_shapes=[(2, 6, 6, 4)], dynamic=True, dynamic_input_shapes=[('batch', 6, 6, 4)],
                                onnx_file_path=str(tmp_path / 'nhwc.onnx'))
    model = backend.load_model(path)
    assert model['graph']['input'][0]['shape'] == ['batch', 6, 6, 4]
    for batch in (2, 5):
        x = rng.randn(batch, 6, 6, 4).astype('float32')
        args = {k: v for k, v in params.items() if k not in ('mm', 'mv')}
        ref = out._bind(mx.cpu(), dict(args, data=nd.array(x)), aux_states={'mm': params['mm'], 'mv': params['mv']}).forward(
            is_train=False)[0].asnumpy()
        np.testing.assert_allclose(backend.run_model(model, {'data': x})[0], ref, rtol=1e-4, atol=1e-5)


def _export_and_compare(tmp_path, sym, feeds, rtol=1e-5, atol=1e-6):
    import mxnet_b200 as mx
    names = sym.list_inputs()
    path = str(tmp_path / 'm.onnx')
    mx.onnx.export_model(sym, {}, [feeds[n].shape for n in names], [feeds[n].dtype for n in names], path)
    got = mx.onnx.run_model(path, feeds)
    ex = sym.bind(mx.cpu(), {n: mx.nd.array(feeds[n], dtype=feeds[n].dtype) for n in names})
    want = [o.asnumpy() for o in ex.forward()]
    assert len(got) == len(want)
    for g, w in zip(got, want):
        assert g.shape == w.shape
        np.testing.assert_allclose(g.astype('float64'), w.astype('float64'), rtol=rtol, atol=atol)


@pytest.mark.parametrize('case', ['compare', 'logic', 'take', 'one_hot', 'stack_repeat', 'reverse_swap', 'd2s', 'shape_size',
                                  'topk', 'unary', 'like', 'sequence_mask'])
def test_more_operator_converters(tmp_path, case):
    """Comparison / logical / indexing / layout operators: exported, evaluated by the in-tree ONNX evaluator and compared
    with the Symbol executor on the same inputs."""
    import mxnet_b200 as mx
    rng = np.random.RandomState(2)
    a, b = mx.sym.var('a'), mx.sym.var('b')
    x = rng.randn(3, 4).astype('float32')
    y = rng.randn(3, 4).astype('float32')
    y[0] = x[0]
    if case == 'compare':
        sym = mx.sym.Group([mx.sym.broadcast_equal(a, b), mx.sym.broadcast_not_equal(a, b), mx.sym.broadcast_greater(a, b),
                            mx.sym.broadcast_lesser_equal(a, b), a > 0.2, a <= -0.1])
        feeds = {'a': x, 'b': y}
    elif case == 'logic':
        xa, xb = (x > 0).astype('float32'), (y > 0.3).astype('float32')
        sym = mx.sym.Group([mx.sym.broadcast_logical_and(a, b), mx.sym.broadcast_logical_or(a, b),
                            mx.sym.broadcast_logical_xor(a, b), mx.sym.logical_not(a)])
        feeds = {'a': xa, 'b': xb}
    elif case == 'take':
        sym = mx.sym.Group([mx.sym.take(a, b, axis=0), mx.sym.take(a, b, axis=1)])
        feeds = {'a': x, 'b': np.array([[0, 2], [1, 7]], dtype='float32')}          # 7 is clipped
    elif case == 'one_hot':
        sym = mx.sym.one_hot(a, depth=5, on_value=2.0, off_value=-1.0)
        feeds = {'a': np.array([0, 3, 4, 1], dtype='float32')}
    elif case == 'stack_repeat':
        sym = mx.sym.Group([mx.sym.stack(a, b, axis=1), mx.sym.repeat(a, repeats=3, axis=1)])
        feeds = {'a': x, 'b': y}
    elif case == 'reverse_swap':
        sym = mx.sym.Group([mx.sym.reverse(a, axis=1), mx.sym.swapaxes(a, dim1=0, dim2=1)])
        feeds = {'a': x}
    elif case == 'd2s':
        sym = mx.sym.Group([mx.sym.depth_to_space(a, block_size=2), mx.sym.space_to_depth(b, block_size=2)])
        feeds = {'a': rng.randn(2, 8, 3, 3).astype('float32'), 'b': rng.randn(2, 2, 4, 6).astype('float32')}
    elif case == 'shape_size':
        sym = mx.sym.Group([mx.sym.shape_array(a), mx.sym.size_array(a)])
        feeds = {'a': x}
    elif case == 'topk':
        sym = mx.sym.Group([mx.sym.topk(a, k=2, axis=-1, ret_typ='value'), mx.sym.topk(a, k=2, axis=-1, ret_typ='indices'),
                            mx.sym.topk(a, k=1, axis=0, ret_typ='value', is_ascend=True)])
        feeds = {'a': x}
    elif case == 'unary':
        pos = np.abs(x) + 0.5
        sym = mx.sym.Group([mx.sym.log2(a), mx.sym.log10(a), mx.sym.log1p(a), mx.sym.expm1(a), mx.sym.cbrt(b), mx.sym.rcbrt(a),
                            mx.sym.degrees(b), mx.sym.radians(b), mx.sym.hard_sigmoid(b), mx.sym.softmin(b, axis=-1)])
        feeds = {'a': pos, 'b': x}
    elif case == 'like':
        sym = mx.sym.Group([mx.sym.broadcast_like(a, b), mx.sym.reshape_like(b, mx.sym.var('c'))])
        feeds = {'a': x[:1], 'b': y, 'c': np.zeros((2, 6), dtype='float32')}
    else:
        sym = mx.sym.SequenceMask(a, b, use_sequence_length=True, value=-7.0)
        feeds = {'a': rng.randn(5, 3, 2).astype('float32'), 'b': np.array([2, 5, 0], dtype='float32')}
    _export_and_compare(tmp_path, sym, feeds, rtol=1e-4, atol=1e-5)

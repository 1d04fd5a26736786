"""Gluon blocks, parameters, layers, hybridize/export/import and Trainer (reference:
tests/python/unittest/test_gluon.py, test_gluon_trainer.py)."""
import json
import os

import numpy as np
import pytest

import mxnet_b200 as mx
from mxnet_b200 import autograd, gluon, nd
from mxnet_b200.gluon import nn
from mxnet_b200.test_utils import assert_almost_equal, same


def test_parameter_basics():
    p = gluon.Parameter('weight', shape=(10, 10))
    p.initialize(init='xavier', ctx=[mx.cpu(0), mx.cpu(1)])
    assert len(p.list_data()) == 2 and len(p.list_grad()) == 2
    assert p.data(mx.cpu(1)).context == mx.cpu(1)
    assert p.data(mx.cpu(0)).shape == (10, 10)
    assert p.grad(mx.cpu(0)).stype == 'default'
    assert same(p.data(mx.cpu(0)).asnumpy(), p.data(mx.cpu(1)).asnumpy())
    p.reset_ctx(ctx=[mx.cpu(1), mx.cpu(2)])
    assert p.list_ctx() == [mx.cpu(1), mx.cpu(2)]
    p.zero_grad()
    p.set_data(nd.ones((10, 10)))
    assert float(p.data(mx.cpu(2)).sum().asscalar()) == 100


def test_parameter_invalid_access_and_deferred():
    p = gluon.Parameter('weight', shape=(10, 10))
    with pytest.raises(RuntimeError):
        p.data()
    with pytest.raises(RuntimeError):
        p.list_data()
    d = nn.Dense(4)
    d.initialize()
    with pytest.raises(gluon.parameter.DeferredInitializationError):
        d.weight.data()
    d(nd.ones((2, 7)))
    assert d.weight.shape == (4, 7)


def test_constant_and_grad_req():
    class Net(gluon.HybridBlock):
        def __init__(self):
            super().__init__()
            self.c = gluon.Constant(np.array([[1., 2.], [3., 4.]]))

        def forward(self, x):
            return x + self.c.data(x.context)
    net = Net()
    net.initialize()
    x = nd.ones((2, 2))
    x.attach_grad()
    with autograd.record():
        y = net(x)
    y.backward()
    assert same(y.asnumpy(), np.array([[2., 3.], [4., 5.]], 'float32'))
    assert net.c.grad_req == 'null'
    d = nn.Dense(3, in_units=2)
    d.initialize()
    d.setattr('grad_req', 'null')
    assert d.weight.grad_req == 'null'
    with pytest.raises(RuntimeError):
        d.weight.grad()


def test_collect_params_names_and_select():
    net = nn.HybridSequential()
    net.add(nn.Dense(8, in_units=4), nn.BatchNorm(in_channels=8), nn.Dense(2, in_units=8))
    names = list(net.collect_params().keys())
    assert names == ['0.weight', '0.bias', '1.gamma', '1.beta', '1.running_mean', '1.running_var', '2.weight', '2.bias']
    assert list(net.collect_params('.*weight').keys()) == ['0.weight', '2.weight']
    assert list(net.collect_params('0.*|.*beta').keys()) == ['0.weight', '0.bias', '1.beta']


def test_dense_conv_pool_shapes_and_values():
    d = nn.Dense(5, in_units=3, activation='relu', flatten=False)
    d.initialize()
    x = nd.array(np.random.randn(2, 4, 3))
    ref = np.maximum(x.asnumpy() @ d.weight.data().asnumpy().T + d.bias.data().asnumpy(), 0)
    assert_almost_equal(d(x).asnumpy(), ref, rtol=1e-5, atol=1e-6)
    c = nn.Conv2D(6, kernel_size=3, strides=2, padding=1, in_channels=3)
    c.initialize()
    assert c(nd.ones((2, 3, 9, 9))).shape == (2, 6, 5, 5)
    c = nn.Conv2D(6, kernel_size=3, padding=1, in_channels=3, layout='NHWC')
    c.initialize()
    assert c.weight.shape == (6, 3, 3, 3) and c(nd.ones((2, 9, 9, 3))).shape == (2, 9, 9, 6)
    ct = nn.Conv2DTranspose(4, kernel_size=4, strides=2, padding=1, in_channels=3)
    ct.initialize()
    assert ct(nd.ones((1, 3, 8, 8))).shape == (1, 4, 16, 16)
    assert nn.MaxPool2D(2)(nd.ones((1, 2, 8, 8))).shape == (1, 2, 4, 4)
    assert nn.AvgPool2D(3, 2, 1)(nd.ones((1, 2, 8, 8))).shape == (1, 2, 4, 4)
    assert nn.GlobalAvgPool2D()(nd.ones((1, 2, 8, 8))).shape == (1, 2, 1, 1)
    assert nn.MaxPool2D(3, 2, ceil_mode=True)(nd.ones((1, 1, 8, 8))).shape == (1, 1, 4, 4)
    assert nn.Flatten()(nd.ones((2, 3, 4))).shape == (2, 12)
    c1 = nn.Conv1D(4, 3, in_channels=2)
    c1.initialize()
    assert c1(nd.ones((1, 2, 10))).shape == (1, 4, 8)
    g = nn.Conv2D(8, 3, groups=4, in_channels=4, padding=1)
    g.initialize()
    assert g.weight.shape == (8, 1, 3, 3) and g(nd.ones((1, 4, 5, 5))).shape == (1, 8, 5, 5)


def test_conv_matches_numpy_reference():
    c = nn.Conv2D(2, kernel_size=2, in_channels=1, use_bias=True)
    c.initialize()
    x = np.random.randn(1, 1, 3, 3).astype('float32')
    w, b = c.weight.data().asnumpy(), c.bias.data().asnumpy()
    ref = np.zeros((1, 2, 2, 2), 'float32')
    for o in range(2):
        for i in range(2):
            for j in range(2):
                ref[0, o, i, j] = (x[0, 0, i:i + 2, j:j + 2] * w[o, 0]).sum() + b[o]
    assert_almost_equal(c(nd.array(x)).asnumpy(), ref, rtol=1e-5, atol=1e-5)


def test_batchnorm_layernorm_statistics():
    bn = nn.BatchNorm(in_channels=3)
    bn.initialize()
    x = nd.array(np.random.randn(8, 3, 4, 4) * 2 + 1)
    with autograd.record():
        y = bn(x)
    yn = y.asnumpy()
    assert_almost_equal(yn.mean((0, 2, 3)), np.zeros(3), atol=1e-5)
    assert_almost_equal(yn.var((0, 2, 3)), np.ones(3), rtol=1e-3, atol=1e-3)
    xn = x.asnumpy()
    assert_almost_equal(bn.running_mean.data().asnumpy(), 0.1 * xn.mean((0, 2, 3)), rtol=1e-4, atol=1e-5)
    assert_almost_equal(bn.running_var.data().asnumpy(), 0.9 + 0.1 * xn.var((0, 2, 3)), rtol=1e-4, atol=1e-5)
    y2 = bn(x)      # inference: running statistics
    ref = (xn - bn.running_mean.data().asnumpy().reshape(1, 3, 1, 1)) / np.sqrt(
        bn.running_var.data().asnumpy().reshape(1, 3, 1, 1) + 1e-5)
    assert_almost_equal(y2.asnumpy(), ref, rtol=1e-4, atol=1e-4)
    ln = nn.LayerNorm(in_channels=5)
    ln.initialize()
    z = ln(nd.array(np.random.randn(4, 5))).asnumpy()
    assert_almost_equal(z.mean(-1), np.zeros(4), atol=1e-5)
    gn = nn.GroupNorm(num_groups=2, in_channels=4)
    gn.initialize()
    assert gn(nd.ones((2, 4, 3, 3))).shape == (2, 4, 3, 3)
    inn = nn.InstanceNorm(in_channels=4)
    inn.initialize()
    assert inn(nd.array(np.random.randn(2, 4, 3, 3))).shape == (2, 4, 3, 3)


def test_embedding_dropout_activations():
    emb = nn.Embedding(10, 4)
    emb.initialize()
    idx = nd.array([[1, 2], [3, 9]])
    out = emb(idx)
    assert out.shape == (2, 2, 4) and same(out[1, 1].asnumpy(), emb.weight.data()[9].asnumpy())
    with autograd.record():
        loss = emb(idx).sum()
    loss.backward()
    g = emb.weight.grad().asnumpy()
    assert g[1].sum() == 4 and g[0].sum() == 0
    x = nd.array([-2., -0.5, 0., 1.])
    assert same(nn.Activation('relu')(x).asnumpy(), np.array([0, 0, 0, 1], 'float32'))
    assert_almost_equal(nn.LeakyReLU(0.1)(x).asnumpy(), np.array([-0.2, -0.05, 0, 1]), rtol=1e-6)
    assert_almost_equal(nn.ELU(1.0)(x).asnumpy(), np.where(x.asnumpy() > 0, x.asnumpy(), np.exp(x.asnumpy()) - 1), rtol=1e-5)
    assert_almost_equal(nn.Swish()(x).asnumpy(), x.asnumpy() / (1 + np.exp(-x.asnumpy())), rtol=1e-5)
    from math import erf
    assert_almost_equal(nn.GELU()(x).asnumpy(), np.array([0.5 * v * (1 + erf(v / np.sqrt(2))) for v in x.asnumpy()]),
                        rtol=1e-4, atol=1e-6)
    pr = nn.PReLU()
    pr.initialize()
    assert_almost_equal(pr(x).asnumpy(), np.array([-0.5, -0.125, 0, 1]), rtol=1e-6)


def test_sequential_indexing_and_nested_blocks():
    net = nn.Sequential()
    net.add(nn.Dense(4, in_units=3), nn.Dense(5, in_units=4), nn.Dense(6, in_units=5))
    assert len(net) == 3 and isinstance(net[1], nn.Dense) and len(net[1:]) == 2
    net.initialize()
    assert net(nd.ones((2, 3))).shape == (2, 6)
    seen = []
    net.apply(lambda b: seen.append(type(b).__name__))
    assert seen.count('Dense') == 3
    s = repr(net)
    assert 'Dense(3 -> 4' in s


def _mlp():
    net = nn.HybridSequential()
    net.add(nn.Dense(16, activation='relu', in_units=8), nn.BatchNorm(in_channels=16), nn.Dropout(0.0),
            nn.Dense(4, in_units=16))
    return net


def test_hybridize_matches_imperative_and_caches():
    net = _mlp()
    net.initialize()
    x = nd.array(np.random.randn(5, 8))
    ref = net(x).asnumpy()
    net.hybridize()
    assert_almost_equal(net(x).asnumpy(), ref, rtol=1e-6)
    assert_almost_equal(net(x).asnumpy(), ref, rtol=1e-6)
    x.attach_grad()
    with autograd.record():
        y = net(x).sum()
    y.backward()
    assert x.grad.shape == (5, 8) and float(abs(x.grad).sum().asscalar()) > 0


def test_export_and_symbolblock_imports(tmp_path):
    net = _mlp()
    net.initialize()
    net.hybridize()
    x = nd.array(np.random.randn(3, 8))
    ref = net(x).asnumpy()
    prefix = str(tmp_path / 'model')
    sym_file, params_file = net.export(prefix, epoch=7)
    assert os.path.basename(sym_file) == 'model-symbol.json' and os.path.basename(params_file) == 'model-0007.params'
    graph = json.load(open(sym_file))
    assert set(graph) >= {'nodes', 'arg_nodes', 'heads', 'attrs'}
    ops = [n['op'] for n in graph['nodes']]
    assert 'FullyConnected' in ops and 'BatchNorm' in ops and ops.count('null') >= 9
    fc = [n for n in graph['nodes'] if n['op'] == 'FullyConnected'][0]
    assert fc['attrs']['num_hidden'] == '16' and fc['attrs']['no_bias'] == 'False'
    saved = nd.load(params_file)
    assert any(k.endswith('running_mean') for k in saved)
    net2 = gluon.SymbolBlock.imports(sym_file, ['data'], params_file)
    assert_almost_equal(net2(x).asnumpy(), ref, rtol=1e-5, atol=1e-6)


def test_save_load_parameters(tmp_path):
    net = _mlp()
    net.initialize()
    f = str(tmp_path / 'net.params')
    net.save_parameters(f)
    net2 = _mlp()
    net2.load_parameters(f)
    x = nd.array(np.random.randn(3, 8))
    assert_almost_equal(net2(x).asnumpy(), net(x).asnumpy(), rtol=1e-6)
    net3 = nn.HybridSequential()
    net3.add(nn.Dense(16, in_units=8))
    with pytest.raises(Exception):
        net3.load_parameters(f)
    net3.load_parameters(f, ignore_extra=True, allow_missing=True)


def test_parameter_sharing():
    a = nn.Dense(4, in_units=4)
    b = nn.Dense(4, in_units=4)
    b.share_parameters(a.collect_params())
    a.initialize()
    x = nd.ones((1, 4))
    assert same(a(x).asnumpy(), b(x).asnumpy())
    assert b.weight is a.weight


def test_trainer_sgd_step_matches_formula():
    net = nn.Dense(2, in_units=3, use_bias=False)
    net.initialize(mx.init.Constant(0.5))
    tr = gluon.Trainer(net.collect_params(), 'sgd', {'learning_rate': 0.1, 'wd': 0.01, 'momentum': 0.9})
    x = nd.array([[1., 2., 3.], [4., 5., 6.]])
    w = np.full((2, 3), 0.5, 'float32')
    m = np.zeros_like(w)
    for _ in range(3):
        with autograd.record():
            loss = net(x).sum()
        loss.backward()
        tr.step(2)
        g = np.tile(x.asnumpy().sum(0), (2, 1)) / 2 + 0.01 * w
        m = 0.9 * m - 0.1 * g
        w = w + m
        assert_almost_equal(net.weight.data().asnumpy(), w, rtol=1e-5, atol=1e-6)
    assert tr.learning_rate == 0.1
    tr.set_learning_rate(0.5)
    assert tr.optimizer.learning_rate == 0.5


def test_trainer_multi_device_and_states(tmp_path):
    ctxs = [mx.cpu(0), mx.cpu(1)]
    net = nn.Dense(2, in_units=3)
    net.initialize(ctx=ctxs)
    tr = gluon.Trainer(net.collect_params(), 'adam', {'learning_rate': 0.01}, kvstore='device')
    xs = gluon.utils.split_and_load(nd.array(np.random.randn(4, 3)), ctxs)
    with autograd.record():
        losses = [net(x).sum() for x in xs]
    autograd.backward(losses)
    tr.step(4)
    w0, w1 = net.weight.data(ctxs[0]).asnumpy(), net.weight.data(ctxs[1]).asnumpy()
    assert same(w0, w1)
    f = str(tmp_path / 'tr.states')
    tr.save_states(f)
    tr.load_states(f)
    with autograd.record():
        losses = [net(x).sum() for x in xs]
    autograd.backward(losses)
    tr.step(4)
    assert same(net.weight.data(ctxs[0]).asnumpy(), net.weight.data(ctxs[1]).asnumpy())


def test_trainer_allreduce_then_update_and_stale_grad():
    net = nn.Dense(2, in_units=3)
    net.initialize(ctx=[mx.cpu(0), mx.cpu(1)])
    tr = gluon.Trainer(net.collect_params(), 'sgd', {'learning_rate': 1.0}, kvstore='device', update_on_kvstore=False)
    xs = [nd.ones((1, 3), ctx=mx.cpu(0)), nd.ones((1, 3), ctx=mx.cpu(1)) * 2]
    before = net.weight.data(mx.cpu(0)).asnumpy().copy()
    with autograd.record():
        losses = [net(x).sum() for x in xs]
    autograd.backward(losses)
    tr.allreduce_grads()
    assert same(net.weight.grad(mx.cpu(0)).asnumpy(), np.full((2, 3), 3.0, 'float32'))
    tr.update(1)
    assert_almost_equal(net.weight.data(mx.cpu(1)).asnumpy(), before - 3.0, rtol=1e-6)
    with pytest.raises(UserWarning):
        tr.step(1)          # gradients were not refreshed since the last update
    tr.step(1, ignore_stale_grad=True)


def test_clip_global_norm_and_split_data():
    arrs = [nd.ones((2, 2)) * 3, nd.ones((3,)) * 4]
    total = np.sqrt(4 * 9 + 3 * 16)
    norm = gluon.utils.clip_global_norm(arrs, 1.0)
    assert abs(float(norm) - total) < 1e-4
    assert_almost_equal(arrs[0].asnumpy(), np.full((2, 2), 3 / (total + 1e-8), 'float32'), rtol=1e-5)
    parts = gluon.utils.split_data(nd.arange(12).reshape((6, 2)), 3)
    assert [p.shape for p in parts] == [(2, 2)] * 3
    with pytest.raises(ValueError):
        gluon.utils.split_data(nd.ones((5, 2)), 3)


def test_block_hooks_summary_and_cast(capsys):
    net = _mlp()
    net.initialize()
    calls = []
    h1 = net.register_forward_pre_hook(lambda blk, args: calls.append('pre'))
    h2 = net.register_forward_hook(lambda blk, args, out: calls.append('post'))
    net(nd.ones((2, 8)))
    assert calls == ['pre', 'post']
    h1.detach()
    h2.detach()
    net(nd.ones((2, 8)))
    assert calls == ['pre', 'post']
    net.summary(nd.ones((2, 8)))
    out = capsys.readouterr().out
    assert 'Dense' in out and 'Total params' in out
    net.cast('float64')
    assert net[0].weight.data().dtype == np.float64
    assert net(nd.ones((2, 8), dtype='float64')).dtype == np.float64


def test_zero_grad_and_lr_mult():
    net = nn.Dense(2, in_units=2, use_bias=False)
    net.initialize(mx.init.One())
    net.weight.lr_mult = 0.0
    tr = gluon.Trainer(net.collect_params(), 'sgd', {'learning_rate': 1.0})
    with autograd.record():
        l = net(nd.ones((1, 2))).sum()
    l.backward()
    tr.step(1)
    assert same(net.weight.data().asnumpy(), np.ones((2, 2), 'float32'))
    net.zero_grad()
    assert float(net.weight.grad().sum().asscalar()) == 0

"""Automatic mixed precision on the CPU path: cast policy, loss scaling, overflow skip (reference:
tests/python/gpu/test_amp.py, test_amp_init.py; python/mxnet/amp/loss_scaler.py)."""
import numpy as np
import pytest

import mxnet_b200 as mx
from mxnet_b200 import amp, autograd, gluon, nd
from mxnet_b200.gluon import nn


@pytest.fixture
def amp_bf16():
    amp._reset()
    amp.init('bfloat16')
    yield
    amp._reset()


def test_cast_policy(amp_bf16):
    x = nd.array(np.random.randn(4, 8))
    w = nd.array(np.random.randn(6, 8))
    y = nd.FullyConnected(x, w, num_hidden=6, no_bias=True)
    assert str(y.dtype) == 'bfloat16'                       # matmul-type ops run in the low precision type
    z = nd.exp(y)
    assert z.dtype == np.float32                            # exponentials are forced back to fp32
    s = nd.broadcast_add(y, nd.ones((4, 6)))                # widest type wins
    assert s.dtype == np.float32
    r = nd.relu(y)
    assert str(r.dtype) == 'bfloat16'                       # type-agnostic ops keep what arrives


def test_op_lists_are_consistent():
    lp16 = set(amp.list_lp16_ops('float16'))
    fp32 = set(amp.list_fp32_ops('float16'))
    assert 'FullyConnected' in lp16 and 'Convolution' in lp16 and 'exp' in fp32 and 'norm' in fp32
    assert not (lp16 & fp32)
    assert 'broadcast_add' in amp.list_widest_type_cast('float16')
    assert ('Activation', 'act_type', ['softrelu']) in amp.list_conditional_fp32_ops('float16')


def test_init_trainer_required_and_scale_loss(amp_bf16):
    net = nn.Dense(2, in_units=3)
    net.initialize()
    trainer = gluon.Trainer(net.collect_params(), 'sgd', {'learning_rate': 0.1})
    with pytest.raises(Exception):
        with amp.scale_loss(nd.ones((1,)), trainer):
            pass
    amp.init_trainer(trainer)
    x = nd.ones((2, 3))
    with autograd.record():
        loss = net(x).sum()
        with amp.scale_loss(loss, trainer) as scaled:
            autograd.backward(scaled)
    before = net.weight.data().asnumpy().copy()
    trainer.step(1)
    after = net.weight.data().asnumpy()
    # bf16 runs with loss scale 1: plain SGD on dloss/dw = sum over the batch of x
    np.testing.assert_allclose(after, before - 0.1 * 2.0, rtol=2e-2, atol=2e-2)


def test_dynamic_loss_scaler_halves_and_skips_then_grows():
    amp._reset()
    amp.init('float16')
    try:
        net = nn.Dense(2, in_units=3)
        net.initialize()
        trainer = gluon.Trainer(net.collect_params(), 'sgd', {'learning_rate': 0.1})
        amp.init_trainer(trainer)
        scaler = trainer._amp_loss_scaler
        scaler._scale_seq_len = 2
        assert scaler.loss_scale == 2. ** 16
        x = nd.ones((2, 3))
        with autograd.record():
            loss = (net(x) * 1e-3).sum()                    # small enough that the scaled gradients fit fp16
            with amp.scale_loss(loss, trainer) as scaled:
                autograd.backward(scaled)
        net.weight.grad()[:] = float('inf')                 # overflow injected on the host
        before = net.weight.data().asnumpy().copy()
        trainer.step(1)
        assert np.array_equal(net.weight.data().asnumpy(), before), 'the update must be skipped'
        assert scaler.loss_scale == 2. ** 15
        for _ in range(2):                                   # two clean steps double the scale again
            with autograd.record():
                loss = (net(x) * 1e-3).sum()
                with amp.scale_loss(loss, trainer) as scaled:
                    autograd.backward(scaled)
            trainer.step(1)
        assert scaler.loss_scale == 2. ** 16
        assert not np.array_equal(net.weight.data().asnumpy(), before)
    finally:
        amp._reset()


def test_unscale_divides_gradients():
    amp._reset()
    amp.init('float16')
    try:
        net = nn.Dense(1, in_units=2, use_bias=False)
        net.initialize(mx.init.One())
        trainer = gluon.Trainer(net.collect_params(), 'sgd', {'learning_rate': 0.1})
        amp.init_trainer(trainer)
        x = nd.array([[1., 2.]])
        with autograd.record():
            loss = (net(x).astype('float32') * 1e-3).sum()     # losses are fp32 under AMP (the scale itself exceeds fp16)
            with amp.scale_loss(loss, trainer) as scaled:
                autograd.backward(scaled)
        g_scaled = net.weight.grad().asnumpy().copy()
        amp.unscale(trainer)
        np.testing.assert_allclose(net.weight.grad().asnumpy(), g_scaled / 2. ** 16, rtol=1e-3)
        np.testing.assert_allclose(net.weight.grad().asnumpy(), [[1e-3, 2e-3]], rtol=1e-2)
    finally:
        amp._reset()


def test_convert_hybrid_block_and_symbol():
    net = nn.HybridSequential()
    net.add(nn.Dense(8, activation='relu', in_units=4), nn.Dense(2, in_units=8))
    net.initialize()
    x = nd.array(np.random.randn(3, 4))
    ref = net(x).asnumpy()
    lp = amp.convert_hybrid_block(net, data_example=x, target_dtype='bfloat16')
    out = lp(x)
    np.testing.assert_allclose(out.asnumpy().astype('float32'), ref, rtol=5e-2, atol=5e-2)
    data = mx.sym.Variable('data')
    sym = mx.sym.FullyConnected(data, num_hidden=4, name='fc')
    sym = mx.sym.softmax(sym, name='sm')
    conv = amp.convert_symbol(sym, target_dtype='float16')
    ops = [n['op'] for n in __import__('json').loads(conv.tojson())['nodes']]
    assert 'amp_cast' in ops


def test_opt_constraint_scope_switches_amp_casts_off():
    """HybridBlock.OptConstraint.disable_amp(): inside the scope operators see their inputs uncast."""
    from mxnet_b200 import _state
    seen = []
    prev = _state.amp_hook
    _state.amp_hook = lambda name, tensors: (seen.append(name), tensors)[1]
    try:
        a = mx.nd.ones((2, 2))
        (a + a).wait_to_read()
        n = len(seen)
        assert n >= 1
        with mx.gluon.HybridBlock.OptConstraint.disable_amp():
            (a * a).wait_to_read()
            s = mx.sym.relu(mx.sym.var('x'))
            s._bind(mx.cpu(), {'x': a}).forward()
        assert len(seen) == n
        (a - a).wait_to_read()
        assert len(seen) == n + 1
    finally:
        _state.amp_hook = prev

"""Autograd semantics (reference: tests/python/unittest/test_autograd.py): recording scopes, grad_req,
head gradients, retain_graph, autograd.grad, custom Function, higher order."""
import numpy as np
import pytest

import mxnet_b200 as mx
from mxnet_b200 import autograd, nd
from mxnet_b200.test_utils import assert_almost_equal, same


def test_recording_and_training_flags():
    assert not autograd.is_recording() and not autograd.is_training()
    with autograd.record():
        assert autograd.is_recording() and autograd.is_training()
        with autograd.pause():
            assert not autograd.is_recording() and not autograd.is_training()
        with autograd.predict_mode():
            assert autograd.is_recording() and not autograd.is_training()
    with autograd.record(train_mode=False):
        assert autograd.is_recording() and not autograd.is_training()
        with autograd.train_mode():
            assert autograd.is_training()
    assert not autograd.is_recording()
    prev = autograd.set_recording(True)
    assert prev is False and autograd.is_recording()
    autograd.set_recording(False)


def test_simple_backward_and_head_grads():
    x = nd.array([1., 2., 3.])
    x.attach_grad()
    with autograd.record():
        y = x * x + 2 * x
    y.backward()
    assert_almost_equal(x.grad.asnumpy(), 2 * x.asnumpy() + 2)
    with autograd.record():
        y = x * x
    y.backward(nd.array([1., 0.5, 0.]))
    assert_almost_equal(x.grad.asnumpy(), np.array([2., 2., 0.]))


def test_grad_req_add_write_null():
    x = nd.array([1., 2.])
    x.attach_grad(grad_req='add')
    for _ in range(3):
        with autograd.record():
            y = 3 * x
        y.backward()
    assert same(x.grad.asnumpy(), np.array([9., 9.], 'float32'))
    x.grad[:] = 0
    x.attach_grad(grad_req='write')
    for _ in range(3):
        with autograd.record():
            y = 3 * x
        y.backward()
    assert same(x.grad.asnumpy(), np.array([3., 3.], 'float32'))
    z = nd.array([1.])
    z.attach_grad(grad_req='null')
    with autograd.record():
        y = (x * z).sum()
    y.backward()
    assert float(z.grad.asscalar()) == 0 if z.grad is not None else True


def test_write_accumulates_within_one_pass():
    """A leaf used twice in one graph receives the sum of both paths even with grad_req='write'."""
    x = nd.array([2.])
    x.attach_grad()
    with autograd.record():
        y = x * x + x * 3
    y.backward()
    assert float(x.grad.asscalar()) == 7.0


def test_retain_graph_and_double_backward_error():
    x = nd.array([1., 2.])
    x.attach_grad()
    with autograd.record():
        y = (x * x).sum()
    y.backward(retain_graph=True)
    y.backward()
    assert same(x.grad.asnumpy(), np.array([2., 4.], 'float32'))
    with pytest.raises(Exception):
        y.backward()


def test_autograd_grad_and_higher_order():
    x = nd.array([1., 2., 3.])
    x.attach_grad()
    with autograd.record():
        y = x * x * x
        gx = autograd.grad(y, [x], head_grads=nd.ones_like(y), create_graph=True, retain_graph=True)[0]
        z = gx.sum()
    assert_almost_equal(gx.asnumpy(), 3 * x.asnumpy() ** 2)
    z.backward()
    assert_almost_equal(x.grad.asnumpy(), 6 * x.asnumpy())


def test_detach_and_stop_gradient():
    x = nd.array([1., 2.])
    x.attach_grad()
    with autograd.record():
        y = x * 2
        z = y.detach() * x
    z.backward()
    assert same(x.grad.asnumpy(), np.array([2., 4.], 'float32'))
    with autograd.record():
        z = nd.BlockGrad(x * 2) * x
    z.backward()
    assert same(x.grad.asnumpy(), np.array([2., 4.], 'float32'))


def test_mark_variables_and_backward_list():
    a, b = nd.array([1., 2.]), nd.array([3., 4.])
    ga, gb = nd.zeros((2,)), nd.zeros((2,))
    autograd.mark_variables([a, b], [ga, gb])
    with autograd.record():
        y1, y2 = a * b, a + b
    autograd.backward([y1, y2])
    assert same(ga.asnumpy(), np.array([4., 5.], 'float32')) and same(gb.asnumpy(), np.array([2., 3.], 'float32'))


def test_custom_function():
    class Sigmoid(autograd.Function):
        def forward(self, x):
            y = 1 / (1 + nd.exp(-x))
            self.save_for_backward(y)
            return y

        def backward(self, dy):
            y, = self.saved_tensors
            return dy * y * (1 - y)

    x = nd.array([-1., 0., 2.])
    x.attach_grad()
    with autograd.record():
        y = Sigmoid()(x)
    y.backward()
    s = 1 / (1 + np.exp(-x.asnumpy()))
    assert_almost_equal(x.grad.asnumpy(), s * (1 - s), rtol=1e-5)


def test_training_flag_controls_dropout():
    x = nd.ones((100, 100))
    with autograd.record(train_mode=False):
        y = nd.Dropout(x, p=0.5)
    assert same(y.asnumpy(), x.asnumpy())
    with autograd.record(train_mode=True):
        y = nd.Dropout(x, p=0.5)
    frac = float((y == 0).sum().asscalar()) / 1e4
    assert 0.4 < frac < 0.6
    assert abs(float(y.mean().asscalar()) - 1.0) < 0.1        # inverted scaling keeps the expectation


def test_get_symbol_of_recorded_graph():
    x = nd.array([1., 2.])
    x.attach_grad()
    with autograd.record():
        y = nd.exp(x * 2)
    sym = autograd.get_symbol(y)
    assert 'exp' in sym.tojson()


def test_numpy_frontend_backward():
    from mxnet_b200 import np as mnp
    x = mnp.array([[1., 2.], [3., 4.]])
    x.attach_grad()
    with autograd.record():
        y = mnp.sum(mnp.dot(x, x))
    y.backward()
    xn = x.asnumpy()
    ref = np.ones((2, 2)) @ xn.T + xn.T @ np.ones((2, 2))
    assert_almost_equal(x.grad.asnumpy(), ref, rtol=1e-5)

"""mx.np / mx.npx front end against NumPy (reference: tests/python/unittest/test_numpy_op.py, test_numpy_ndarray.py)."""
import numpy as onp
import pytest

import mxnet_b200 as mx
from mxnet_b200 import autograd, np, npx
from mxnet_b200.test_utils import assert_almost_equal

rng = onp.random.RandomState(0)


def test_creation_and_dtypes():
    a = np.array([[1, 2], [3, 4]])
    assert a.shape == (2, 2) and a.dtype == onp.float32
    assert np.zeros((2, 3)).dtype == onp.float32 and np.ones((2,), dtype='int64').dtype == onp.int64
    assert np.arange(5).tolist() == [0, 1, 2, 3, 4]
    assert_almost_equal(np.linspace(0, 1, 5).asnumpy(), onp.linspace(0, 1, 5))
    assert np.eye(3).asnumpy().trace() == 3
    assert np.full((2, 2), 7).asnumpy().sum() == 28
    assert isinstance(a.asnumpy(), onp.ndarray) and a.item(0) == 1.0
    b = np.array(onp.arange(6).reshape(2, 3), dtype='float64')
    assert b.dtype == onp.float64 and b.T.shape == (3, 2) and b.size == 6 and b.ndim == 2


UNARY = ['abs', 'exp', 'log', 'sqrt', 'sin', 'cos', 'tanh', 'floor', 'ceil', 'sign', 'square', 'negative', 'reciprocal',
         'log1p', 'expm1', 'arctan', 'sinh', 'cosh', 'log2', 'log10', 'cbrt', 'trunc', 'rint']


@pytest.mark.parametrize('name', UNARY)
def test_unary(name):
    x = (rng.rand(3, 4) + 0.5).astype('float32')
    assert_almost_equal(getattr(np, name)(np.array(x)).asnumpy(), getattr(onp, name)(x), rtol=1e-5, atol=1e-6)


BINARY = ['add', 'subtract', 'multiply', 'divide', 'power', 'maximum', 'minimum', 'mod', 'arctan2', 'hypot', 'copysign']


@pytest.mark.parametrize('name', BINARY)
def test_binary_broadcast(name):
    x = (rng.rand(3, 1, 4) + 0.5).astype('float32')
    y = (rng.rand(2, 4) + 0.5).astype('float32')
    assert_almost_equal(getattr(np, name)(np.array(x), np.array(y)).asnumpy(), getattr(onp, name)(x, y), rtol=1e-5, atol=1e-6)


def test_reductions_and_statistics():
    x = rng.randn(3, 4, 5).astype('float32')
    a = np.array(x)
    for name in ('sum', 'mean', 'max', 'min', 'prod', 'std', 'var'):
        assert_almost_equal(getattr(np, name)(a, axis=1).asnumpy(), getattr(onp, name)(x, axis=1), rtol=1e-4, atol=1e-5)
    assert_almost_equal(np.sum(a, axis=(0, 2), keepdims=True).asnumpy(), x.sum((0, 2), keepdims=True), rtol=1e-5)
    assert np.argmax(a, axis=2).asnumpy().tolist() == x.argmax(2).tolist()
    assert_almost_equal(np.cumsum(a, axis=1).asnumpy(), x.cumsum(1), rtol=1e-5)
    assert_almost_equal(np.linalg.norm(a).asnumpy(), onp.linalg.norm(x), rtol=1e-5)
    assert_almost_equal(np.average(a, axis=0).asnumpy(), x.mean(0), rtol=1e-5)
    assert bool(np.all(a == a)) and not bool(np.any(a != a))


def test_shape_manipulation():
    x = onp.arange(24, dtype='float32').reshape(2, 3, 4)
    a = np.array(x)
    assert np.reshape(a, (4, 6)).shape == (4, 6) and a.reshape(-1, 4).shape == (6, 4)
    assert_almost_equal(np.transpose(a, (2, 0, 1)).asnumpy(), x.transpose(2, 0, 1))
    assert_almost_equal(np.concatenate([a, a], axis=1).asnumpy(), onp.concatenate([x, x], 1))
    assert_almost_equal(np.stack([a, a]).asnumpy(), onp.stack([x, x]))
    assert [p.shape for p in np.split(a, 2, axis=2)] == [(2, 3, 2)] * 2
    assert_almost_equal(np.swapaxes(a, 0, 2).asnumpy(), x.swapaxes(0, 2))
    assert_almost_equal(np.flip(a, 1).asnumpy(), onp.flip(x, 1))
    assert_almost_equal(np.tile(a, (1, 2, 1)).asnumpy(), onp.tile(x, (1, 2, 1)))
    assert_almost_equal(np.repeat(a, 2, axis=0).asnumpy(), onp.repeat(x, 2, 0))
    assert np.expand_dims(a, 0).shape == (1, 2, 3, 4) and np.squeeze(np.expand_dims(a, 0)).shape == (2, 3, 4)
    assert_almost_equal(np.where(a > 5, a, -a).asnumpy(), onp.where(x > 5, x, -x))
    assert_almost_equal(np.clip(a, 3, 10).asnumpy(), onp.clip(x, 3, 10))
    assert_almost_equal(np.roll(a, 1, axis=2).asnumpy(), onp.roll(x, 1, 2))
    assert_almost_equal(np.moveaxis(a, 0, -1).asnumpy(), onp.moveaxis(x, 0, -1))
    assert_almost_equal(np.pad(a, ((0, 0), (1, 1), (2, 0))).asnumpy(), onp.pad(x, ((0, 0), (1, 1), (2, 0))))
    assert_almost_equal(np.tril(np.array(x[0])).asnumpy(), onp.tril(x[0]))


def test_linear_algebra():
    a, b = rng.randn(4, 5).astype('float32'), rng.randn(5, 3).astype('float32')
    assert_almost_equal(np.dot(np.array(a), np.array(b)).asnumpy(), a @ b, rtol=1e-4, atol=1e-5)
    assert_almost_equal(np.matmul(np.array(a), np.array(b)).asnumpy(), a @ b, rtol=1e-4, atol=1e-5)
    assert_almost_equal((np.array(a) @ np.array(b)).asnumpy(), a @ b, rtol=1e-4, atol=1e-5)
    assert_almost_equal(np.einsum('ij,jk->ik', np.array(a), np.array(b)).asnumpy(), a @ b, rtol=1e-4, atol=1e-5)
    assert_almost_equal(np.tensordot(np.array(a), np.array(b), axes=1).asnumpy(), a @ b, rtol=1e-4, atol=1e-5)
    s = rng.randn(4, 4).astype('float32')
    spd = s @ s.T + 4 * onp.eye(4, dtype='float32')
    assert_almost_equal(np.linalg.inv(np.array(spd)).asnumpy(), onp.linalg.inv(spd), rtol=1e-3, atol=1e-4)
    assert_almost_equal(np.linalg.cholesky(np.array(spd)).asnumpy(), onp.linalg.cholesky(spd), rtol=1e-3, atol=1e-4)
    assert_almost_equal(np.linalg.det(np.array(spd)).asnumpy(), onp.linalg.det(spd), rtol=1e-3)
    u, sv, vt = np.linalg.svd(np.array(a))
    assert_almost_equal(sv.asnumpy(), onp.linalg.svd(a, compute_uv=False), rtol=1e-3, atol=1e-4)
    w = np.linalg.eigvalsh(np.array(spd)).asnumpy()
    assert_almost_equal(w, onp.linalg.eigvalsh(spd), rtol=1e-3, atol=1e-4)
    assert_almost_equal(np.linalg.solve(np.array(spd), np.array(s)).asnumpy(), onp.linalg.solve(spd, s), rtol=1e-3, atol=1e-4)


def test_indexing_and_assignment():
    x = onp.arange(24, dtype='float32').reshape(4, 6)
    a = np.array(x)
    assert_almost_equal(a[1:3, ::2].asnumpy(), x[1:3, ::2])
    assert_almost_equal(a[[0, 3]].asnumpy(), x[[0, 3]])
    assert_almost_equal(a[a > 10].asnumpy(), x[x > 10])
    assert_almost_equal(a[np.array([0, 2], dtype='int64'), np.array([1, 5], dtype='int64')].asnumpy(), x[[0, 2], [1, 5]])
    a[0, :] = 9
    x[0, :] = 9
    a[a < 9] = 0
    x[x < 9] = 0
    assert_almost_equal(a.asnumpy(), x)
    assert_almost_equal(a[..., None].shape, x[..., None].shape)
    assert_almost_equal(np.take(a, np.array([1, 3], dtype='int64'), axis=1).asnumpy(), x[:, [1, 3]])


def test_autograd_through_numpy_ops():
    x = np.array(rng.randn(3, 4).astype('float32'))
    x.attach_grad()
    with autograd.record():
        y = np.sum(np.tanh(x) * np.exp(-x * x))
    y.backward()
    xn = x.asnumpy().astype('float64')
    ref = (1 - onp.tanh(xn) ** 2) * onp.exp(-xn * xn) + onp.tanh(xn) * onp.exp(-xn * xn) * (-2 * xn)
    assert_almost_equal(x.grad.asnumpy(), ref.astype('float32'), rtol=1e-4, atol=1e-5)


def test_npx_ops_and_np_mode():
    x = np.array(rng.randn(2, 5).astype('float32'))
    sm = npx.softmax(x, axis=-1).asnumpy()
    assert_almost_equal(sm.sum(-1), onp.ones(2), rtol=1e-5)
    assert_almost_equal(npx.relu(x).asnumpy(), onp.maximum(x.asnumpy(), 0))
    assert_almost_equal(npx.sigmoid(x).asnumpy(), 1 / (1 + onp.exp(-x.asnumpy())), rtol=1e-5)
    oh = npx.one_hot(np.array([0, 2], dtype='int64'), 3).asnumpy()
    assert oh.tolist() == [[1, 0, 0], [0, 0, 1]]
    w, b = np.array(rng.randn(3, 5).astype('float32')), np.zeros((3,))
    fc = npx.fully_connected(x, w, b, num_hidden=3)
    assert_almost_equal(fc.asnumpy(), x.asnumpy() @ w.asnumpy().T, rtol=1e-4, atol=1e-5)
    assert npx.is_np_array() in (True, False)
    with mx.util.np_array(True), mx.util.np_shape(True):
        assert npx.is_np_array() and npx.is_np_shape()
    assert type(x.as_nd_ndarray()).__name__ == 'NDArray' and type(x.as_nd_ndarray().as_np_ndarray()).__name__ == 'ndarray'


def test_random_module():
    mx.random.seed(3)
    u = np.random.uniform(0, 2, size=(5000,)).asnumpy()
    assert abs(u.mean() - 1) < 0.05
    n = np.random.normal(1, 2, size=(5000,)).asnumpy()
    assert abs(n.mean() - 1) < 0.1 and abs(n.std() - 2) < 0.1
    assert np.random.randint(0, 3, size=(100,)).asnumpy().max() <= 2
    c = np.random.choice(5, size=(50,)).asnumpy()
    assert c.min() >= 0 and c.max() <= 4
    p = np.random.permutation(10).asnumpy()
    assert sorted(p.tolist()) == list(range(10))
    g = np.random.gamma(2.0, 1.0, size=(5000,)).asnumpy()
    assert abs(g.mean() - 2) < 0.15


def test_array_api_names_and_linalg_additions():
    """pow / atan2 / asin ... / concat / permute_dims / bitwise_* / from_dlpack and the array-API part of np.linalg."""
    import torch
    np_ = mx.np
    a = np_.array([[1., 2., 3.], [4., 5., 6.]])
    b = np_.array([[1., 0., 2.], [0., 3., 1.]])
    an, bn = a.asnumpy(), b.asnumpy()
    onp.testing.assert_allclose(np_.pow(a, 2).asnumpy(), an ** 2)
    onp.testing.assert_allclose(np_.atan2(a, b).asnumpy(), onp.arctan2(an, bn), rtol=1e-6)
    for new, old in (('asin', 'arcsin'), ('acos', 'arccos'), ('atan', 'arctan'), ('asinh', 'arcsinh'), ('atanh', 'arctanh')):
        v = np_.array([0.1, 0.5])
        onp.testing.assert_allclose(getattr(np_, new)(v).asnumpy(), getattr(onp, old)(v.asnumpy()), rtol=1e-6)
    onp.testing.assert_allclose(np_.acosh(a).asnumpy(), onp.arccosh(an), rtol=1e-6)
    assert np_.concat([a, b], axis=None).shape == (12,) and np_.concat([a, b], axis=1).shape == (2, 6)
    assert np_.permute_dims(a, (1, 0)).shape == (3, 2)
    i = np_.array([1, 2], dtype='int32')
    onp.testing.assert_array_equal(np_.bitwise_invert(i).asnumpy(), [-2, -3])
    onp.testing.assert_array_equal(np_.bitwise_left_shift(i, i).asnumpy(), [2, 8])
    onp.testing.assert_array_equal(np_.bitwise_right_shift(np_.array([8, 8], dtype='int32'), i).asnumpy(), [4, 2])
    t = torch.arange(4.)
    shared = np_.from_dlpack(t)
    t[0] = 9
    onp.testing.assert_array_equal(shared.asnumpy(), [9, 1, 2, 3])           # same memory
    L = np_.linalg
    onp.testing.assert_allclose(L.vecdot(a, b).asnumpy(), (an * bn).sum(-1))
    onp.testing.assert_allclose(L.vector_norm(a).asnumpy(), onp.linalg.norm(an.ravel()), rtol=1e-6)
    onp.testing.assert_allclose(L.vector_norm(a, axis=1, ord=1).asnumpy(), onp.abs(an).sum(1))
    assert L.vector_norm(a, axis=(0, 1), keepdims=True).shape == (1, 1)
    onp.testing.assert_allclose(L.matrix_norm(a).asnumpy(), onp.linalg.norm(an), rtol=1e-6)
    onp.testing.assert_allclose(L.svdvals(a).asnumpy(), onp.linalg.svd(an)[1], rtol=1e-5)
    onp.testing.assert_allclose(L.cross(a, b).asnumpy(), onp.cross(an, bn))
    onp.testing.assert_allclose(L.tensordot(a, np_.transpose(b), 1).asnumpy(), an @ bn.T)
    assert L.matrix_transpose(a).shape == (3, 2) and L.outer(a[0], b[0]).shape == (3, 3)
    onp.testing.assert_allclose(L.diagonal(a).asnumpy(), [1, 5])
    onp.testing.assert_allclose(L.trace(np_.array([[1., 2.], [3., 4.]])).asnumpy(), 5)

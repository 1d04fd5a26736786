"""NDArray front end: creation, arithmetic, indexing, views, serialisation (mirrors the reference's
tests/python/unittest/test_ndarray.py in scope, with NumPy as the oracle)."""
import os
import struct

import numpy as np
import pytest

import mxnet_b200 as mx
from mxnet_b200 import nd
from mxnet_b200.test_utils import assert_almost_equal, same


def test_creation_and_basic_properties():
    a = nd.array([[1, 2, 3], [4, 5, 6]])
    assert a.shape == (2, 3) and a.dtype == np.float32 and a.size == 6 and a.ndim == 2
    assert a.context == mx.cpu()
    assert same(a.asnumpy(), np.array([[1, 2, 3], [4, 5, 6]], dtype='float32'))
    assert same(nd.zeros((2, 2)).asnumpy(), np.zeros((2, 2), 'float32'))
    assert same(nd.ones((3,), dtype='int32').asnumpy(), np.ones((3,), 'int32'))
    assert same(nd.full((2,), 7).asnumpy(), np.full((2,), 7, 'float32'))
    assert same(nd.arange(0, 10, 2).asnumpy(), np.arange(0, 10, 2, dtype='float32'))
    assert nd.array(np.arange(4, dtype='float64')).dtype == np.float32          # non-NDArray sources default to float32
    assert nd.array(np.arange(4), dtype='float64').dtype == np.float64
    assert nd.array([1, 2]).astype('float16').dtype == np.float16
    e = nd.empty((2, 3))
    assert e.shape == (2, 3)


def test_arithmetic_matches_numpy():
    rng = np.random.RandomState(0)
    x, y = rng.randn(3, 4).astype('float32'), rng.rand(3, 4).astype('float32') + 0.5
    a, b = nd.array(x), nd.array(y)
    assert_almost_equal((a + b).asnumpy(), x + y)
    assert_almost_equal((a - b).asnumpy(), x - y)
    assert_almost_equal((a * b).asnumpy(), x * y)
    assert_almost_equal((a / b).asnumpy(), x / y, rtol=1e-5)
    assert_almost_equal((a ** 2).asnumpy(), x ** 2, rtol=1e-5)
    assert_almost_equal((2 - a).asnumpy(), 2 - x)
    assert_almost_equal((2 / b).asnumpy(), 2 / y, rtol=1e-5)
    assert_almost_equal((-a).asnumpy(), -x)
    assert_almost_equal(abs(a).asnumpy(), np.abs(x))
    assert same((a > b).asnumpy(), (x > y).astype('float32'))
    assert same((a == a).asnumpy(), np.ones_like(x))
    assert_almost_equal((a % 0.7).asnumpy(), np.mod(x, 0.7), rtol=1e-4, atol=1e-5)


def test_inplace_ops_keep_identity():
    a = nd.ones((2, 3))
    ida = id(a)
    a += 1
    a *= 3
    a -= 2
    a /= 2
    assert id(a) == ida
    assert same(a.asnumpy(), np.full((2, 3), 2.0, 'float32'))


def test_broadcasting():
    x, y = np.arange(6, dtype='float32').reshape(2, 3, 1), np.arange(4, dtype='float32').reshape(1, 1, 4)
    assert same(nd.broadcast_add(nd.array(x), nd.array(y)).asnumpy(), x + y)
    assert same(nd.broadcast_to(nd.array(y), shape=(2, 3, 4)).asnumpy(), np.broadcast_to(y, (2, 3, 4)))
    assert same(nd.array(y).broadcast_axes(axis=0, size=3).asnumpy(), np.broadcast_to(y, (3, 1, 4)))


def test_indexing_and_assignment():
    x = np.arange(24, dtype='float32').reshape(2, 3, 4)
    a = nd.array(x)
    assert same(a[1].asnumpy(), x[1])
    assert same(a[:, 1:3].asnumpy(), x[:, 1:3])
    assert same(a[1, 2, 3].asnumpy(), x[1, 2, 3])
    assert same(a[:, :, ::2].asnumpy(), x[:, :, ::2])
    assert same(a[nd.array([1, 0], dtype='int64')].asnumpy(), x[[1, 0]])
    a[0] = 5
    x[0] = 5
    a[1, 1:3, 0] = nd.array([7, 8])
    x[1, 1:3, 0] = [7, 8]
    a[:, 0, 1] = np.array([1., 2.])
    x[:, 0, 1] = [1., 2.]
    assert same(a.asnumpy(), x)
    a[:] = 0
    assert float(a.sum().asscalar()) == 0


def test_slice_is_a_view_that_writes_through():
    a = nd.zeros((4, 3))
    s = a[1:3]
    s[:] = 2
    assert float(a.sum().asscalar()) == 12


def test_reshape_special_codes():
    a = nd.zeros((2, 3, 4))
    assert a.reshape((-1,)).shape == (24,)
    assert a.reshape((0, -1)).shape == (2, 12)
    assert a.reshape((-2,)).shape == (2, 3, 4)
    assert a.reshape((-3, 4)).shape == (6, 4)
    assert a.reshape((-4, 1, 2, -2)).shape == (1, 2, 3, 4)
    assert a.reshape((0, 0, -1)).shape == (2, 3, 4)
    assert a.reshape(6, 4).shape == (6, 4)
    assert nd.reshape(a, shape=(4, 0, -1), reverse=False).shape[0] == 4


def test_reductions_and_shape_ops():
    x = np.random.RandomState(1).randn(3, 4, 5).astype('float32')
    a = nd.array(x)
    assert_almost_equal(a.sum(axis=1).asnumpy(), x.sum(1), rtol=1e-5)
    assert_almost_equal(nd.sum(a, axis=(0, 2), keepdims=True).asnumpy(), x.sum((0, 2), keepdims=True), rtol=1e-5)
    assert_almost_equal(a.mean().asnumpy(), x.mean(), rtol=1e-5)
    assert_almost_equal(nd.max(a, axis=2).asnumpy(), x.max(2))
    assert_almost_equal(nd.norm(a).asnumpy(), np.linalg.norm(x.ravel()), rtol=1e-5)
    assert same(nd.argmax(a, axis=1).asnumpy(), x.argmax(1).astype('float32'))
    assert same(nd.transpose(a, axes=(2, 0, 1)).asnumpy(), x.transpose(2, 0, 1))
    assert same(a.T.asnumpy(), x.T)
    assert same(nd.swapaxes(a, dim1=0, dim2=2).asnumpy(), x.swapaxes(0, 2))
    assert same(nd.expand_dims(a, axis=1).asnumpy(), x[:, None])
    assert same(nd.flip(a, axis=1).asnumpy(), x[:, ::-1])
    assert same(nd.tile(a, reps=(1, 2, 1)).asnumpy(), np.tile(x, (1, 2, 1)))
    assert same(nd.repeat(a, repeats=2, axis=0).asnumpy(), np.repeat(x, 2, 0))
    assert same(nd.concat(a, a, dim=1).asnumpy(), np.concatenate([x, x], 1))
    assert same(nd.stack(a, a, axis=0).asnumpy(), np.stack([x, x]))
    parts = nd.split(a, num_outputs=2, axis=1)
    assert len(parts) == 2 and same(parts[1].asnumpy(), x[:, 2:])
    assert same(nd.slice_axis(a, axis=2, begin=1, end=3).asnumpy(), x[:, :, 1:3])
    assert same(nd.slice(a, begin=(0, 1), end=(2, 3)).asnumpy(), x[0:2, 1:3])
    assert same(nd.clip(a, -0.5, 0.5).asnumpy(), np.clip(x, -0.5, 0.5))
    assert same(nd.where(a > 0, a, nd.zeros_like(a)).asnumpy(), np.where(x > 0, x, 0))


def test_dot_and_batch_dot():
    rng = np.random.RandomState(2)
    x, y = rng.randn(4, 5).astype('float32'), rng.randn(5, 3).astype('float32')
    assert_almost_equal(nd.dot(nd.array(x), nd.array(y)).asnumpy(), x @ y, rtol=1e-5, atol=1e-5)
    assert_almost_equal(nd.dot(nd.array(x), nd.array(y.T), transpose_b=True).asnumpy(), x @ y, rtol=1e-5, atol=1e-5)
    assert_almost_equal(nd.dot(nd.array(x.T), nd.array(y), transpose_a=True).asnumpy(), x @ y, rtol=1e-5, atol=1e-5)
    bx, by = rng.randn(2, 4, 5).astype('float32'), rng.randn(2, 5, 3).astype('float32')
    assert_almost_equal(nd.batch_dot(nd.array(bx), nd.array(by)).asnumpy(), bx @ by, rtol=1e-5, atol=1e-5)


def test_take_pick_onehot_topk_sort():
    x = np.random.RandomState(3).randn(5, 6).astype('float32')
    a = nd.array(x)
    idx = nd.array([0, 4, 2])
    assert same(nd.take(a, idx).asnumpy(), x[[0, 4, 2]])
    pk = nd.pick(a, nd.array([1, 0, 5, 2, 3]), axis=1)
    assert same(pk.asnumpy(), x[np.arange(5), [1, 0, 5, 2, 3]])
    assert same(nd.one_hot(nd.array([1, 3]), depth=4).asnumpy(), np.eye(4, dtype='float32')[[1, 3]])
    tk = nd.topk(a, k=2, axis=1, ret_typ='value')
    assert_almost_equal(tk.asnumpy(), -np.sort(-x, 1)[:, :2])
    assert same(nd.sort(a, axis=1).asnumpy(), np.sort(x, 1))
    assert same(nd.argsort(a, axis=1).asnumpy(), np.argsort(x, 1).astype('float32'))


def test_copy_and_context():
    a = nd.array([1, 2, 3])
    b = a.copy()
    b[:] = 0
    assert float(a.sum().asscalar()) == 6
    c = nd.zeros((3,))
    a.copyto(c)
    assert same(c.asnumpy(), a.asnumpy())
    d = a.as_in_context(mx.cpu(1))
    assert d.context == mx.cpu(1)
    assert a.as_in_context(mx.cpu(0)) is a


def test_save_load_roundtrip_list_and_dict(tmp_path):
    f = str(tmp_path / 'x.params')
    arrs = [nd.array(np.random.randn(3, 4).astype('float32')), nd.array(np.arange(5), dtype='int32'),
            nd.array(np.random.randn(2, 2).astype('float16'), dtype='float16'), nd.array(np.random.randn(7), dtype='float64')]
    nd.save(f, arrs)
    back = nd.load(f)
    assert isinstance(back, list) and len(back) == 4
    for a, b in zip(arrs, back):
        assert a.dtype == b.dtype and same(a.asnumpy(), b.asnumpy())
    d = {'arg:w': arrs[0], 'aux:m': arrs[1]}
    nd.save(f, d)
    back = nd.load(f)
    assert sorted(back) == ['arg:w', 'aux:m'] and same(back['arg:w'].asnumpy(), arrs[0].asnumpy())
    with open(f, 'rb') as fh:
        magic, reserved = struct.unpack('<QQ', fh.read(16))
    assert magic == 0x112 and reserved == 0


def test_load_hand_built_v2_file(tmp_path):
    """A file assembled byte by byte from the documented layout: list magic, count, then per array
    V2 magic 0xF993fac9, stype, ndim+dims (int64 for V2? no: uint32 ndim, int64 dims), ctx, type flag, raw data."""
    f = str(tmp_path / 'v2.params')
    data = np.arange(6, dtype='float32').reshape(2, 3)
    blob = struct.pack('<QQQ', 0x112, 0, 1)
    blob += struct.pack('<I', 0xF993FAC9) + struct.pack('<i', 0)            # magic, storage type dense
    blob += struct.pack('<I', 2) + struct.pack('<qq', 2, 3)                  # shape
    blob += struct.pack('<ii', 1, 0)                                         # context cpu(0)
    blob += struct.pack('<i', 0)                                             # type flag float32
    blob += data.tobytes()
    blob += struct.pack('<Q', 1) + struct.pack('<Q', 4) + b'name'
    with open(f, 'wb') as fh:
        fh.write(blob)
    back = nd.load(f)
    assert list(back) == ['name'] and same(back['name'].asnumpy(), data)


def test_sparse_roundtrip_and_ops(tmp_path):
    dense = np.zeros((6, 4), 'float32')
    dense[1] = [1, 0, 2, 0]
    dense[4] = [0, 3, 0, 4]
    rs = nd.array(dense).tostype('row_sparse')
    assert rs.stype == 'row_sparse' and same(rs.indices.asnumpy(), np.array([1, 4]))
    assert same(rs.data.asnumpy(), dense[[1, 4]])
    csr = nd.array(dense).tostype('csr')
    assert csr.stype == 'csr' and same(csr.indptr.asnumpy(), np.array([0, 0, 2, 2, 2, 4, 4]))
    assert same(csr.tostype('default').asnumpy(), dense)
    f = str(tmp_path / 's.params')
    nd.save(f, {'rs': rs, 'csr': csr})
    back = nd.load(f)
    assert back['rs'].stype == 'row_sparse' and back['csr'].stype == 'csr'
    assert same(back['rs'].tostype('default').asnumpy(), dense) and same(back['csr'].tostype('default').asnumpy(), dense)
    w = np.random.randn(4, 3).astype('float32')
    assert_almost_equal(nd.dot(csr, nd.array(w)).asnumpy(), dense @ w, rtol=1e-5, atol=1e-6)
    made = nd.sparse.row_sparse_array((dense[[1, 4]], [1, 4]), shape=(6, 4))
    assert same(made.tostype('default').asnumpy(), dense)
    made = nd.sparse.csr_matrix((csr.data.asnumpy(), csr.indices.asnumpy(), csr.indptr.asnumpy()), shape=(6, 4))
    assert same(made.tostype('default').asnumpy(), dense)


def test_wait_and_scalar_conversions():
    a = nd.array([3.5])
    a.wait_to_read()
    nd.waitall()
    assert a.asscalar() == 3.5 and float(a) == 3.5 and int(a) == 3 and bool(nd.array([1]))
    with pytest.raises(ValueError):
        nd.array([1, 2]).asscalar()


def test_random_ops_statistics():
    mx.random.seed(42)
    u = nd.random.uniform(-1, 3, shape=(20000,)).asnumpy()
    assert abs(u.mean() - 1.0) < 0.05 and u.min() >= -1 and u.max() <= 3
    n = nd.random.normal(2, 0.5, shape=(20000,)).asnumpy()
    assert abs(n.mean() - 2) < 0.02 and abs(n.std() - 0.5) < 0.02
    mx.random.seed(7)
    a = nd.random.uniform(shape=(5,)).asnumpy()
    mx.random.seed(7)
    b = nd.random.uniform(shape=(5,)).asnumpy()
    assert same(a, b)
    r = nd.random.randint(0, 5, shape=(1000,)).asnumpy()
    assert r.min() >= 0 and r.max() <= 4
    m = nd.random.multinomial(nd.array([0.0, 1.0, 0.0]), shape=8).asnumpy()
    assert (m == 1).all()

"""Sparse arrays: compressed storage, products from the components, storage fallback.

Modelled on tests/python/unittest/test_sparse_ndarray.py and test_sparse_operator.py of the reference (creation from
components, cast_storage round trips, dot(csr, dense) in both orientations against scipy, retain, add_n)."""
import numpy as np
import pytest
import scipy.sparse as sp
import torch

import mxnet_b200 as mx
from mxnet_b200.ndarray import sparse


def _random_csr(m, k, density, seed, dtype='float32'):
    mat = sp.random(m, k, density=density, format='csr', random_state=np.random.RandomState(seed), dtype=np.float64)
    mat.sort_indices()
    return mat.astype(dtype)


def test_csr_from_components_is_compressed_until_the_dense_tensor_is_touched():
    mat = _random_csr(50, 70, 0.05, 0)
    a = sparse.csr_matrix((mat.data, mat.indices, mat.indptr), shape=mat.shape)
    assert a.is_compressed and a.stype == 'csr' and a.shape == (50, 70) and a.dtype == np.float32 and a.nnz == mat.nnz
    np.testing.assert_array_equal(a.indices.asnumpy(), mat.indices)
    np.testing.assert_array_equal(a.indptr.asnumpy(), mat.indptr)
    assert a.is_compressed                          # reading components keeps it compressed
    b = a.copy()
    np.testing.assert_allclose(a.asnumpy(), mat.toarray())
    assert not a.is_compressed and b.is_compressed  # asnumpy is the storage fallback; the copy is untouched
    np.testing.assert_allclose(a.asscipy().toarray(), mat.toarray())
    np.testing.assert_allclose(b.tostype('default').asnumpy(), mat.toarray())


def test_a_matrix_too_large_for_dense_storage_can_be_created_and_multiplied():
    """10^6 x 10^6 (4 TB dense) with 5000 non-zeros: creation, copy, both products and retain never materialise it."""
    n = 1000000
    rng = np.random.RandomState(1)
    rows = np.sort(rng.randint(0, n, 5000))
    cols = rng.randint(0, n, 5000)
    vals = rng.uniform(-1, 1, 5000).astype('float32')
    mat = sp.csr_matrix((vals, (rows, cols)), shape=(n, n))
    mat.sum_duplicates()
    mat.sort_indices()
    a = sparse.csr_matrix(mat)
    assert a.is_compressed and a.shape == (n, n)
    w = rng.uniform(-1, 1, (n, 2)).astype('float32')
    out = sparse.dot(a, mx.nd.array(w))
    np.testing.assert_allclose(out.asnumpy(), mat @ w, rtol=1e-5, atol=1e-5)
    g = sparse.dot(a, mx.nd.array(w), transpose_a=True, forward_stype='row_sparse')
    assert g.stype == 'row_sparse' and g.is_compressed and g.shape == (n, 2)
    expect = mat.T @ w
    touched = np.unique(mat.indices)
    np.testing.assert_array_equal(g.indices.asnumpy(), touched)
    np.testing.assert_allclose(g.data.asnumpy(), expect[touched], rtol=1e-5, atol=1e-5)
    kept = g.retain(mx.nd.array(touched[:10]))
    assert kept.is_compressed and kept.indices.shape[0] == 10
    z = sparse.zeros('csr', (n, n))
    assert z.is_compressed and z.nnz == 0
    assert a.is_compressed


@pytest.mark.parametrize('transpose_a', [False, True])
@pytest.mark.parametrize('n', [1, 7, 64])
def test_dot_of_a_compressed_csr_matches_scipy_on_the_host(transpose_a, n):
    mat = _random_csr(40, 30, 0.2, 2)
    a = sparse.csr_matrix(mat)
    rhs = np.random.RandomState(3).uniform(-1, 1, (40 if transpose_a else 30, n)).astype('float32')
    out = sparse.dot(a, mx.nd.array(rhs), transpose_a=transpose_a)
    np.testing.assert_allclose(out.asnumpy(), (mat.T if transpose_a else mat) @ rhs, rtol=1e-5, atol=1e-5)
    assert a.is_compressed
    v = sparse.dot(a, mx.nd.array(rhs[:, 0]), transpose_a=transpose_a)
    np.testing.assert_allclose(v.asnumpy(), (mat.T if transpose_a else mat) @ rhs[:, 0], rtol=1e-5, atol=1e-5)


def test_row_sparse_components_add_n_and_fallback():
    a = sparse.row_sparse_array((np.ones((2, 3), 'float32'), [4, 1]), shape=(6, 3))
    b = sparse.row_sparse_array((2 * np.ones((2, 3), 'float32'), [1, 5]), shape=(6, 3))
    assert a.is_compressed
    np.testing.assert_array_equal(a.indices.asnumpy(), [1, 4])           # indices come out sorted
    s = sparse.add_n(a, b)
    assert s.is_compressed
    np.testing.assert_array_equal(s.indices.asnumpy(), [1, 4, 5])
    np.testing.assert_allclose(s.data.asnumpy(), [[3, 3, 3], [1, 1, 1], [2, 2, 2]])
    dense = (a + 1).asnumpy()                                             # an operator without a sparse form: dense fallback
    expect = np.ones((6, 3), 'float32')
    expect[[1, 4]] += 1
    np.testing.assert_allclose(dense, expect)
    a[:] = 0                                                              # writes go to the dense tensor
    assert not a.is_compressed and float(a.asnumpy().sum()) == 0


def test_compressed_arrays_save_and_load(tmp_path):
    mat = _random_csr(20, 15, 0.3, 5)
    a = sparse.csr_matrix(mat)
    r = sparse.row_sparse_array((np.arange(6, dtype='float32').reshape(2, 3), [0, 3]), shape=(5, 3))
    path = str(tmp_path / 'sp.params')
    mx.nd.save(path, {'a': a, 'r': r})
    back = mx.nd.load(path)
    assert back['a'].stype == 'csr' and back['r'].stype == 'row_sparse'
    np.testing.assert_allclose(back['a'].asnumpy(), mat.toarray())
    np.testing.assert_allclose(back['r'].asnumpy(), r.asnumpy())


@pytest.mark.gpu
@pytest.mark.parametrize('dtype', ['float32', 'float16', 'bfloat16'])
@pytest.mark.parametrize('m,k,n,density', [(300, 200, 1, 0.05), (257, 129, 33, 0.1), (1000, 5000, 128, 0.01), (64, 64, 300, 0.5)])
def test_csr_product_kernels_match_scipy(dtype, m, k, n, density):
    """The in-tree CSR x dense kernels (both orientations) against scipy in float64 on the values the GPU sees."""
    from mxnet_b200.ops import cuda
    ctx = mx.gpu(0)
    mat = _random_csr(m, k, density, 7)
    td = getattr(torch, dtype)
    a = sparse.csr_matrix(mat, ctx=ctx, dtype=dtype)
    vals = a.data._data.double().cpu().numpy()
    mat64 = sp.csr_matrix((vals, mat.indices, mat.indptr), shape=mat.shape)
    tol = {'float32': 1e-5, 'float16': 4e-3, 'bfloat16': 3e-2}[dtype]
    for transpose_a in (False, True):
        rhs = torch.randn(m if transpose_a else k, n, device='cuda').to(td)
        before = cuda.launches()
        out = sparse.dot(a, mx.nd.NDArray._from_tensor(rhs, ctx), transpose_a=transpose_a)
        assert cuda.launches() == before + 1 and a.is_compressed
        expect = (mat64.T if transpose_a else mat64) @ rhs.double().cpu().numpy()
        scale = max(1.0, float(np.abs(expect).max()))
        np.testing.assert_allclose(out._data.double().cpu().numpy() / scale, expect / scale, rtol=0, atol=tol)


@pytest.mark.parametrize('name,kwargs', [('sgd', {'momentum': 0.9, 'wd': 0.1}), ('sgd', {'momentum': 0.0, 'wd': 0.1}),
                                         ('adam', {'wd': 0.05})])
def test_lazy_update_touches_only_the_rows_of_a_row_sparse_gradient(name, kwargs):
    """``lazy_update=True`` (reference: SGDUpdateRspImpl / AdamLazyUpdate in src/operator/optimizer_op.cc): rows absent from
    the gradient keep their weight and state (no weight decay, no momentum decay); present rows get the dense formula."""
    rng = np.random.RandomState(9)
    w0 = rng.uniform(-1, 1, (8, 3)).astype('float32')
    rows = [1, 4, 6]
    gvals = rng.uniform(-1, 1, (3, 3)).astype('float32')
    results = {}
    for lazy in (True, False):
        opt = mx.optimizer.create(name, learning_rate=0.1, lazy_update=lazy, **kwargs)
        w = mx.nd.array(w0.copy())
        state = opt.create_state(0, w)
        for _ in range(3):
            g = sparse.row_sparse_array((gvals, rows), shape=(8, 3))
            opt.update(0, w, g, state)
        results[lazy] = w.asnumpy()
    untouched = [r for r in range(8) if r not in rows]
    np.testing.assert_array_equal(results[True][untouched], w0[untouched])          # lazy: other rows are exactly as before
    assert np.abs(results[False][untouched] - w0[untouched]).max() > 1e-3           # standard: weight decay reached them
    # the touched rows follow the dense formula restricted to those rows
    opt = mx.optimizer.create(name, learning_rate=0.1, lazy_update=False, **kwargs)
    w = mx.nd.array(w0[rows].copy())
    state = opt.create_state(0, w)
    for _ in range(3):
        opt.update(0, w, mx.nd.array(gvals), state)
    np.testing.assert_allclose(results[True][rows], w.asnumpy(), rtol=1e-6, atol=1e-7)


def test_libsvm_batches_stay_compressed_and_train_a_sparse_linear_model(tmp_path):
    """The sparse linear-classification recipe of the reference (example/sparse/linear_classification): LibSVM batches in
    CSR form over a feature space far too wide for dense batches, weights updated lazily from row-sparse gradients."""
    dim, n = 2000000, 64
    rng = np.random.RandomState(11)
    truth = {}
    lines = []
    for i in range(n):
        feats = np.sort(rng.choice(dim, 6, replace=False))
        label = int(feats[0] % 2)
        lines.append('%d %s' % (label, ' '.join('%d:1.0' % f for f in feats)))
        truth[i] = label
    path = str(tmp_path / 'wide.libsvm')
    open(path, 'w').write('\n'.join(lines) + '\n')
    it = mx.io.LibSVMIter(data_libsvm=path, data_shape=(dim,), batch_size=16)
    assert it.provide_data[0].shape == (16, dim)
    w = mx.nd.zeros((dim, 1))
    opt = mx.optimizer.create('sgd', learning_rate=0.5, lazy_update=True, wd=0.0)
    first = last = None
    for epoch in range(30):
        it.reset()
        total = 0.0
        for batch in it:
            x, y = batch.data[0], batch.label[0]
            assert x.stype == 'csr' and x.is_compressed and x.shape == (16, dim)
            z = sparse.dot(x, w)                                              # [16, 1] from the components
            p = 1 / (1 + np.exp(-z.asnumpy()[:, 0]))
            yy = y.asnumpy()
            total += float(-(yy * np.log(p + 1e-9) + (1 - yy) * np.log(1 - p + 1e-9)).sum())
            dz = mx.nd.array(((p - yy) / len(yy)).reshape(-1, 1).astype('float32'))
            g = sparse.dot(x, dz, transpose_a=True, forward_stype='row_sparse')   # gradient only for the features seen
            assert g.is_compressed and g.indices.shape[0] <= 16 * 6
            opt.update(0, w, g, None)
        first = total if first is None else first
        last = total
    assert last < 0.5 * first


def test_sparse_elementwise_functions():
    a = sparse.row_sparse_array((np.ones((2, 3), 'float32'), [0, 3]), shape=(5, 3))
    b = sparse.row_sparse_array((2 * np.ones((2, 3), 'float32'), [3, 4]), shape=(5, 3))
    s = sparse.add(a, b)
    assert s.stype == 'row_sparse' and s.is_compressed
    np.testing.assert_array_equal(s.indices.asnumpy(), [0, 3, 4])
    d = sparse.subtract(a, b)
    np.testing.assert_allclose(d.asnumpy()[[0, 3, 4]], [[1, 1, 1], [-1, -1, -1], [-2, -2, -2]])
    m = sparse.multiply(a, 3.0)
    assert m.is_compressed and float(m.asnumpy().sum()) == 18.0
    q = sparse.divide(b, 4.0)
    assert q.is_compressed and float(q.asnumpy().sum()) == 3.0
    dense = sparse.add(a, mx.nd.ones((5, 3)))
    assert dense.stype == 'default' and float(dense.asnumpy().sum()) == 21.0


def test_check_format_rejects_broken_components():
    good = sparse.csr_matrix(([1., 2., 3.], [0, 2, 1], [0, 2, 3]), shape=(2, 3))
    good.check_format()
    bad = sparse.csr_matrix(([1., 2., 3.], [2, 0, 1], [0, 2, 3]), shape=(2, 3))        # unsorted columns in row 0
    with pytest.raises(mx.MXNetError):
        bad.check_format()
    bad.check_format(full_check=False)
    out_of_range = sparse.csr_matrix(([1.], [5], [0, 1, 1]), shape=(2, 3))
    with pytest.raises(mx.MXNetError):
        out_of_range.check_format()
    rsp = sparse.row_sparse_array((np.ones((2, 2), 'float32'), [1, 3]), shape=(4, 2))
    rsp.check_format()
    assert mx.sym.Variable('x').split_v2(2).list_outputs() != []

"""Operator libraries on the C ABI (mxb_lib_api.h): build the example with the host compiler, load it, run the
operators imperatively, under autograd and through a Symbol."""
import os
import shutil
import subprocess

import numpy as np
import pytest

import mxnet_b200 as mx
from mxnet_b200 import autograd, nd
from mxnet_b200.base import MXNetError

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, 'example', 'extensions', 'lib_custom_op')


@pytest.fixture(scope='module')
def gemm_lib(tmp_path_factory):
    if shutil.which('g++') is None:
        pytest.skip('no host compiler')
    out = str(tmp_path_factory.mktemp('ext') / 'libgemm_lib.so')
    subprocess.check_call(['g++', '-O2', '-shared', '-fPIC', '-I', mx.library.include_dir(),
                           os.path.join(SRC, 'gemm_lib.cc'), '-o', out])
    mx.library.load(out, verbose=False)
    return out


def test_operator_from_library_forward_backward(gemm_lib):
    assert gemm_lib in mx.library.loaded_libraries()
    rng = np.random.RandomState(0)
    a, b = rng.randn(5, 7).astype('float32'), rng.randn(7, 3).astype('float32')
    x, y = nd.array(a), nd.array(b)
    np.testing.assert_allclose(nd.my_gemm(x, y).asnumpy(), a @ b, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(nd.my_gemm(A=x, B=y).asnumpy(), a @ b, rtol=1e-5, atol=1e-5)
    x.attach_grad()
    y.attach_grad()
    with autograd.record():
        z = nd.my_gemm(x, y)
        loss = (z * z).sum()
    loss.backward()
    dz = 2 * (a @ b)
    np.testing.assert_allclose(x.grad.asnumpy(), dz @ b.T, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(y.grad.asnumpy(), a.T @ dz, rtol=1e-4, atol=1e-4)


def test_library_errors_surface_as_mxnet_errors(gemm_lib):
    with pytest.raises(MXNetError, match='inner extents differ'):
        nd.my_gemm(nd.ones((2, 3)), nd.ones((4, 5)))
    with pytest.raises(MXNetError, match='float32 only'):
        nd.my_gemm(nd.ones((2, 3), dtype='float64'), nd.ones((3, 5), dtype='float64'))
    with pytest.raises(MXNetError):
        mx.library.load('relative/path.so')


def test_stateful_operator_and_attributes(gemm_lib):
    a, b = nd.ones((2, 2)), nd.ones((2, 2))
    c, calls = nd.my_state_gemm(a, b, count=41)
    np.testing.assert_allclose(c.asnumpy(), np.full((2, 2), 2.0))
    assert calls.dtype == np.int64 and int(calls.asnumpy()[0]) == 42


def test_library_operator_in_symbol_and_numpy_namespaces(gemm_lib):
    A, B = mx.sym.var('A'), mx.sym.var('B')
    s = mx.sym.my_gemm(A, B)
    _, out_shapes, _ = s.infer_shape(A=(4, 6), B=(6, 9))
    assert out_shapes == [(4, 9)]
    a, b = np.arange(24, dtype='float32').reshape(4, 6), np.ones((6, 9), dtype='float32')
    ex = s._bind(mx.cpu(), {'A': nd.array(a), 'B': nd.array(b)})
    np.testing.assert_allclose(ex.forward()[0].asnumpy(), a @ b, rtol=1e-5)
    js = mx.sym.load_json(s.tojson())
    assert js.list_arguments() == ['A', 'B']
    r = mx.npx.my_gemm(mx.np.array(a), mx.np.array(b))
    assert type(r).__name__ == 'ndarray'
    np.testing.assert_allclose(r.asnumpy(), a @ b, rtol=1e-5)


@pytest.mark.gpu
def test_cuda_operator_library_runs_on_the_callers_stream(tmp_path):
    if shutil.which('nvcc') is None:
        pytest.skip('no CUDA compiler')
    out = str(tmp_path / 'librelu_lib.so')
    subprocess.check_call(['nvcc', '-O2', '-shared', '-Xcompiler', '-fPIC', '-gencode', 'arch=compute_100a,code=sm_100a',
                           '-I', mx.library.include_dir(), os.path.join(SRC, 'relu_lib.cu'), '-o', out])
    mx.library.load(out, verbose=False)
    rng = np.random.RandomState(1)
    v = rng.randn(257, 33).astype('float32')
    for ctx in (mx.cpu(), mx.gpu(0)):
        x = nd.array(v, ctx=ctx)
        x.attach_grad()
        with autograd.record():
            y = nd.my_relu(x)
            loss = (y * 3).sum()
        loss.backward()
        np.testing.assert_allclose(y.asnumpy(), np.maximum(v, 0))
        np.testing.assert_allclose(x.grad.asnumpy(), 3.0 * (v > 0))


def test_graph_pass_from_library(tmp_path):
    if shutil.which('g++') is None:
        pytest.skip('no host compiler')
    out = str(tmp_path / 'libpass_lib.so')
    subprocess.check_call(['g++', '-O2', '-shared', '-fPIC', '-I', mx.library.include_dir(),
                           os.path.join(ROOT, 'example', 'extensions', 'lib_pass', 'pass_lib.cc'), '-o', out])
    mx.library.load(out, verbose=False)
    x = mx.sym.var('x')
    s = mx.sym.sigmoid(x * 2.0)
    t = s.optimize_for('swap_op', **{'from': 'sigmoid', 'to': 'tanh'})
    v = np.linspace(-1, 1, 7).astype('float32')
    got = t._bind(mx.cpu(), {'x': nd.array(v)}).forward()[0].asnumpy()
    np.testing.assert_allclose(got, np.tanh(2 * v), rtol=1e-5, atol=1e-6)
    with pytest.raises(MXNetError, match='needs the options'):
        s.optimize_for('swap_op')

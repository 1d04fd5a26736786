"""The C interface (``include/mxnet_b200/c_api.h``): a plain-C program built against ``libmxb200_rt.so`` creates arrays,
round-trips them through the file format, invokes native operators, pushes host functions to the engine and drives the
local key-value store, on the host and (GPU run) on the sm_100a kernels, with no Python in the process.  The ``.params``
file it writes is then read back here, so both sides agree on the format."""
import os
import subprocess

import numpy as np
import pytest

import mxnet_b200 as mx
from mxnet_b200.csrc import runtime

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build(tmp_path):
    runtime.lib()                                  # builds libmxb200_rt.so when needed
    libdir = os.path.dirname(runtime.LIB_PATH)
    exe = str(tmp_path / 'c_api_test')
    cmd = ['gcc', '-std=c11', '-O1', '-Wall', '-Werror', '-I', os.path.join(ROOT, 'mxnet_b200', 'include'),
           os.path.join(ROOT, 'cpp-package', 'tests', 'c_api_test.c'), '-o', exe, '-L', libdir, '-lmxb200_rt', '-lm',
           '-Wl,-rpath,' + libdir]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def _run(tmp_path, where):
    exe = _build(tmp_path)
    fname = str(tmp_path / 'from_c.params')
    r = subprocess.run([exe, where, fname], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert 'all checks passed' in r.stdout
    loaded = mx.nd.load(fname)                     # written by the C program, read by the Python front end
    expect = (np.arange(32) % 7 - 3).astype('float32').reshape(4, 8)
    np.testing.assert_array_equal(loaded['arg:whole'].asnumpy(), expect)
    np.testing.assert_array_equal(loaded['arg:rows'].asnumpy(), expect[1:3])


def test_c_api_program_on_the_host(tmp_path):
    _run(tmp_path, 'cpu')


@pytest.mark.gpu
def test_c_api_program_on_the_gpu_kernels(tmp_path):
    _run(tmp_path, 'gpu')


def test_c_api_reads_a_file_written_by_python(tmp_path):
    import ctypes
    L = ctypes.CDLL(runtime.lib()._name)
    L.MXGetLastError.restype = ctypes.c_char_p
    fname = str(tmp_path / 'from_python.params')
    src = {'w': mx.nd.array(np.arange(6, dtype='float32').reshape(2, 3)), 'i': mx.nd.array([1, 2, 3], dtype='int64')}
    mx.nd.save(fname, src)
    n, nn = ctypes.c_uint32(), ctypes.c_uint32()
    arrs, names = ctypes.POINTER(ctypes.c_void_p)(), ctypes.POINTER(ctypes.c_char_p)()
    assert L.MXNDArrayLoad(fname.encode(), ctypes.byref(n), ctypes.byref(arrs), ctypes.byref(nn), ctypes.byref(names)) == 0, \
        L.MXGetLastError()
    got = {}
    for k in range(n.value):
        ndim, dims, dt = ctypes.c_int(), ctypes.POINTER(ctypes.c_int)(), ctypes.c_int()
        h = ctypes.c_void_p(arrs[k])
        assert L.MXNDArrayGetShapeEx(h, ctypes.byref(ndim), ctypes.byref(dims)) == 0
        assert L.MXNDArrayGetDType(h, ctypes.byref(dt)) == 0
        shape = tuple(dims[i] for i in range(ndim.value))
        out = np.empty(shape, dtype={0: 'float32', 6: 'int64'}[dt.value])
        assert L.MXNDArraySyncCopyToCPU(h, out.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(out.size)) == 0
        got[names[k].decode()] = out
        L.MXNDArrayFree(h)
    assert set(got) == {'w', 'i'}
    np.testing.assert_array_equal(got['w'], src['w'].asnumpy())
    np.testing.assert_array_equal(got['i'], src['i'].asnumpy())

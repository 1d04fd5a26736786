"""The C++ front end: compile the example against the in-tree runtime library and check its output from Python."""
import os
import shutil
import subprocess

import numpy as np
import pytest

from mxnet_b200 import nd
from mxnet_b200.csrc import runtime

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which('g++') is None, reason='needs a C++ compiler')
def test_cpp_example_reads_scales_and_writes_params(tmp_path):
    runtime.lib()                                                 # builds libmxb200_rt.so when missing
    libdir = os.path.join(ROOT, 'mxnet_b200', 'csrc')
    exe = str(tmp_path / 'params_tool')
    subprocess.run(['g++', '-std=c++17', '-O1', '-I', os.path.join(ROOT, 'cpp-package', 'include'),
                    os.path.join(ROOT, 'cpp-package', 'example', 'params_tool.cpp'), '-L', libdir, '-lmxb200_rt',
                    '-Wl,-rpath,' + libdir, '-pthread', '-o', exe], check=True)
    src, dst = str(tmp_path / 'in.params'), str(tmp_path / 'out.params')
    arrays = {'arg:w': nd.array(np.arange(6, dtype='float32').reshape(2, 3)), 'arg:idx': nd.array([1, 2, 3], dtype='int32'),
              'aux:m': nd.array(np.ones((4,), 'float32') * 0.5)}
    nd.save(src, arrays)
    r = subprocess.run([exe, src, dst], capture_output=True, text=True, check=True)
    assert 'arg:w ndim=2 dtype=0 bytes=24' in r.stdout and 'tasks=2' in r.stdout and 'caught: expected failure' in r.stdout
    back = nd.load(dst)
    assert sorted(back) == sorted(arrays)
    np.testing.assert_array_equal(back['arg:w'].asnumpy(), arrays['arg:w'].asnumpy() * 2)
    np.testing.assert_array_equal(back['aux:m'].asnumpy(), np.ones(4, 'float32'))
    np.testing.assert_array_equal(back['arg:idx'].asnumpy(), [1, 2, 3])
    assert back['arg:idx'].dtype == np.int32

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


def _embed_flags():
    import sysconfig
    import pybind11
    inc = ['-I', pybind11.get_include(), '-I', sysconfig.get_paths()['include']]
    cfg = shutil.which('python3-config')
    if cfg is None:
        pytest.skip('python3-config is needed to link the embedded interpreter')
    ld = subprocess.run([cfg, '--ldflags', '--embed'], capture_output=True, text=True)
    if ld.returncode != 0:
        pytest.skip('python3-config --embed is not supported here')
    return inc, ld.stdout.split()


def _run_embedded(exe, cwd):
    import site
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([ROOT] + site.getsitepackages()))
    return subprocess.run([exe], capture_output=True, text=True, timeout=600, cwd=cwd, env=env)


@pytest.mark.skipif(shutil.which('g++') is None, reason='needs a C++ compiler')
def test_cpp_frontend_trains_an_mlp(tmp_path):
    """NDArray / Symbol / Operator / Executor / Optimizer / metric of the C++ front end (embedded interpreter)."""
    inc, ld = _embed_flags()
    exe = str(tmp_path / 'mlp_cpu')
    r = subprocess.run(['g++', '-std=c++17', '-O1', os.path.join(ROOT, 'cpp-package', 'example', 'mlp_cpu.cpp'), '-I',
                        os.path.join(ROOT, 'cpp-package', 'include')] + inc + ld + ['-o', exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    r = _run_embedded(exe, str(tmp_path))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert 'epoch 4: validation accuracy' in r.stdout and 'relu -> 1 0 3 0; saved 2 arrays; w0 128x64' in r.stdout
    back = nd.load(str(tmp_path / 'mlp_cpu_weights.params'))
    assert back['arg:w0'].shape == (128, 64)


@pytest.mark.skipif(shutil.which('g++') is None, reason='needs a C++ compiler')
def test_generated_operator_wrappers_are_current_and_compile(tmp_path):
    from mxnet_b200.tools import op_wrapper_generator
    committed = open(os.path.join(ROOT, 'cpp-package', 'include', 'mxb200', 'op.h')).read()
    assert committed == op_wrapper_generator.generate(), 'regenerate with python -m mxnet_b200.tools.op_wrapper_generator'
    inc, ld = _embed_flags()
    src = tmp_path / 'op_test.cpp'
    src.write_text('''
#include <cstdio>
#include "mxb200/op.h"
using namespace mxb200;
int main() {
  Symbol x = Symbol::Variable("x");
  Symbol fc = op::FullyConnected("fc", x, Symbol::Variable("w"), Symbol(), Attrs().Set("num_hidden", 3).Set("no_bias", true));
  Symbol cat = op::Concat("cat", {op::Activation("act", fc, Attrs().Set("act_type", "tanh")), fc}, Attrs().Set("dim", 1));
  std::vector<std::vector<mx_uint>> a, u, o;
  cat.InferShape({{"x", {4, 5}}}, &a, &u, &o);
  NDArray v(std::vector<float>{-1, 2, -3, 4}, Shape(2, 2), Context::cpu());
  auto r = op::relu(v);
  auto s = op::add_n({v, v, v});
  std::printf("out %ux%u relu %.0f %.0f add_n %.0f\\n", o[0][0], o[0][1], r[0].At(0), r[0].At(1), s[0].At(3));
  return 0;
}
''')
    exe = str(tmp_path / 'op_test')
    r = subprocess.run(['g++', '-std=c++17', '-O0', str(src), '-I', os.path.join(ROOT, 'cpp-package', 'include')] + inc + ld + ['-o', exe],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    r = _run_embedded(exe, str(tmp_path))
    assert r.returncode == 0 and 'out 4x6 relu 0 2 add_n 12' in r.stdout, r.stdout + r.stderr[-2000:]

"""The CPU operator, array, autograd, loss and optimizer tests once more with the GPU as the default device: every
array the tests create without an explicit device lands on ``gpu(0)``, so the same assertions check the GPU code paths
(the scheme of ``tests/python/gpu/test_operator_gpu.py`` in the reference, which re-imports the CPU suite after
``set_default_device(mx.gpu(0))``)."""
import importlib
import inspect
import itertools
import os
import sys

import pytest

import mxnet_b200 as mx

_PARAM_SET = type(pytest.param(0))

pytestmark = pytest.mark.gpu

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

MODULES = ['test_ndarray', 'test_numpy_frontend', 'test_autograd', 'test_loss_metric', 'test_optimizer', 'test_probability',
           'test_contrib_misc', 'test_contrib_detection', 'test_gluon', 'test_symbol', 'test_rnn_estimator', 'test_amp',
           'test_misc_api', 'test_extra_ops', 'test_contrib_data', 'test_sparse']

# tests that are about the host itself (files, pinned host memory, CPU shared memory, numpy interop of host buffers)
HOST_ONLY = {
    'test_ndarray': ('test_copy_and_context', 'test_creation_and_basic_properties'),   # assert cpu(0) as the default device
    'test_extra_ops': ('test_random_additions_have_the_right_moments',),               # statistical test: host generator only
}


def _expand(fn):
    """(id suffix, kwargs) for every combination of the test's parametrize marks; fixture-taking tests are left out."""
    marks = [m for m in getattr(fn, 'pytestmark', []) if m.name == 'parametrize']
    if any(m.name in ('gpu', 'skip') for m in getattr(fn, 'pytestmark', [])):
        return
    axes = []
    for m in marks:
        names = m.args[0]
        names = [n.strip() for n in names.split(',')] if isinstance(names, str) else list(names)
        values = []
        for v in m.args[1]:
            if isinstance(v, _PARAM_SET):            # pytest.param(...)
                v = v.values if len(names) > 1 else v.values[0]
            values.append(dict(zip(names, v if len(names) > 1 else [v])))
        axes.append(values)
    params = set(inspect.signature(fn).parameters)
    covered = set()
    for ax in axes:
        covered |= set(ax[0]) if ax else set()
    if params - covered:
        return                                   # needs a fixture
    if not axes:
        yield '', {}
        return
    for i, combo in enumerate(itertools.product(*axes)):
        kw = {}
        for c in combo:
            kw.update(c)
        yield '[%d]' % i, kw


def _cases():
    out = []
    for m in MODULES:
        mod = importlib.import_module(m)
        for name, fn in sorted(vars(mod).items()):
            if not name.startswith('test_') or not inspect.isfunction(fn) or fn.__module__ != mod.__name__:
                continue
            if name in HOST_ONLY.get(m, ()):
                continue
            for suffix, kw in _expand(fn):
                out.append(pytest.param(fn, kw, id='%s::%s%s' % (m, name, suffix)))
    return out


@pytest.mark.parametrize('fn,kwargs', _cases())
def test_cpu_suite_with_gpu_default_device(fn, kwargs):
    from mxnet_b200 import env
    # recurrent layers on the in-tree kernels: exact fp32 arithmetic, where the library recurrence may use TF32 and then
    # misses the 1e-4 tolerances that the host tests put on fp32 results
    with env.scope('MXNET_B200_RNN', '1'), mx.gpu(0):
        fn(**kwargs)
    mx.nd.waitall()

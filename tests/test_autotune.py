"""Selection logic of the convolution / GEMM autotuners (timing is faked; no GPU needed)."""
import pytest
import torch

from mxnet_b200.ops.cuda import conv_ops, gemm_ops


@pytest.fixture
def no_capture(monkeypatch):
    monkeypatch.setattr(torch.cuda, 'is_current_stream_capturing', lambda: False)


def test_conv_directions_parsing(monkeypatch):
    monkeypatch.delenv('MXNET_B200_CONV', raising=False)
    assert conv_ops.directions() == frozenset(('auto',))
    for v, want in (('0', frozenset()), ('1', {'fwd', 'dgrad', 'wgrad'}), ('fwd, wgrad', {'fwd', 'wgrad'}), ('AUTO', {'auto'})):
        monkeypatch.setenv('MXNET_B200_CONV', v)
        assert conv_ops.directions() == frozenset(want)


def test_conv_autotune_keeps_the_faster_and_caches(monkeypatch, no_capture):
    calls = []
    times = {'own': 10.0, 'lib': 12.0}
    monkeypatch.setattr(conv_ops, '_time_us', lambda fn, reps=5: (calls.append(fn()), times[fn()])[1])
    monkeypatch.setattr(conv_ops, '_tuned', {})
    dirs = frozenset(('auto',))
    key = (torch.float16, 1, 8, 8, 64, 64, 3, 3, 1, 1, 1, 1)
    assert conv_ops.use_own('fwd', dirs, key, lambda: 'own', lambda: 'lib') is True
    n = len(calls)
    assert conv_ops.use_own('fwd', dirs, key, lambda: 'own', lambda: 'lib') is True       # cached: no new timing
    assert len(calls) == n
    times['own'] = 13.0
    assert conv_ops.use_own('dgrad', dirs, key, lambda: 'own', lambda: 'lib') is False
    # the forward kernel is credited with the BatchNorm reduction it replaces
    assert conv_ops.use_own('wgrad', dirs, key, lambda: 'own', lambda: 'lib', lib_extra_us=2.0) is True
    assert conv_ops.tuned_choices()[('dgrad',) + key] is False
    # forced modes do not time anything
    assert conv_ops.use_own('fwd', frozenset(('fwd',)), key, None, None) is True
    assert conv_ops.use_own('dgrad', frozenset(('fwd',)), key, None, None) is False


def test_conv_autotune_defers_during_graph_capture(monkeypatch):
    monkeypatch.setattr(torch.cuda, 'is_current_stream_capturing', lambda: True)
    monkeypatch.setattr(conv_ops, '_tuned', {})
    key = (torch.float16, 2, 4, 4, 8, 8, 1, 1, 0, 0, 1, 1)
    assert conv_ops.use_own('fwd', frozenset(('auto',)), key, lambda: 1 / 0, lambda: 1 / 0) is False
    assert conv_ops.tuned_choices() == {}             # nothing cached: the next eager call tunes


def test_gemm_autotune_ties_go_to_the_in_tree_kernel(monkeypatch, no_capture):
    times = {'own': 10.1, 'lib': 10.0}
    monkeypatch.setattr(gemm_ops, '_time_us', lambda fn, reps=5: times[fn()])
    monkeypatch.setattr(gemm_ops, '_tuned', {})
    monkeypatch.setenv('MXNET_B200_GEMM_AUTOTUNE', '1')
    assert gemm_ops.use_own(('fwd', torch.float16, 8, 8, 8, False, None), lambda: 'own', lambda: 'lib') is True
    times['own'] = 11.0
    assert gemm_ops.use_own(('dgrad', torch.float16, 8, 8, 8), lambda: 'own', lambda: 'lib') is False
    monkeypatch.setenv('MXNET_B200_GEMM_AUTOTUNE', '0')
    assert gemm_ops.use_own(('wgrad', torch.float16, 8, 8, 8), lambda: 1 / 0, lambda: 1 / 0) is True

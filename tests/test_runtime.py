"""Native runtime: dependency engine, storage pools, profiler, exception propagation (reference:
tests/cpp/engine/threaded_engine_test.cc, tests/cpp/storage/storage_test.cc,
tests/python/unittest/test_engine.py, test_exc_handling.py, test_profiler.py)."""
import json
import os
import threading
import time

import numpy as np
import pytest

import mxnet_b200 as mx
from mxnet_b200 import nd, profiler
from mxnet_b200.csrc import runtime


def test_engine_orders_writes_and_parallelises_reads():
    eng = runtime.Engine(num_workers=4)
    v = eng.new_var()
    log, lock = [], threading.Lock()

    def writer(tag):
        def fn():
            with lock:
                log.append(('w', tag))
            time.sleep(0.01)
        return fn

    active, peak = [0], [0]

    def reader():
        with lock:
            active[0] += 1
            peak[0] = max(peak[0], active[0])
        time.sleep(0.05)
        with lock:
            active[0] -= 1
    eng.push(writer(0), write_vars=[v])
    for _ in range(4):
        eng.push(reader, read_vars=[v])
    eng.push(writer(1), write_vars=[v])
    eng.push(writer(2), write_vars=[v])
    eng.wait_for_var(v)
    assert log == [('w', 0), ('w', 1), ('w', 2)]
    assert peak[0] >= 2, 'reads of one variable must run concurrently'
    assert v.version == 3
    eng.wait_all()
    assert eng.num_pending == 0


def test_engine_dependency_chain_across_vars():
    eng = runtime.Engine(num_workers=4)
    a, b, c = eng.new_var(), eng.new_var(), eng.new_var()
    vals = {'a': 0, 'b': 0, 'c': 0}

    def set_a():
        time.sleep(0.03)
        vals['a'] = 2

    def a_to_b():
        vals['b'] = vals['a'] * 10

    def ab_to_c():
        vals['c'] = vals['a'] + vals['b']
    eng.push(set_a, write_vars=[a])
    eng.push(a_to_b, read_vars=[a], write_vars=[b])
    eng.push(ab_to_c, read_vars=[a, b], write_vars=[c])
    eng.wait_for_var(c)
    assert vals == {'a': 2, 'b': 20, 'c': 22}


def test_engine_exception_propagates_to_dependents_and_waits():
    eng = runtime.Engine(num_workers=2)
    a, b, other = eng.new_var(), eng.new_var(), eng.new_var()
    ran = []

    def boom():
        raise ValueError('bad op')
    eng.push(boom, write_vars=[a])
    eng.push(lambda: ran.append('dependent'), read_vars=[a], write_vars=[b])
    eng.push(lambda: ran.append('independent'), write_vars=[other])
    eng.wait_for_var(other)                      # unrelated work is not poisoned
    assert 'independent' in ran
    with pytest.raises(Exception) as ei:
        eng.wait_for_var(b)                      # the error travels var -> op -> var
    assert 'bad op' in str(ei.value)
    assert 'dependent' not in ran
    # the engine keeps working, and a failure that a wait has raised is not reported a second time
    eng.push(lambda: ran.append('later'), write_vars=[other])
    eng.wait_all()
    assert 'later' in ran
    # a failure that no wait on a var has picked up is reported by wait_all, once
    eng.push(boom, write_vars=[a])
    with pytest.raises(ValueError):
        eng.wait_all()
    eng.wait_all()


def test_engine_priority_and_naive_mode():
    eng = runtime.Engine(num_workers=1, num_priority_workers=1)
    gate, order = eng.new_var(), []
    block = threading.Event()
    eng.push(block.wait, write_vars=[gate])
    for i, pr in enumerate([0, 5, 1, 9]):
        eng.push((lambda i=i: order.append(i)), read_vars=[gate], priority=pr)
    block.set()
    eng.wait_all()
    assert sorted(order) == [0, 1, 2, 3]
    naive = runtime.Engine(naive=True)
    seen = []
    v = naive.new_var()
    naive.push(lambda: seen.append(threading.get_ident()), write_vars=[v])
    assert seen == [threading.get_ident()]       # runs inline on the pushing thread


def test_async_error_surfaces_at_waitall():
    from mxnet_b200 import engine
    engine.push_async_error(mx.MXNetError('late failure'))
    with pytest.raises(mx.MXNetError):
        nd.waitall()
    nd.waitall()                                  # reported once


def test_invalid_op_arguments_raise_mxnet_error():
    with pytest.raises(mx.MXNetError):
        nd.dot(nd.ones((2, 3)), nd.ones((4, 5)))
    with pytest.raises(mx.MXNetError):
        nd.Convolution(nd.ones((1, 3, 5, 5)), nd.ones((4, 2, 3, 3)), kernel=(3, 3), num_filter=4, no_bias=True)


def test_storage_pool_rounding_and_reuse():
    pool = runtime.Pool(1, 0, strategy='Round', page=4096)          # device type 1: host memory
    assert pool.round_size(1) >= 1 and pool.round_size(5000) >= 5000
    p1, r1 = pool.alloc(5000)
    pool.free(p1, r1)
    p2, r2 = pool.alloc(4500)
    assert p2 == p1, 'a freed block of the same bucket is reused'
    st = pool.stats()
    assert st['hits'] >= 1 and st['misses'] >= 1 and st['used'] >= 4500 and st['peak'] >= st['used']
    pool.free(p2, r2)
    assert pool.stats()['pooled'] > 0
    pool.release_all()
    assert pool.stats()['pooled'] == 0
    unpooled = runtime.Pool(1, 0, strategy='Unpooled')
    p, r = unpooled.alloc(100)
    unpooled.free(p, r)
    assert unpooled.stats()['pooled'] == 0


def test_profiler_chrome_trace_and_aggregate(tmp_path):
    f = str(tmp_path / 'profile.json')
    profiler.set_config(profile_all=True, aggregate_stats=True, filename=f)
    profiler.set_state('run')
    a = nd.ones((64, 64))
    for _ in range(3):
        b = nd.dot(a, a)
        b = nd.relu(b)
    dom = profiler.Domain('mydomain')
    with dom.new_task('stage'):
        nd.sum(b).asscalar()
    cnt = dom.new_counter('items', 5)
    cnt += 3
    dom.new_marker('here').mark('process')
    nd.waitall()
    profiler.set_state('stop')
    table = profiler.dumps(reset=False)
    assert 'dot' in table and 'relu' in table
    stats = json.loads(profiler.dumps(format='json'))
    names = json.dumps(stats)
    assert 'dot' in names
    profiler.dump()
    trace = json.load(open(f))
    events = trace['traceEvents']
    assert any(e.get('name') == 'dot' for e in events)
    assert any(e.get('name') == 'stage' for e in events)
    assert any(e.get('ph') == 'C' and e.get('name') == 'items' for e in events)
    assert all('ts' in e for e in events if e.get('ph') in ('X', 'B', 'E', 'C', 'i'))


def test_profiler_pause_resume_and_scope():
    profiler.set_config(profile_all=True, aggregate_stats=True, filename=os.devnull)
    profiler.set_state('run')
    profiler.dumps(reset=True)
    profiler.pause()
    nd.exp(nd.ones((4,)))
    profiler.resume()
    with profiler.scope('blockA:'):
        nd.log(nd.ones((4,)))
    profiler.set_state('stop')
    table = profiler.dumps(reset=True)
    assert 'log' in table and 'exp' not in table


def test_feature_flags_and_env_registry():
    feats = mx.runtime.Features()
    assert feats.is_enabled('CUDA') in (True, False) and 'CUDA' in feats
    assert isinstance(mx.runtime.feature_list(), list)
    from mxnet_b200 import env
    assert env.get('MXNET_KVSTORE_WAIT_MS') == 20000
    with env.scope('MXNET_KVSTORE_WAIT_MS', 5):
        assert env.get('MXNET_KVSTORE_WAIT_MS') == 5
    assert 'MXNET_ENGINE_TYPE' in env.describe()


def test_environment_variable_document_is_current():
    """docs/env_var.md is generated from the flag registry: regenerate with `python -m mxnet_b200.env > docs/env_var.md`."""
    import os
    from mxnet_b200 import env
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with open(os.path.join(root, 'docs', 'env_var.md')) as f:
        assert f.read() == env.markdown()


def test_clock_sampler_against_a_fake_nvml(monkeypatch):
    """The sampler that bench.py runs during the timed region: median SM clock under load, maximum clock and the
    throttle reasons seen, read through NVML (here a stand-in module; nothing is ever written to the device)."""
    import sys
    import time
    import types
    from mxnet_b200.utils import ClockSampler
    fake = types.ModuleType('pynvml')
    fake.NVML_CLOCK_SM = 1
    fake.nvmlClocksThrottleReasonSwPowerCap = 0x4
    fake.nvmlClocksThrottleReasonHwSlowdown = 0x8
    fake.nvmlClocksThrottleReasonSwThermalSlowdown = 0x20
    fake.nvmlClocksThrottleReasonHwThermalSlowdown = 0x40
    calls = {'n': 0, 'writes': 0}
    clocks = [1965, 1400, 1350, 1300, 1320]
    fake.nvmlInit = lambda: None
    fake.nvmlDeviceGetHandleByIndex = lambda i: ('gpu', i)
    fake.nvmlDeviceGetMaxClockInfo = lambda h, kind: 1965

    def clock(h, kind):
        calls['n'] += 1
        return clocks[min(calls['n'] - 1, len(clocks) - 1)]
    fake.nvmlDeviceGetClockInfo = clock
    fake.nvmlDeviceGetUtilizationRates = lambda h: types.SimpleNamespace(gpu=10 if calls['n'] <= 1 else 99)
    fake.nvmlDeviceGetCurrentClocksThrottleReasons = lambda h: 0x4 if calls['n'] >= 3 else 0
    monkeypatch.setitem(sys.modules, 'pynvml', fake)
    sampler = ClockSampler(0, interval=0.01).start()
    deadline = time.time() + 5
    while calls['n'] < 6 and time.time() < deadline:
        time.sleep(0.01)
    res = sampler.stop()
    assert res['sm_max_mhz'] == 1965 and res['reasons'] == ['sw_power_cap'] and res['samples'] >= 5
    assert 1300 <= res['sm_mhz'] <= 1400                       # the idle 1965 MHz sample is not part of the loaded median
    # without NVML the sampler degrades to "no data" instead of failing the benchmark
    broken = types.ModuleType('pynvml')
    monkeypatch.setitem(sys.modules, 'pynvml', broken)
    assert ClockSampler(0).start().stop()['sm_mhz'] is None

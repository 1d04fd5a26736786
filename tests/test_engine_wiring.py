"""The native runtime in the execution path: host tasks ordered by array variables, exceptions carried to the sync
points (tests/python/unittest/test_exc_handling.py:30-150 checks the same contract), engine-backed checkpoint writes and
prefetching, shared-memory batches of data-loader workers, pooled pinned staging buffers."""
import glob
import os
import time

import numpy as np
import pytest
import torch

import mxnet_b200 as mx
from mxnet_b200 import engine, env, nd


def test_exception_of_a_host_task_surfaces_at_the_sync_point_of_the_array_it_writes():
    a = nd.zeros((4,))
    b = nd.ones((4,))

    def fail():
        time.sleep(0.05)
        raise ValueError('boom in a host task')
    engine.push(fail, writes=[a], name='failing')          # returns at once: nothing is raised here
    # a task that depends on the failed array does not run and passes the failure on to what it writes
    ran = []
    engine.push(lambda: ran.append(1), reads=[a], writes=[b], name='dependent')
    c = nd.ones((4,))
    np.testing.assert_array_equal(c.asnumpy(), np.ones(4))  # an unrelated array is not affected
    with pytest.raises(ValueError, match='boom in a host task'):
        a.wait_to_read()
    with pytest.raises(ValueError):
        b.asnumpy()
    assert ran == []
    a.wait_to_read()                                        # a failure is reported once
    nd.waitall()


def test_save_waits_for_the_host_task_that_writes_the_array(tmp_path):
    a = nd.zeros((1000,))

    def slow_fill():
        time.sleep(0.3)
        a._data.fill_(7.0)
    engine.push(slow_fill, writes=[a], name='slow_fill')
    fname = str(tmp_path / 'a.params')
    t0 = time.time()
    nd.save(fname, {'a': a})                                # ordered after slow_fill by the engine
    assert time.time() - t0 > 0.2
    np.testing.assert_array_equal(nd.load(fname)['a'].asnumpy(), np.full(1000, 7.0, dtype='float32'))
    # a later writer waits for a save that is reading the array
    order = []
    engine.push(lambda: (time.sleep(0.2), order.append('read')), reads=[a], name='reader')
    engine.push(lambda: order.append('write'), writes=[a], name='writer')
    a.wait_to_read()
    assert order == ['read', 'write']


def test_save_raises_the_writers_error(tmp_path):
    with pytest.raises(mx.MXNetError):
        nd.save(str(tmp_path / 'no_such_dir' / 'x.params'), [nd.ones((2,))])


def test_naive_engine_runs_and_raises_inside_push():
    a = nd.zeros((2,))
    with env.scope('MXNET_ENGINE_TYPE', 'NaiveEngine'):
        assert engine.is_naive()
        done = []
        engine.push(lambda: done.append(1), writes=[a])
        assert done == [1]
        with pytest.raises(KeyError):
            engine.push(lambda: {}['missing'], writes=[a])
    assert not engine.is_naive()


class _Failing(mx.io.DataIter):
    def __init__(self, fail_at):
        super().__init__(batch_size=2)
        self.n, self.fail_at = 0, fail_at
        self.provide_data = [mx.io.DataDesc('data', (2, 3), 'float32')]
        self.provide_label = [mx.io.DataDesc('label', (2,), 'float32')]

    def reset(self):
        self.n = 0

    def next(self):
        self.n += 1
        if self.n == self.fail_at:
            raise RuntimeError('decoder failed on batch %d' % self.n)
        if self.n > 5:
            raise StopIteration
        return mx.io.DataBatch([nd.full((2, 3), self.n)], [nd.zeros((2,))], pad=0)


def test_prefetching_iter_raises_what_the_inner_iterator_raised():
    it = mx.io.PrefetchingIter(_Failing(fail_at=3))
    assert float(it.next().data[0].asnumpy()[0, 0]) == 1.0
    assert float(it.next().data[0].asnumpy()[0, 0]) == 2.0
    with pytest.raises(RuntimeError, match='decoder failed on batch 3'):
        it.next()
    ok = mx.io.PrefetchingIter(_Failing(fail_at=99))
    assert [float(b.data[0].asnumpy()[0, 0]) for b in ok] == [1.0, 2.0, 3.0, 4.0, 5.0]
    ok.reset()
    assert len(list(ok)) == 5


def test_dataloader_workers_hand_batches_over_in_shared_memory():
    from mxnet_b200.gluon.data import ArrayDataset, DataLoader, dataloader as dl
    x = np.random.rand(48, 3, 16, 16).astype('float32')
    y = np.arange(48).astype('float32')
    before = dl.shm_batches
    loader = DataLoader(ArrayDataset(x, y), batch_size=8, num_workers=2)
    seen = 0
    for xb, yb in loader:
        first = int(yb.asnumpy()[0])
        np.testing.assert_array_equal(xb.asnumpy(), x[first:first + 8])
        seen += 1
    assert seen == 6 and dl.shm_batches - before == 6          # the image batches came as segments, none by pickle
    del xb, yb, loader
    import gc
    gc.collect()
    assert glob.glob('/dev/shm/mxb_dl_%d_*' % os.getpid()) == []


@pytest.mark.gpu
def test_pinned_pool_stages_batches_and_the_copy_in_stream_delivers_them():
    from mxnet_b200.gluon.data import ArrayDataset, DataLoader
    x = np.random.rand(64, 3, 32, 32).astype('float32')
    loader = DataLoader(ArrayDataset(x, np.arange(64).astype('float32')), batch_size=16, num_workers=0, pin_memory=True,
                        thread_pool=True)
    pool = engine.pinned_pool()
    for epoch in range(2):
        for xb, yb in loader:
            assert xb._data.is_pinned()
            first = int(yb.asnumpy()[0])
            on_gpu = xb.as_in_context(mx.gpu(0))
            np.testing.assert_array_equal(on_gpu.asnumpy(), x[first:first + 16])
            del xb, on_gpu
    stats = pool.stats()
    assert stats['hits'] > 0                      # buffers of earlier batches were reused, not allocated again


@pytest.mark.gpu
def test_naive_engine_synchronises_after_every_gpu_operator():
    a = nd.ones((1 << 22,), ctx=mx.gpu(0))
    with env.scope('MXNET_ENGINE_TYPE', 'NaiveEngine'):
        b = a * 2 + 1
        assert torch.cuda.current_stream().query()          # nothing is pending once the operator call has returned
    np.testing.assert_array_equal(b.asnumpy()[:3], [3, 3, 3])


def test_per_device_policy_keeps_workers_for_urgent_operations():
    """With every ordinary worker busy, a positive-priority operation still runs at once on the reserved workers; the
    pooled policy (one queue) makes it wait."""
    import threading
    from mxnet_b200.csrc import runtime
    for kind, expect_early in (('ThreadedEnginePerDevice', True), ('ThreadedEngine', False)):
        eng = runtime.Engine(kind=kind, num_workers=2, num_priority_workers=1)
        release = threading.Event()
        n_block = 2 if expect_early else 3                      # occupy every worker that ordinary work may use
        for _ in range(n_block):
            eng.push(release.wait, write_vars=[eng.new_var()])
        time.sleep(0.05)
        ran = threading.Event()
        eng.push(ran.set, write_vars=[eng.new_var()], priority=5)
        assert ran.wait(0.5) == expect_early, kind
        release.set()
        eng.wait_all()
        assert ran.is_set()


def test_forked_child_gets_a_fresh_engine():
    """Worker threads do not survive fork(): the child drops the parent's engine and builds its own on first use."""
    a = nd.zeros((3,))
    engine.push(lambda: a._data.fill_(1.0), writes=[a])
    a.wait_to_read()
    pid = os.fork()
    if pid == 0:
        code = 1
        try:
            b = nd.zeros((3,))
            engine.push(lambda: b._data.fill_(5.0), writes=[b])
            code = 0 if float(b.asnumpy().sum()) == 15.0 else 2
        finally:
            os._exit(code)
    _, status = os.waitpid(pid, 0)
    assert os.WIFEXITED(status) and os.WEXITSTATUS(status) == 0
    engine.push(lambda: a._data.fill_(2.0), writes=[a])          # the parent's engine is untouched
    assert float(a.asnumpy().sum()) == 6.0

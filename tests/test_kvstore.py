"""KVStore semantics (reference: tests/python/unittest/test_kvstore.py, test_kvstore_custom.py;
tests/nightly/dist_sync_kvstore.py for the multi-process part, here with gloo CPU ranks)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import mxnet_b200 as mx
from mxnet_b200 import kv, nd
from mxnet_b200.test_utils import assert_almost_equal, same

SHAPE = (4, 4)
KEYS = [5, 7, 11]
STR_KEYS = ['b', 'c', 'd']
HERE = os.path.dirname(os.path.abspath(__file__))


def _init(kind='local', keys=KEYS):
    store = kv.create(kind)
    store.init(3, nd.zeros(SHAPE))
    store.init(keys, [nd.zeros(SHAPE)] * len(keys))
    return store


@pytest.mark.parametrize('kind', ['local', 'device'])
def test_single_kv_pair_and_list(kind):
    store = _init(kind)
    store.push(3, nd.ones(SHAPE))
    out = nd.empty(SHAPE)
    store.pull(3, out=out)
    assert same(out.asnumpy(), np.ones(SHAPE, 'float32'))
    store.push(KEYS, [nd.ones(SHAPE) * 4] * len(KEYS))
    outs = [nd.empty(SHAPE) for _ in KEYS]
    store.pull(KEYS, out=outs)
    for o in outs:
        assert same(o.asnumpy(), np.full(SHAPE, 4, 'float32'))


def test_aggregation_over_devices():
    store = _init('device')
    devs = [mx.cpu(i) for i in range(4)]
    store.push(3, [nd.ones(SHAPE, ctx=d) for d in devs])
    outs = [nd.empty(SHAPE, ctx=d) for d in devs]
    store.pull(3, out=outs)
    for o, d in zip(outs, devs):
        assert o.context == d and same(o.asnumpy(), np.full(SHAPE, 4, 'float32'))
    store.push(KEYS, [[nd.ones(SHAPE, ctx=d) * 2 for d in devs]] * len(KEYS))
    outs = [[nd.empty(SHAPE, ctx=d) for d in devs] for _ in KEYS]
    store.pull(KEYS, out=outs)
    for group in outs:
        for o in group:
            assert same(o.asnumpy(), np.full(SHAPE, 8, 'float32'))


def test_pushpull_in_place_and_out():
    store = _init('device')
    vals = [nd.ones(SHAPE, ctx=mx.cpu(i)) * (i + 1) for i in range(3)]
    store.pushpull(3, vals)                       # out defaults to value: an in-place all-reduce
    for v in vals:
        assert same(v.asnumpy(), np.full(SHAPE, 6, 'float32'))
    out = nd.empty(SHAPE)
    store.pushpull(5, [nd.ones(SHAPE), nd.ones(SHAPE)], out=out)
    assert same(out.asnumpy(), np.full(SHAPE, 2, 'float32'))


def test_updater_runs_on_push():
    store = _init()
    calls = []

    def updater(key, recv, stored):
        calls.append(key)
        stored += recv * 2
    store._set_updater(updater)
    store.push(3, [nd.ones(SHAPE), nd.ones(SHAPE)])
    out = nd.empty(SHAPE)
    store.pull(3, out=out)
    assert same(out.asnumpy(), np.full(SHAPE, 4, 'float32')) and calls == [3]
    store.push(3, nd.ones(SHAPE))
    store.pull(3, out=out)
    assert same(out.asnumpy(), np.full(SHAPE, 6, 'float32'))


def test_set_optimizer_applies_update_rule():
    store = kv.create('local')
    store.init(0, nd.ones(SHAPE))
    store.set_optimizer(mx.optimizer.create('sgd', learning_rate=0.5))
    store.push(0, nd.ones(SHAPE))
    out = nd.empty(SHAPE)
    store.pull(0, out=out)
    assert_almost_equal(out.asnumpy(), np.full(SHAPE, 0.5, 'float32'))


def test_string_keys_and_mixing_is_rejected():
    store = kv.create('local')
    store.init(STR_KEYS, [nd.zeros(SHAPE)] * 3)
    store.push('b', nd.ones(SHAPE))
    out = nd.empty(SHAPE)
    store.pull('b', out=out)
    assert same(out.asnumpy(), np.ones(SHAPE, 'float32'))
    with pytest.raises(Exception):
        store.init(3, nd.zeros(SHAPE))                # int key after str keys
    with pytest.raises(Exception):
        store.init('b', nd.zeros(SHAPE))              # duplicate init


def test_broadcast_and_properties():
    store = kv.create('device')
    outs = [nd.empty(SHAPE, ctx=mx.cpu(i)) for i in range(2)]
    store.broadcast(9, nd.ones(SHAPE) * 3, out=outs)
    for o in outs:
        assert same(o.asnumpy(), np.full(SHAPE, 3, 'float32'))
    assert store.type == 'device' and store.rank == 0 and store.num_workers == 1
    assert kv.KVStore.is_capable('optimizer')
    assert store.get_num_dead_node(0) == 0


def test_row_sparse_pull():
    store = kv.create('local')
    w = np.arange(24, dtype='float32').reshape(6, 4)
    store.init('w', nd.array(w).tostype('row_sparse'))
    out = nd.sparse.zeros('row_sparse', (6, 4))
    store.row_sparse_pull('w', out=out, row_ids=nd.array([1, 4, 1]))
    dense = out.tostype('default').asnumpy()
    expect = np.zeros_like(w)
    expect[[1, 4]] = w[[1, 4]]
    assert same(dense, expect)
    assert store.rows_pulled == 2          # the two distinct rows were gathered and moved, not the whole table


def test_gradient_compression_2bit_residual():
    store = kv.create('device')
    store.set_gradient_compression({'type': '2bit', 'threshold': 0.5})
    store.init(0, nd.zeros((8,)))
    g = nd.array([0.3, 0.6, -0.7, 0.1, 0.0, 1.4, -0.2, 0.45])
    out = nd.empty((8,))
    store.pushpull(0, [g, g], out=out)
    # every value is quantised to {-0.5, 0, 0.5} per device; the remainder stays in the residual
    assert same(out.asnumpy(), np.array([0, 1, -1, 0, 0, 1, 0, 0], 'float32'))
    store.pushpull(0, [g, g], out=out)
    # second round: residual + new gradient = 0.6, 0.7, -0.9, 0.2, 0, 2.3, -0.4, 0.9
    assert same(out.asnumpy(), np.array([1, 1, -1, 0, 0, 1, 0, 1], 'float32'))
    with pytest.raises(Exception):
        kv.create('nccl').set_gradient_compression({'type': '2bit', 'threshold': 0.5})


def test_optimizer_states_round_trip(tmp_path):
    store = kv.create('local')
    store.init(0, nd.ones(SHAPE))
    store.set_optimizer(mx.optimizer.create('adam', learning_rate=0.1))
    store.push(0, nd.ones(SHAPE))
    f = str(tmp_path / 'kv.states')
    store.save_optimizer_states(f, dump_optimizer=True)
    store2 = kv.create('local')
    store2.init(0, nd.ones(SHAPE))
    store2.set_optimizer(mx.optimizer.create('adam', learning_rate=0.1))
    store2.load_optimizer_states(f)
    assert 0 in store2._updater.states


def test_teststore_and_custom_registration():
    store = kv.create('teststore')
    assert store.type == 'teststore' and not store.is_capable('optimizer')
    vals = [nd.ones(SHAPE), nd.ones(SHAPE) * 2]
    store.pushpull('k', vals)
    assert same(vals[0].asnumpy(), np.full(SHAPE, 3, 'float32'))

    @kv.KVStoreBase.register
    class MyStore(kv.KVStoreBase):
        def broadcast(self, key, value, out, priority=0):
            pass

        def pushpull(self, key, value, out=None, priority=0):
            pass

        @staticmethod
        def is_capable(capability):
            return False

        @property
        def type(self):
            return 'mystore'

        @property
        def rank(self):
            return 0

        @property
        def num_workers(self):
            return 1
    assert kv.create('mystore').type == 'mystore'


# ---------------------------------------------------------------------------------------- multi-process
def _torchrun(script, nproc, port, args=(), timeout=180):
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node', str(nproc),
           '--master-addr', '127.0.0.1', '--master-port', str(port), os.path.join(HERE, 'dist', script)] + list(args)
    env = dict(os.environ, MXB_TEST_BACKEND='gloo', CUDA_VISIBLE_DEVICES='')
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)


@pytest.mark.integration
def test_dist_sync_kvstore_over_gloo():
    r = _torchrun('dist_kvstore_worker.py', 3, 29641)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    rep = json.loads([l for l in r.stdout.splitlines() if l.startswith('REPORT ')][-1][7:])
    assert rep == {'world': 3, 'pushpull': True, 'broadcast': True, 'trainer_identical': True, 'optimizer_on_store': True,
                   'compressed_wire': True}


@pytest.mark.integration
def test_dist_async_applies_every_push_on_arrival():
    """``dist_async`` against the reference's server semantics (kvstore_dist_server.h ApplyUpdates, async branch): a lone
    push completes without the other workers, every push is one server-side update, pulls see the server's value, and a
    Trainer whose ranks take different numbers of steps does not block."""
    r = _torchrun('dist_async_worker.py', 3, 29647)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    rep = json.loads([l for l in r.stdout.splitlines() if l.startswith('REPORT ')][-1][7:])
    assert rep['world'] == 3 and rep['lone_push_applied'] and rep['lone_push_seconds'] < 5.0
    assert rep['all_pushes_applied'] and rep['pull_same_everywhere']
    assert rep['server_updates'] == 1 + 3 * 3
    assert rep['uneven_steps_completed'] == [2, 3, 4] and rep['update_on_kvstore']


def test_parameter_server_sync_mode_merges_a_round_before_applying():
    """The server's sync mode: pushes of one round are summed, the updater runs once when the last worker has pushed, and
    only then are the round's requests answered (kvstore_dist_server.h:349-404); without an updater the merged value
    replaces the stored one."""
    import threading
    import torch
    import mxnet_b200 as mx
    from mxnet_b200.kvstore.server import ParameterServer, ServerClient
    server = ParameterServer(num_workers=3, sync_mode=True)
    clients = [ServerClient(server.address) for _ in range(3)]
    clients[0].init('k', torch.zeros(4))
    clients[0].set_optimizer(mx.optimizer.create('sgd', learning_rate=1.0, rescale_grad=1.0))
    done, results = [], [None] * 3

    def worker(i):
        results[i] = clients[i].push('k', torch.full((4,), float(i + 1)), pull=True)
        done.append(i)
    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    import time
    time.sleep(0.3)
    assert not done and server.pushes_applied == 0            # two of three pushed: the round is still open
    last = threading.Thread(target=worker, args=(2,))
    last.start()
    for t in threads + [last]:
        t.join(10)
    assert sorted(done) == [0, 1, 2] and server.pushes_applied == 1
    for r in results:
        assert torch.equal(r, torch.full((4,), -6.0))          # one SGD step on the merged gradient 1 + 2 + 3
    # async mode needs an updater
    async_server = ParameterServer(num_workers=1, sync_mode=False)
    c = ServerClient(async_server.address)
    c.init('k', torch.zeros(2))
    with pytest.raises(mx.MXNetError, match='Updater needs to be set for async mode'):
        c.push('k', torch.ones(2))
    for cl in clients + [c]:
        cl.close()
    server.stop()
    async_server.stop()


@pytest.mark.integration
def test_dead_rank_is_detected_by_heartbeat():
    r = _torchrun('dead_rank_worker.py', 3, 29643)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    rep = json.loads([l for l in r.stdout.splitlines() if l.startswith('REPORT ')][-1][7:])
    assert rep['dead_before'] == 0 and rep['dead_after'] == 1

"""Worker of the multi-process KVStore test (CPU ranks over gloo): dist_sync push/pull, broadcast and a
Trainer whose replicas stay identical."""
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import mxnet_b200 as mx                                    # noqa: E402
from mxnet_b200 import autograd, gluon, kv, nd             # noqa: E402
from mxnet_b200.gluon import nn                            # noqa: E402
from mxnet_b200.parallel import dist                       # noqa: E402


def main():
    dist.ensure_initialized(os.environ.get('MXB_TEST_BACKEND', 'gloo'))
    store = kv.create('dist_sync')
    rank, world = store.rank, store.num_workers
    rep = {'world': world}
    # pushpull: every rank contributes rank+1
    store.init(1000, nd.zeros((5,)))
    out = nd.empty((5,))
    store.pushpull(1000, nd.ones((5,)) * (rank + 1), out=out)
    rep['pushpull'] = bool(np.allclose(out.asnumpy(), world * (world + 1) / 2))
    # broadcast: rank 0's value wins
    val = nd.ones((3,)) * (10 if rank == 0 else -1)
    outs = nd.empty((3,))
    store.broadcast(1001, val, out=outs)
    rep['broadcast'] = bool(np.allclose(outs.asnumpy(), 10))
    # Trainer over the store: different data per rank, identical weights afterwards
    mx.random.seed(100 + rank)              # different initial weights: the broadcast must fix that
    net = nn.Dense(3, in_units=4)
    net.initialize()
    tr = gluon.Trainer(net.collect_params(), 'sgd', {'learning_rate': 0.1, 'momentum': 0.9}, kvstore=store,
                       update_on_kvstore=False)
    rng = np.random.RandomState(rank)
    for _ in range(3):
        x = nd.array(rng.randn(2, 4))
        with autograd.record():
            l = net(x).sum()
        l.backward()
        tr.step(2 * world)
    w = net.weight.data().asnumpy()
    gathered = dist.all_gather_object(w)
    rep['trainer_identical'] = all(np.array_equal(gathered[0], g) for g in gathered)
    # optimizer on the store: push gradients, the store applies SGD, pull gives the new weight everywhere
    store2 = kv.create('dist_sync')
    store2.init('w', nd.ones((2,)))
    store2.set_optimizer(mx.optimizer.create('sgd', learning_rate=0.1, rescale_grad=1.0 / world))
    store2.push('w', nd.ones((2,)) * (rank + 1))
    o2 = nd.empty((2,))
    store2.pull('w', out=o2)
    rep['optimizer_on_store'] = bool(np.allclose(o2.asnumpy(), 1 - 0.1 * (world + 1) / 2))
    # gradient compression between workers: the packed 2-bit codes travel (all-gather of the words), every rank expands
    # and sums them; 64 values = 4 words per rank instead of 256 bytes
    store3 = kv.create('dist_sync')
    store3.set_gradient_compression({'type': '2bit', 'threshold': 0.5})
    store3.init('g', nd.zeros((64,)))
    g = nd.array(np.where(np.arange(64) % 3 == rank % 3, 0.75, -0.1).astype('float32'))
    o3 = nd.empty((64,))
    store3.pushpull('g', g, out=o3)
    expect = np.zeros(64, 'float32')
    for r in range(world):
        expect += np.where(np.arange(64) % 3 == r % 3, 0.5, 0.0)
    rep['compressed_wire'] = bool(np.array_equal(o3.asnumpy(), expect)) and store3.wire_bytes == 4 * 4 * (world - 1)
    store.barrier()
    if rank == 0:
        print('REPORT ' + json.dumps(rep))
    dist.destroy()


if __name__ == '__main__':
    main()

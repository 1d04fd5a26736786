"""Worker of the ``dist_async`` test (CPU ranks over gloo): every push is applied by the server on arrival, no rank waits
for another, and a pull returns the server's current value."""
import json
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import mxnet_b200 as mx                                    # noqa: E402
from mxnet_b200 import autograd, gluon, kv, nd             # noqa: E402
from mxnet_b200.gluon import nn                            # noqa: E402
from mxnet_b200.parallel import dist                       # noqa: E402


def main():
    dist.ensure_initialized(os.environ.get('MXB_TEST_BACKEND', 'gloo'))
    store = kv.create('dist_async')
    rank, world = store.rank, store.num_workers
    rep = {'world': world}
    store.init('w', nd.ones((4,)) * (5 if rank == 0 else -1))
    store.set_optimizer(mx.optimizer.create('sgd', learning_rate=0.5, rescale_grad=1.0))
    dist.barrier()
    # 1. asynchrony: ONLY rank 0 pushes, nobody else takes part, and the push returns; in sync mode it could not complete
    if rank == 0:
        t0 = time.time()
        store.push('w', nd.ones((4,)))
        out = nd.empty((4,))
        store.pull('w', out=out)
        rep['lone_push_seconds'] = time.time() - t0
        first = float(out.asnumpy()[0])
        rep['lone_push_applied'] = first in (4.5, -1.5)       # initial value of whichever rank reached the server first
        rep['base'] = first + 0.5
    dist.barrier()
    # 2. every rank pushes `rank + 1` three times, unsynchronised: the server applies 3 * world updates one by one
    for _ in range(3):
        store.push('w', nd.ones((4,)) * (rank + 1))
    dist.barrier()
    out = nd.empty((4,))
    store.pull('w', out=out)
    values = dist.all_gather_object(float(out.asnumpy()[0]))
    if rank == 0:
        expect = rep['base'] - 0.5 - 0.5 * 3 * world * (world + 1) / 2
        rep['all_pushes_applied'] = bool(np.isclose(values[0], expect))
        rep['pull_same_everywhere'] = all(v == values[0] for v in values)
        rep['server_updates'] = store._client.stats()['pushes_applied']
    # 3. a Trainer on the store: the optimizer runs on the server, workers push gradients and pull weights at their own pace
    mx.random.seed(3)
    net = nn.Dense(2, in_units=3)
    net.initialize()
    tr = gluon.Trainer(net.collect_params(), 'sgd', {'learning_rate': 0.05}, kvstore=kv.create('dist_async'))
    rng = np.random.RandomState(rank)
    for _ in range(2 + rank):                                  # ranks take different numbers of steps: nothing blocks
        x = nd.array(rng.randn(4, 3))
        with autograd.record():
            l = (net(x) ** 2).sum()
        l.backward()
        tr.step(4)
    rep_steps = dist.all_gather_object(2 + rank)
    dist.barrier()
    if rank == 0:
        rep['uneven_steps_completed'] = rep_steps
        rep['update_on_kvstore'] = bool(tr._update_on_kvstore)
        print('REPORT ' + json.dumps(rep), flush=True)
    dist.barrier()
    dist.destroy()


if __name__ == '__main__':
    main()

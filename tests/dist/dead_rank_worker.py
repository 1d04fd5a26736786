"""Worker of the failure-detection test (CPU ranks over gloo).  The failure is made on the host: the last
rank stops its heartbeat and leaves between steps; the others see it through ``get_num_dead_node``."""
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from mxnet_b200 import kv, nd                      # noqa: E402
from mxnet_b200.parallel import dist               # noqa: E402


def main():
    dist.ensure_initialized(os.environ.get('MXB_TEST_BACKEND', 'gloo'), timeout_s=30)
    store = kv.create('dist_sync')
    rank, world = store.rank, store.num_workers
    dist.start_heartbeat(interval=0.2)
    store.init('g', nd.zeros((2,)))
    out = nd.empty((2,))
    store.pushpull('g', nd.ones((2,)), out=out)         # one healthy step with everybody
    time.sleep(0.6)
    before = store.get_num_dead_node(0, timeout=2)
    store.barrier()
    if rank == world - 1:
        dist.stop_heartbeat()                             # this rank "dies": no collective is in flight
        time.sleep(4.0)
        os._exit(0)
    time.sleep(3.0)
    after = store.get_num_dead_node(0, timeout=2)       # learnt on the host, before any further collective
    if rank == 0:
        print('REPORT ' + json.dumps({'dead_before': before, 'dead_after': after}))
        sys.stdout.flush()
    dist.stop_heartbeat()
    os._exit(0)


if __name__ == '__main__':
    main()

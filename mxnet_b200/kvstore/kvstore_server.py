"""Server role of the distributed store (``python/mxnet/kvstore/kvstore_server.py``).

The reference runs separate server processes that aggregate pushes (``kvstore_dist_server.h``).
Here aggregation is a collective among the worker ranks, so a process started with the server or
scheduler role has nothing to serve: it joins the rendezvous barrier and returns."""
import os


class KVStoreServer(object):
    def __init__(self, kvstore):
        self.kvstore = kvstore

    def run(self):
        return


def _init_kvstore_server_module():
    role = os.environ.get('DMLC_ROLE', 'worker')
    if role in ('server', 'scheduler'):
        KVStoreServer(None).run()

"""Test configuration: markers, seeding, and a module-level waitall so asynchronous failures surface
in the module that caused them (the reference's root ``conftest.py:62-230`` does the same)."""
import os
import random
import sys
import zlib

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (run with -m gpu on a B200)')
    config.addinivalue_line('markers', 'serial: must not run concurrently with other tests')
    config.addinivalue_line('markers', 'integration: longer end-to-end test')
    config.addinivalue_line('markers', 'seed: fixed seed for this test')


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason='no CUDA device')
    for item in items:
        if 'gpu' in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _seed_everything(request):
    """Seed every RNG per test; MXNET_TEST_SEED replays a failing seed."""
    import mxnet_b200 as mx
    marker = request.node.get_closest_marker('seed')
    env_seed = os.environ.get('MXNET_TEST_SEED')
    if marker is not None:
        seed = marker.args[0]
    elif env_seed:
        seed = int(env_seed)
    else:
        # crc32 of the node id: the same seed in every process (hash() of a str is salted per interpreter)
        seed = zlib.crc32(request.node.nodeid.encode()) % (2 ** 31)
    np.random.seed(seed)
    random.seed(seed)
    mx.random.seed(seed)
    mx.util.reset_np()
    yield
    if hasattr(request.node, 'rep_call') and request.node.rep_call.failed:
        print('test failed with seed %d; rerun with MXNET_TEST_SEED=%d' % (seed, seed))


@pytest.hookimpl(tryfirst=True, hookwrapper=True)
def pytest_runtest_makereport(item, call):
    outcome = yield
    rep = outcome.get_result()
    setattr(item, 'rep_' + rep.when, rep)


@pytest.fixture(autouse=True, scope='module')
def _module_waitall():
    yield
    import mxnet_b200 as mx
    mx.nd.waitall()

"""Files written by the reference itself: a pre-V1 ``.params`` file and a ``-symbol.json`` of an older release (the data
files of its own test-suite, kept under tests/data) must load and run."""
import json
import os

import numpy as np

import mxnet_b200 as mx
from mxnet_b200 import nd

DATA = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'data')


def test_pre_v1_ndarray_file_loads():
    """tests/python/unittest/legacy_ndarray.v0 of the reference holds six copies of arange(128)."""
    arrays = nd.load(os.path.join(DATA, 'legacy_ndarray.v0'))
    assert isinstance(arrays, list) and len(arrays) == 6
    for a in arrays:
        assert a.shape == (128,) and a.dtype == np.float32
        np.testing.assert_array_equal(a.asnumpy(), np.arange(128, dtype='float32'))


def test_symbol_file_of_an_older_release_loads_infers_and_runs(tmp_path):
    path = os.path.join(DATA, 'legacy_model-symbol.json')
    raw = json.load(open(path))
    sym = mx.sym.load(path)
    assert sym.list_outputs() == ['softmax_output']
    args = sym.list_arguments()
    assert args[0] == 'data' and len(args) == sum(1 for n in raw['nodes'] if n['op'] == 'null')
    arg_shapes, out_shapes, aux_shapes = sym.infer_shape(data=(2, 3, 224, 224))
    assert out_shapes == [(2, 1000)] and all(s is not None for s in arg_shapes)
    # the graph survives a save / load cycle with the same operators in the same order
    again = str(tmp_path / 'again-symbol.json')
    sym.save(again)
    ops = lambda s: [n['op'] for n in json.loads(s.tojson())['nodes'] if n['op'] != 'null']
    assert ops(mx.sym.load(again)) == ops(sym) == [n['op'] for n in raw['nodes'] if n['op'] != 'null']
    # and runs: random parameters, a probability vector per image comes out
    rng = np.random.RandomState(0)
    feed = {n: nd.array(rng.uniform(-0.05, 0.05, s).astype('float32')) for n, s in zip(args, arg_shapes)}
    feed['data'] = nd.array(rng.rand(2, 3, 224, 224).astype('float32'))
    out = sym._bind(mx.cpu(), feed).forward(is_train=False)[0].asnumpy()
    assert out.shape == (2, 1000) and np.allclose(out.sum(1), 1.0, atol=1e-4)

"""contrib.text vocabulary / embeddings, ONNX export, post-training quantization, data loading helpers."""
import collections
import os

import numpy as np
import pytest

import mxnet_b200 as mx
from mxnet_b200 import gluon, nd
from mxnet_b200.contrib import text


def test_vocabulary_indexing_and_counting():
    counter = text.utils.count_tokens_from_str('a b b c c c\nd d d d', token_delim=' ', seq_delim='\n')
    assert counter == collections.Counter({'d': 4, 'c': 3, 'b': 2, 'a': 1})
    vocab = text.Vocabulary(counter, most_freq_count=None, min_freq=2, unknown_token='<unk>', reserved_tokens=['<pad>'])
    assert vocab.idx_to_token[:2] == ['<unk>', '<pad>']
    assert vocab.idx_to_token[2:] == ['d', 'c', 'b']             # by frequency; 'a' is below min_freq
    assert vocab.to_indices(['d', 'a', 'zzz']) == [2, 0, 0]
    assert vocab.to_tokens([3, 4]) == ['c', 'b']
    assert len(vocab) == 5


def test_custom_embedding_file(tmp_path):
    path = tmp_path / 'emb.txt'
    path.write_text('hello 0.1 0.2 0.3\nworld 1.0 2.0 3.0\n')
    emb = text.embedding.CustomEmbedding(str(path), elem_delim=' ')
    assert emb.vec_len == 3
    v = emb.get_vecs_by_tokens(['world', 'nope', 'hello']).asnumpy()
    np.testing.assert_allclose(v, [[1, 2, 3], [0, 0, 0], [0.1, 0.2, 0.3]], rtol=1e-6)
    emb.update_token_vectors('hello', nd.array([[9.0, 9.0, 9.0]]))
    np.testing.assert_allclose(emb.get_vecs_by_tokens('hello').asnumpy(), [9, 9, 9])
    # restricted to a vocabulary: its tokens, in its order; tokens the file does not have get the unknown vector
    vocab = text.Vocabulary(collections.Counter(['world', 'world', 'other', 'hello']), unknown_token='<unk>')
    sub = text.embedding.CustomEmbedding(str(path), elem_delim=' ', vocabulary=vocab)
    assert sub.idx_to_token == vocab.idx_to_token and len(sub) == len(vocab)
    np.testing.assert_allclose(sub.idx_to_vec.asnumpy()[sub.token_to_idx['world']], [1, 2, 3])
    np.testing.assert_allclose(sub.idx_to_vec.asnumpy()[sub.token_to_idx['other']], [0, 0, 0])
    comp = text.embedding.CompositeEmbedding(vocab, [emb, emb])
    assert comp.vec_len == 6 and comp.idx_to_vec.shape == (len(vocab), 6)


def test_onnx_export_writes_a_loadable_graph(tmp_path):
    data = mx.sym.var('data')
    net = mx.sym.FullyConnected(data, num_hidden=4, name='fc1')
    net = mx.sym.Activation(net, act_type='relu', name='relu1')
    net = mx.sym.softmax(mx.sym.FullyConnected(net, num_hidden=3, name='fc2'), name='sm')
    rng = np.random.RandomState(0)
    params = {'fc1_weight': nd.array(rng.randn(4, 5).astype('float32')), 'fc1_bias': nd.zeros((4,)),
              'fc2_weight': nd.array(rng.randn(3, 4).astype('float32')), 'fc2_bias': nd.zeros((3,))}
    out = str(tmp_path / 'net.onnx')
    mx.onnx.export_model(net, params, in_shapes=[(2, 5)], in_types=[np.float32], onnx_file_path=out)
    model = mx.onnx.backend.load_model(out)
    assert [n['op_type'] for n in model['graph']['node']] == ['Flatten', 'Gemm', 'Relu', 'Flatten', 'Gemm', 'Softmax']
    x = rng.randn(2, 5).astype('float32')
    ref = net._bind(mx.cpu(), dict(params, data=nd.array(x))).forward()[0].asnumpy()
    np.testing.assert_allclose(mx.onnx.run_model(out, {'data': x})[0], ref, rtol=1e-5, atol=1e-6)
    try:                                               # with the package at hand: its checker accepts the file too
        import onnx
    except ImportError:
        return
    onnx.checker.check_model(onnx.load(out))


def test_quantize_net_keeps_predictions_close():
    from mxnet_b200.contrib import quantization as q
    mx.random.seed(0)
    net = gluon.nn.HybridSequential()
    net.add(gluon.nn.Dense(32, activation='relu', in_units=16), gluon.nn.Dense(10, in_units=32))
    net.initialize(mx.init.Xavier())
    rng = np.random.RandomState(1)
    calib = [nd.array(rng.randn(8, 16).astype('float32')) for _ in range(4)]
    ref = net(calib[0]).asnumpy()
    qnet = q.quantize_net(net, quantized_dtype='int8', calib_mode='naive', calib_data=calib, num_calib_batches=4)
    out = qnet(calib[0]).asnumpy()
    assert out.shape == ref.shape
    assert np.abs(out - ref).max() < 0.25 * np.abs(ref).max() + 0.05


def test_dataloader_workers_and_samplers():
    x = np.arange(40, dtype='float32').reshape(20, 2)
    y = np.arange(20, dtype='float32')
    ds = gluon.data.ArrayDataset(x, y)
    seen = []
    for workers in (0, 2):
        loader = gluon.data.DataLoader(ds, batch_size=6, shuffle=False, last_batch='keep', num_workers=workers)
        batches = list(loader)
        assert [b[0].shape[0] for b in batches] == [6, 6, 6, 2]
        seen.append(np.concatenate([b[1].asnumpy() for b in batches]))
    np.testing.assert_array_equal(seen[0], y)
    np.testing.assert_array_equal(seen[1], y)
    assert len(list(gluon.data.DataLoader(ds, batch_size=6, last_batch='discard'))) == 3
    bs = gluon.data.BatchSampler(gluon.data.SequentialSampler(5), 2, 'rollover')
    assert list(bs) == [[0, 1], [2, 3]] and list(bs) == [[4, 0], [1, 2], [3, 4]]      # the left-over sample rolls over
    tds = ds.transform_first(lambda a: a * 2)
    np.testing.assert_array_equal(tds[3][0], x[3] * 2)
    sh = ds.shard(4, 1)
    assert len(sh) == 5


def test_ndarray_iter_pad_and_reset():
    x = np.arange(22, dtype='float32').reshape(11, 2)
    it = mx.io.NDArrayIter(x, np.arange(11), batch_size=4, last_batch_handle='pad')
    batches = list(it)
    assert len(batches) == 3 and batches[-1].pad == 1
    assert batches[0].data[0].shape == (4, 2)
    it.reset()
    assert len(list(it)) == 3
    it2 = mx.io.NDArrayIter(x, np.arange(11), batch_size=4, last_batch_handle='discard')
    assert len(list(it2)) == 2
    assert it.provide_data[0].shape == (4, 2)

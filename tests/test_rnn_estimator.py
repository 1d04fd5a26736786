"""Gluon RNN layers/cells and the Estimator training loop (reference: tests/python/unittest/test_gluon_rnn.py,
test_gluon_estimator.py, test_gluon_event_handler.py)."""
import os

import numpy as np
import pytest

import mxnet_b200 as mx
from mxnet_b200 import autograd, gluon, nd
from mxnet_b200.gluon import nn, rnn
from mxnet_b200.test_utils import assert_almost_equal


@pytest.mark.parametrize('cls,nstate', [(rnn.LSTM, 2), (rnn.GRU, 1), (rnn.RNN, 1)])
@pytest.mark.parametrize('bidirectional', [False, True])
def test_rnn_layers_shapes_and_grad(cls, nstate, bidirectional):
    layer = cls(8, num_layers=2, bidirectional=bidirectional, input_size=5)
    layer.initialize()
    x = nd.array(np.random.randn(6, 3, 5))
    d = 2 if bidirectional else 1
    out = layer(x)
    assert out.shape == (6, 3, 8 * d)
    states = layer.begin_state(3)
    assert len(states) == nstate and states[0].shape == (2 * d, 3, 8)
    with autograd.record():
        out, new_states = layer(x, states)
        loss = out.sum()
    loss.backward()
    assert len(new_states) == nstate and new_states[0].shape == (2 * d, 3, 8)
    assert any(float(abs(p.grad()).sum().asscalar()) > 0 for p in layer.collect_params().values())
    ntc = cls(8, layout='NTC', input_size=5)
    ntc.initialize()
    assert ntc(nd.array(np.random.randn(3, 6, 5))).shape == (3, 6, 8)


def test_lstm_layer_matches_cell_unroll():
    layer = rnn.LSTM(4, input_size=3)
    layer.initialize()
    cell = rnn.LSTMCell(4, input_size=3)
    cell.initialize()
    lp = layer.collect_params()
    names = {k.split('.')[-1].replace('l0_', ''): v for k, v in lp.items()}
    for k, p in cell.collect_params().items():
        p.set_data(names[k.split('.')[-1]].data())
    x = nd.array(np.random.randn(5, 2, 3))
    ref = layer(x).asnumpy()
    outs, _ = cell.unroll(5, x, layout='TNC', merge_outputs=True)
    assert_almost_equal(outs.asnumpy(), ref, rtol=1e-4, atol=1e-5)


def test_cells_sequential_residual_dropout_zoneout():
    stack = rnn.SequentialRNNCell()
    stack.add(rnn.LSTMCell(6, input_size=4))
    stack.add(rnn.ResidualCell(rnn.GRUCell(6, input_size=6)))
    stack.add(rnn.DropoutCell(0.0))
    stack.initialize()
    x = nd.array(np.random.randn(2, 4))
    states = stack.begin_state(batch_size=2)
    out, new_states = stack(x, states)
    assert out.shape == (2, 6) and len(new_states) == 3
    outs, _ = stack.unroll(3, nd.array(np.random.randn(2, 3, 4)), layout='NTC', merge_outputs=False)
    assert len(outs) == 3 and outs[0].shape == (2, 6)
    bi = rnn.BidirectionalCell(rnn.RNNCell(5, input_size=4), rnn.RNNCell(5, input_size=4))
    bi.initialize()
    outs, _ = bi.unroll(3, nd.array(np.random.randn(2, 3, 4)), layout='NTC', merge_outputs=True)
    assert outs.shape == (2, 3, 10)
    z = rnn.ZoneoutCell(rnn.RNNCell(5, input_size=4), zoneout_outputs=0.5, zoneout_states=0.5)
    z.initialize()
    o, _ = z(x, z.begin_state(batch_size=2))
    assert o.shape == (2, 5)


def test_valid_length_masks_padded_steps():
    cell = rnn.GRUCell(4, input_size=3)
    cell.initialize()
    x = nd.array(np.random.randn(2, 5, 3))
    vl = nd.array([5, 2])
    outs, states = cell.unroll(5, x, layout='NTC', merge_outputs=True, valid_length=vl)
    o = outs.asnumpy()
    assert np.abs(o[1, 2:]).sum() == 0 and np.abs(o[0, 4]).sum() > 0
    short, st2 = cell.unroll(2, x[1:2, :2], layout='NTC', merge_outputs=True)
    assert_almost_equal(states[0].asnumpy()[1], st2[0].asnumpy()[0], rtol=1e-5, atol=1e-6)


def _toy_data(n=64):
    rng = np.random.RandomState(0)
    x = rng.randn(n, 6).astype('float32')
    y = (x[:, 0] + x[:, 1] > 0).astype('float32')
    return gluon.data.DataLoader(gluon.data.ArrayDataset(x, y), batch_size=16)


def test_estimator_fit_with_handlers(tmp_path):
    from mxnet_b200.gluon.contrib.estimator import Estimator
    from mxnet_b200.gluon.contrib.estimator.event_handler import CheckpointHandler, EarlyStoppingHandler, LoggingHandler
    net = nn.HybridSequential()
    net.add(nn.Dense(16, activation='relu', in_units=6), nn.Dense(2, in_units=16))
    net.initialize(mx.init.Xavier())
    acc = mx.metric.Accuracy()
    est = Estimator(net, loss=gluon.loss.SoftmaxCrossEntropyLoss(), train_metrics=acc,
                    trainer=gluon.Trainer(net.collect_params(), 'adam', {'learning_rate': 0.05}))
    ckpt = CheckpointHandler(str(tmp_path), model_prefix='toy', monitor=est.train_metrics[0], save_best=True, epoch_period=1)
    early = EarlyStoppingHandler(monitor=est.train_metrics[0], patience=50, mode='max')
    data = _toy_data()
    est.fit(data, val_data=data, epochs=6, event_handlers=[ckpt, early, LoggingHandler()])
    assert est.train_metrics[0].get()[1] > 0.8
    files = os.listdir(str(tmp_path))
    assert any(f.endswith('.params') for f in files) and any(f.endswith('.states') for f in files)
    assert any('best' in f for f in files)
    scores = est.evaluate(data)
    assert scores is None or True
    # resume from the checkpoint
    net2 = nn.HybridSequential()
    net2.add(nn.Dense(16, activation='relu', in_units=6), nn.Dense(2, in_units=16))
    net2.initialize()
    est2 = Estimator(net2, loss=gluon.loss.SoftmaxCrossEntropyLoss(), train_metrics=mx.metric.Accuracy(),
                     trainer=gluon.Trainer(net2.collect_params(), 'adam', {'learning_rate': 0.05}))
    ck2 = CheckpointHandler(str(tmp_path), model_prefix='toy', resume_from_checkpoint=True)
    est2.fit(data, epochs=7, event_handlers=[ck2])
    assert ck2.trained_epoch == 5 and ck2.current_epoch == 1      # epochs 0..5 came from the checkpoint, one more ran


def test_flat_rnn_param_checkpoints_load_and_cells_infer_shapes(tmp_path):
    """A checkpoint that stores a fused layer as one flat `rnn_param` vector (the 2.x reference's layout) loads into the
    per-matrix parameters; `cell.infer_shape(i, x, is_bidirect)` completes deferred input widths of stacked cells."""
    import numpy as np
    import mxnet_b200 as mx
    from mxnet_b200 import gluon
    layer = gluon.rnn.LSTM(6, num_layers=2, bidirectional=True)
    layer.initialize()
    x = mx.nd.array(np.random.RandomState(0).randn(4, 3, 5).astype('float32'))
    expect = layer(x).asnumpy()
    flat = np.concatenate([getattr(layer, n).data().asnumpy().ravel() for n in layer._param_order()])
    path = str(tmp_path / 'lstm.params')
    mx.nd.save(path, {'rnn_param': mx.nd.array(flat)})
    fresh = gluon.rnn.LSTM(6, num_layers=2, bidirectional=True)       # input width still deferred
    fresh.load_parameters(path)
    np.testing.assert_allclose(fresh(x).asnumpy(), expect, rtol=1e-6, atol=1e-6)
    stack = gluon.rnn.SequentialRNNCell()
    stack.add(gluon.rnn.LSTMCell(7))
    stack.add(gluon.rnn.GRUCell(9))
    stack.infer_shape(0, mx.nd.ones((2, 5)), False)
    assert stack[0].i2h_weight.shape == (28, 5) and stack[1].i2h_weight.shape == (27, 7)
    cell = gluon.rnn.RNNCell(10)
    cell.infer_shape(0, mx.nd.ones((2, 4)), False)
    assert cell.i2h_weight.shape == (10, 4)
    cell2 = gluon.rnn.RNNCell(10)
    cell2.infer_shape(1, mx.nd.ones((2, 4)), True)
    assert cell2.i2h_weight.shape == (10, 20)


def test_conv_cell_deferred_channels_masked_residual_and_exported_constants(tmp_path):
    """``python/mxnet/gluon/rnn/conv_rnn_cell.py`` (input_shape[0] == -1 completed by infer_shape),
    ``rnn_cell.py`` ResidualCell / BidirectionalCell under ``valid_length`` (padded steps are zero, outputs come back
    merged) and export of a graph whose forward made its own begin state."""
    import mxnet_b200 as mx
    from mxnet_b200 import gluon
    seq = mx.np.ones((8, 3, 5, 7))
    cell = gluon.rnn.Conv1DLSTMCell((-1, 7), 10, (3,), (3,))
    cell.infer_shape(0, seq, False)
    assert cell.i2h_weight.shape[1] == 5
    cell.initialize()
    out, _ = cell.unroll(3, seq, merge_outputs=True)
    assert out.shape == (8, 3, 10, 5)

    valid = [3, 6, 2, 5]
    vl = mx.np.array(valid)
    stack = gluon.rnn.SequentialRNNCell()
    stack.add(gluon.rnn.ResidualCell(gluon.rnn.RNNCell(20)))
    stack.add(gluon.rnn.ResidualCell(gluon.rnn.RNNCell(20)))
    bidir = gluon.rnn.BidirectionalCell(gluon.rnn.GRUCell(20), gluon.rnn.GRUCell(20))
    data = mx.np.random.normal(0, 1, size=(6, 4, 20))
    for c in (stack, bidir):
        c.infer_shape(0, data, False)
        c.initialize()
        outs, _ = c.unroll(6, data, valid_length=vl, layout='TNC')
        assert not isinstance(outs, list)
        for i, n in enumerate(valid):
            one, _ = c.unroll(n, data[:n, i:i + 1, :], merge_outputs=True, layout='TNC')
            np.testing.assert_allclose(outs[:n, i:i + 1, :].asnumpy(), one.asnumpy(), rtol=1e-4, atol=1e-5)
            assert float(abs(outs[n:, i:i + 1, :]).sum()) == 0.0

    class Layer(gluon.HybridBlock):
        def __init__(self):
            super().__init__()
            self.cell = gluon.rnn.GRUCell(hidden_size=1)

        def forward(self, s):
            return self.cell.unroll(inputs=s, length=2, merge_outputs=True)[0]

    net = Layer()
    x = mx.np.ones((1, 2, 1))
    net.cell.infer_shape(0, x, False)
    net.initialize()
    net.hybridize()
    want = net(x)
    sym_file, params_file = net.export(str(tmp_path / 'model'))
    back = gluon.SymbolBlock.imports(sym_file, ['data'], params_file)
    np.testing.assert_allclose(back(x).asnumpy(), want.asnumpy(), rtol=1e-5, atol=1e-6)

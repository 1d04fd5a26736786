"""Smaller public modules: initializers, schedulers, callbacks, checkpoints, custom operators, sparse arrays,
control flow, random and linear-algebra operators, model zoo shapes, visualisation, image augmenters, quantization."""
import logging
import os

import numpy as np
import pytest

import mxnet_b200 as mx
from mxnet_b200 import autograd, gluon, nd


# ------------------------------------------------------------------------------------------- initializers
def test_initializers_statistics_and_patterns():
    mx.random.seed(11)
    shape = (64, 128)
    cases = {
        'xavier_uniform': (mx.init.Xavier(rnd_type='uniform', factor_type='avg', magnitude=3), (3.0 / ((64 + 128) / 2)) ** 0.5),
        'msra': (mx.init.MSRAPrelu(factor_type='in', slope=0.0), None),
        'normal': (mx.init.Normal(0.02), 0.02),
        'uniform': (mx.init.Uniform(0.1), 0.1),
    }
    for name, (init, scale) in cases.items():
        p = gluon.Parameter('weight', shape=shape, init=init)
        p.initialize()
        w = p.data().asnumpy()
        assert abs(w.mean()) < 0.02, name
        if name == 'normal':
            np.testing.assert_allclose(w.std(), scale, rtol=0.1)
        if name in ('uniform', 'xavier_uniform'):
            assert np.abs(w).max() <= scale + 1e-6
        if name == 'msra':
            np.testing.assert_allclose(w.std(), (2.0 / 128) ** 0.5, rtol=0.1)
    p = gluon.Parameter('weight', shape=(8, 8), init=mx.init.Orthogonal())
    p.initialize()
    w = p.data().asnumpy()
    np.testing.assert_allclose(w @ w.T, np.eye(8) * (w @ w.T)[0, 0], atol=1e-4)
    for init, val in ((mx.init.Zero(), 0.0), (mx.init.One(), 1.0), (mx.init.Constant(2.5), 2.5)):
        p = gluon.Parameter('weight', shape=(3, 3), init=init)
        p.initialize()
        assert (p.data().asnumpy() == val).all()
    b = gluon.Parameter('bias', shape=(8,), init=mx.init.LSTMBias(forget_bias=1.0))
    b.initialize()
    np.testing.assert_array_equal(b.data().asnumpy(), [0, 0, 1, 1, 0, 0, 0, 0])


def test_lr_schedulers():
    f = mx.lr_scheduler.FactorScheduler(step=10, factor=0.5, base_lr=1.0, stop_factor_lr=0.2)
    assert f(1) == 1.0 and f(11) == 0.5 and f(21) == 0.25 and f(100) == 0.2
    m = mx.lr_scheduler.MultiFactorScheduler(step=[5, 8], factor=0.1, base_lr=1.0)
    np.testing.assert_allclose([m(1), m(6), m(9)], [1.0, 0.1, 0.01])
    p = mx.lr_scheduler.PolyScheduler(max_update=100, base_lr=1.0, pwr=2, final_lr=0.0)
    np.testing.assert_allclose(p(50), 0.25, rtol=1e-6)
    c = mx.lr_scheduler.CosineScheduler(max_update=100, base_lr=1.0, final_lr=0.0, warmup_steps=10, warmup_begin_lr=0.0)
    np.testing.assert_allclose(c(5), 0.5, rtol=1e-6)          # linear warm-up
    np.testing.assert_allclose(c(55), 0.5, rtol=1e-6)         # halfway down the cosine
    assert abs(c(100)) < 1e-12 and abs(c(200)) < 1e-12     # past max_update the last value is kept


def test_speedometer_and_checkpoint_callbacks(tmp_path, caplog):
    from collections import namedtuple
    Param = namedtuple('BatchEndParam', ['epoch', 'nbatch', 'eval_metric', 'locals'])
    metric = mx.gluon.metric.Accuracy()
    metric.update([nd.array([0, 1])], [nd.array([[0.9, 0.1], [0.2, 0.8]])])
    sp = mx.callback.Speedometer(batch_size=2, frequent=2, auto_reset=False)
    with caplog.at_level(logging.INFO):
        for i in range(5):
            sp(Param(0, i, metric, None))
    assert any('samples/sec' in r.getMessage() for r in caplog.records)
    sym = mx.sym.FullyConnected(mx.sym.var('data'), num_hidden=3, name='fc')
    arg = {'fc_weight': nd.array(np.arange(6, dtype='float32').reshape(3, 2)), 'fc_bias': nd.array([1.0, 2.0, 3.0])}
    prefix = str(tmp_path / 'model')
    mx.model.save_checkpoint(prefix, 3, sym, arg, {})
    assert os.path.exists(prefix + '-0003.params') and os.path.exists(prefix + '-symbol.json')
    sym2, arg2, aux2 = mx.model.load_checkpoint(prefix, 3)
    assert sym2.list_arguments() == sym.list_arguments() and aux2 == {}
    for k in arg:
        np.testing.assert_array_equal(arg[k].asnumpy(), arg2[k].asnumpy())


# ------------------------------------------------------------------------------------------- custom operator
def test_custom_operator_forward_backward():
    class Scale2(mx.operator.CustomOp):
        def forward(self, is_train, req, in_data, out_data, aux):
            self.assign(out_data[0], req[0], in_data[0] * 2)

        def backward(self, req, out_grad, in_data, out_data, in_grad, aux):
            self.assign(in_grad[0], req[0], out_grad[0] * 2)

    @mx.operator.register('scale2_test')
    class Scale2Prop(mx.operator.CustomOpProp):
        def list_arguments(self):
            return ['data']

        def infer_shape(self, in_shape):
            return in_shape, [in_shape[0]], []

        def create_operator(self, ctx, shapes, dtypes):
            return Scale2()

    x = nd.array([1.0, -2.0, 3.0])
    x.attach_grad()
    with autograd.record():
        y = nd.Custom(x, op_type='scale2_test')
        z = (y * y).sum()
    z.backward()
    np.testing.assert_allclose(y.asnumpy(), [2, -4, 6])
    np.testing.assert_allclose(x.grad.asnumpy(), 8 * x.asnumpy())


# ------------------------------------------------------------------------------------------- sparse
def test_sparse_arrays_round_trip_and_dot():
    dense = np.array([[0, 1.5, 0], [0, 0, 0], [2.0, 0, 3.0]], dtype='float32')
    csr = nd.array(dense).tostype('csr')
    assert csr.stype == 'csr'
    np.testing.assert_array_equal(csr.indices.asnumpy(), [1, 0, 2])
    np.testing.assert_array_equal(csr.indptr.asnumpy(), [0, 1, 1, 3])
    np.testing.assert_array_equal(csr.tostype('default').asnumpy(), dense)
    rsp = nd.array(dense).tostype('row_sparse')
    np.testing.assert_array_equal(rsp.indices.asnumpy(), [0, 2])
    np.testing.assert_array_equal(rsp.tostype('default').asnumpy(), dense)
    rhs = np.arange(6, dtype='float32').reshape(3, 2)
    np.testing.assert_allclose(nd.dot(csr, nd.array(rhs)).asnumpy(), dense @ rhs)
    made = nd.sparse.csr_matrix((csr.data, csr.indices, csr.indptr), shape=(3, 3))
    np.testing.assert_array_equal(made.asnumpy(), dense)


# ------------------------------------------------------------------------------------------- control flow
def test_contrib_foreach_while_cond():
    def step(x, state):
        new = state[0] + x
        return new * 2, [new]
    outs, states = nd.contrib.foreach(step, nd.array([[1.0], [2.0], [3.0]]), [nd.zeros((1,))])
    np.testing.assert_allclose(outs.asnumpy().reshape(-1), [2, 6, 12])
    np.testing.assert_allclose(states[0].asnumpy(), [6])
    outs, final = nd.contrib.while_loop(lambda i, s: i < 4, lambda i, s: ([s], [i + 1, s + i]),
                                        [nd.array([0.0]), nd.array([0.0])], max_iterations=6)
    np.testing.assert_allclose(final[1].asnumpy(), [6])           # 0 + 1 + 2 + 3
    assert outs[0].shape[0] == 6
    r = nd.contrib.cond(nd.array([1.0]), lambda: nd.array([10.0]), lambda: nd.array([20.0]))
    np.testing.assert_allclose(r.asnumpy(), [10])


# ------------------------------------------------------------------------------------------- random / linalg
def test_random_operators_moments_and_seed():
    mx.random.seed(42)
    a = nd.random.normal(2.0, 3.0, shape=(50000,)).asnumpy()
    np.testing.assert_allclose([a.mean(), a.std()], [2.0, 3.0], rtol=0.05)
    u = nd.random.uniform(-1, 1, shape=(50000,)).asnumpy()
    assert u.min() >= -1 and u.max() <= 1 and abs(u.mean()) < 0.02
    g = nd.random.gamma(2.0, 2.0, shape=(50000,)).asnumpy()
    np.testing.assert_allclose(g.mean(), 4.0, rtol=0.05)
    r = nd.random.randint(0, 5, shape=(10000,)).asnumpy()
    assert set(np.unique(r)) <= {0, 1, 2, 3, 4}
    mx.random.seed(7)
    x1 = nd.random.normal(shape=(5,)).asnumpy()
    mx.random.seed(7)
    np.testing.assert_array_equal(x1, nd.random.normal(shape=(5,)).asnumpy())
    m = nd.random.multinomial(nd.array([0.0, 0.0, 1.0]), shape=(20,)).asnumpy()
    assert (m == 2).all()
    p = nd.array(np.arange(10, dtype='float32'))
    s = nd.random.shuffle(p).asnumpy()
    assert sorted(s.tolist()) == list(range(10))


def test_linalg_operators():
    rng = np.random.RandomState(0)
    a = rng.randn(4, 4).astype('float32')
    spd = a @ a.T + 4 * np.eye(4, dtype='float32')
    L = nd.linalg.potrf(nd.array(spd)).asnumpy()
    np.testing.assert_allclose(L @ L.T, spd, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(nd.linalg.potri(nd.array(L)).asnumpy(), np.linalg.inv(spd), rtol=1e-3, atol=1e-4)
    np.testing.assert_allclose(nd.linalg.sumlogdiag(nd.array(L)).asnumpy(), np.log(np.diag(L)).sum(), rtol=1e-5)
    b = rng.randn(4, 3).astype('float32')
    np.testing.assert_allclose(nd.linalg.gemm2(nd.array(a), nd.array(b), alpha=2.0).asnumpy(), 2 * a @ b, rtol=1e-4, atol=1e-5)
    x = nd.linalg.trsm(nd.array(L), nd.array(b)).asnumpy()
    np.testing.assert_allclose(L @ x, b, rtol=1e-3, atol=1e-4)
    u, lam = nd.linalg.syevd(nd.array(spd))
    np.testing.assert_allclose(np.sort(lam.asnumpy()), np.sort(np.linalg.eigvalsh(spd)), rtol=1e-4)
    np.testing.assert_allclose(nd.linalg.det(nd.array(spd)).asnumpy(), np.linalg.det(spd), rtol=1e-3)
    np.testing.assert_allclose(nd.linalg.inverse(nd.array(spd)).asnumpy(), np.linalg.inv(spd), rtol=1e-3, atol=1e-4)


# ------------------------------------------------------------------------------------------- model zoo / visualisation
@pytest.mark.parametrize('name,size', [('resnet18_v1', 64), ('resnet18_v2', 64), ('mobilenet0_25', 64), ('squeezenet1_1', 96),
                                       ('vgg11', 64), ('densenet121', 224), ('alexnet', 224), ('mobilenet_v2_0_25', 64)])
def test_model_zoo_forward_shapes(name, size):
    from mxnet_b200.gluon.model_zoo import vision
    net = vision.get_model(name, classes=10)
    net.initialize()
    out = net(nd.array(np.random.RandomState(0).randn(1, 3, size, size).astype('float32')))
    assert out.shape == (1, 10)
    assert np.isfinite(out.asnumpy()).all()


def test_print_summary_and_block_summary(capsys):
    data = mx.sym.var('data')
    net = mx.sym.FullyConnected(data, num_hidden=8, name='fc1')
    net = mx.sym.Activation(net, act_type='relu', name='relu1')
    net = mx.sym.FullyConnected(net, num_hidden=2, name='fc2')
    mx.viz.print_summary(net, shape={'data': (1, 4)})
    out = capsys.readouterr().out
    assert 'fc1' in out and 'fc2' in out and 'Total params' in out
    blk = gluon.nn.HybridSequential()
    blk.add(gluon.nn.Dense(8, in_units=4), gluon.nn.Dense(2, in_units=8))
    blk.initialize()
    blk.summary(nd.zeros((1, 4)))
    assert 'Dense' in capsys.readouterr().out


# ------------------------------------------------------------------------------------------- image
def test_image_augmenters_and_resize():
    rng = np.random.RandomState(0)
    img = nd.array(rng.randint(0, 255, (40, 60, 3)).astype('uint8'), dtype='uint8')
    out = mx.image.resize_short(img, 20)
    assert min(out.shape[:2]) == 20 and out.shape[2] == 3
    crop, rect = mx.image.center_crop(img, (30, 20))
    assert crop.shape == (20, 30, 3) and rect == (15, 10, 30, 20)
    augs = mx.image.CreateAugmenter(data_shape=(3, 24, 24), resize=32, rand_crop=True, rand_mirror=True, mean=True, std=True)
    x = img
    for a in augs:
        x = a(x)
    assert x.shape == (24, 24, 3) and x.dtype == np.float32
    flipped = mx.image.HorizontalFlipAug(1.0)(img)
    np.testing.assert_array_equal(flipped.asnumpy(), img.asnumpy()[:, ::-1])
    t = gluon.data.vision.transforms.Compose([gluon.data.vision.transforms.Resize(16), gluon.data.vision.transforms.ToTensor(),
                                              gluon.data.vision.transforms.Normalize(0.5, 0.25)])
    y = t(img)
    assert y.shape == (3, 16, 16)


# ------------------------------------------------------------------------------------------- quantization
def test_quantize_dequantize_round_trip():
    x = nd.array(np.linspace(-3, 3, 64, dtype='float32').reshape(8, 8))
    q, mn, mxv = nd.contrib.quantize_v2(x, out_type='int8')
    assert q.dtype == np.int8
    back = nd.contrib.dequantize(q, mn, mxv, out_type='float32')
    np.testing.assert_allclose(back.asnumpy(), x.asnumpy(), atol=3.0 / 127 + 1e-6)


def test_notebook_pandas_logger_collects_metrics():
    pd = pytest.importorskip('pandas')
    from collections import namedtuple
    from mxnet_b200.notebook.callback import PandasLogger, LiveLearningCurve, args_wrapper
    Param = namedtuple('Param', 'epoch nbatch eval_metric')
    metric = mx.gluon.metric.Accuracy()
    metric.update([mx.nd.array([0, 1, 1])], [mx.nd.array([[0.9, 0.1], [0.2, 0.8], [0.7, 0.3]])])
    log = PandasLogger(batch_size=3, frequent=2)
    for i in range(5):
        log.train_cb(Param(0, i, metric))
    log.eval_cb(Param(0, 5, metric))
    log.epoch_cb()
    assert isinstance(log.train_df, pd.DataFrame) and len(log.train_df) == 3          # batches 0, 2, 4
    assert abs(log.train_df['accuracy'].iloc[-1] - 2 / 3) < 1e-6
    assert {'records_per_sec', 'minibatch_count', 'epoch'} <= set(log.train_df.columns)
    assert len(log.eval_df) == 1 and len(log.epoch_df) == 1
    curve = LiveLearningCurve('accuracy', display_freq=1000, frequent=1)       # collects without a chart when bokeh is absent
    curve.batch_cb(Param(0, 0, metric))
    curve.eval_cb(Param(0, 0, metric))
    assert len(curve._data['train']['accuracy']) == 1 and len(curve._data['eval']['accuracy']) == 1
    merged = args_wrapper(log, curve)
    assert len(merged['batch_end_callback']) == 2


def test_dataloader_iter_pads_the_last_batch():
    from mxnet_b200.contrib.io import DataLoaderIter
    data = np.arange(10 * 4, dtype='float32').reshape(10, 4)
    label = np.arange(10, dtype='float32')
    loader = mx.gluon.data.DataLoader(mx.gluon.data.ArrayDataset(data, label), batch_size=4)
    it = DataLoaderIter(loader)
    assert it.provide_data[0].shape == (4, 4) and it.provide_label[0].name == 'softmax_label'
    batches = list(it)
    assert [b.pad for b in batches] == [0, 0, 2]
    assert batches[-1].data[0].shape == (4, 4)
    np.testing.assert_allclose(batches[-1].data[0].asnumpy()[:2], data[8:])
    it.reset()
    assert len(list(it)) == 3


def test_constraint_check_operator():
    mx.npx.set_np()
    try:
        ok = mx.npx.constraint_check(mx.np.array([1.0, 2.0]) > 0, 'Scale should be larger than zero')
        assert bool(ok.asnumpy())
        with pytest.raises(ValueError, match='larger than zero'):
            mx.npx.constraint_check(mx.np.array([1.0, -2.0]) > 0, 'Scale should be larger than zero')
    finally:
        mx.npx.reset_np()


def test_image_rotation_and_small_api_additions():
    import torch
    from mxnet_b200 import image, util
    img = nd.array(np.arange(3 * 8 * 8, dtype='float32').reshape(3, 8, 8))
    r90 = image.imrotate(img, 90).asnumpy()
    np.testing.assert_allclose(r90, np.rot90(img.asnumpy(), k=1, axes=(1, 2)), atol=1e-4)
    batch = nd.array(np.ones((2, 1, 6, 10), dtype='float32'))
    out = image.imrotate(batch, nd.array([30.0, -45.0]), zoom_in=True).asnumpy()
    assert out.min() > 0.999                                             # no padding shows
    plain = image.imrotate(batch, 30.0).asnumpy()
    assert plain.min() < 0.5
    small = image.imrotate(batch, 30.0, zoom_out=True).asnumpy()
    assert abs(small.sum() - batch.asnumpy().sum() / 1.0) < batch.asnumpy().sum()       # the whole source is inside
    assert small[:, :, 0, 0].max() < 0.5                                                  # corners are padding
    with pytest.raises(ValueError):
        image.imrotate(img, 10, zoom_in=True, zoom_out=True)
    assert image.random_rotate(batch, (-10, 10)).shape == (2, 1, 6, 10)
    aug = image.detection.CreateMultiRandCropAugmenter(min_object_covered=[0.1, 0.5], area_range=[(0.1, 1.0), (0.3, 1.0)])
    assert len(aug.aug_list) == 2 and aug.aug_list[1].min_object_covered == 0.5
    from mxnet_b200.gluon import metric
    np.testing.assert_array_equal(metric.one_hot(np.array([0, 2]), 3), [[1, 0, 0], [0, 0, 1]])
    np.testing.assert_array_equal(metric.predict_with_threshold(np.array([[0.2, 0.9]]), np.array([0.5, 0.95])), [[False, False]])
    handle = mx.gluon.utils.HookHandle()
    hooks = {}
    handle.attach(hooks, lambda *a: None)
    assert len(hooks) == 1
    handle.detach()
    assert not hooks
    assert isinstance(mx.runtime.get_branch(), str) and len(mx.runtime.get_commit_hash()) >= 7
    mx.profiler.set_kvstore_handle(None)
    assert util.get_rtc_compile_opts.__doc__ and util.np_ufunc_legal_option('casting', 'safe')
    assert callable(mx.contrib.quantization.quantize_model_onednn) and callable(mx.amp.amp.warn_if_model_exists)


def test_legacy_python_operators_and_dynamic_unroll():
    import warnings
    from mxnet_b200 import operator as mxop

    class Square(mxop.NumpyOp):
        def forward(self, in_data, out_data):
            out_data[0][:] = in_data[0] ** 2

        def backward(self, out_grad, in_data, out_data, in_grad):
            in_grad[0][:] = 2 * in_data[0] * out_grad[0]

    class Scale(mxop.NDArrayOp):
        def forward(self, in_data, out_data):
            out_data[0][:] = in_data[0] * 3

        def backward(self, out_grad, in_data, out_data, in_grad):
            in_grad[0][:] = out_grad[0] * 3
    with warnings.catch_warnings():
        warnings.simplefilter('ignore')
        s = Scale()(Square()(mx.sym.var('data')))
    x = nd.array([1.0, -2.0, 3.0])
    g = nd.zeros((3,))
    ex = s._bind(mx.cpu(), {'data': x}, args_grad={'data': g})
    np.testing.assert_allclose(ex.forward(is_train=True)[0].asnumpy(), [3, 12, 27])
    ex.backward([nd.ones((3,))])
    np.testing.assert_allclose(g.asnumpy(), [6, -12, 18])
    grouped = mxop.get_all_registered_operators_grouped()
    assert 'broadcast_add' in grouped and 'elemwise_add' in grouped['broadcast_add']

    from mxnet_b200.gluon import rnn
    from mxnet_b200.gluon.rnn.rnn_cell import dynamic_unroll
    cell = rnn.LSTMCell(5, input_size=4)
    cell.initialize()
    data = nd.array(np.random.RandomState(0).randn(3, 2, 4))
    states = cell.begin_state(batch_size=2)
    out, new_states = dynamic_unroll(cell, data, states, valid_length=nd.array([2, 3]), layout='TNC')
    assert out.shape == (3, 2, 5) and not out.asnumpy()[2, 0].any() and out.asnumpy()[2, 1].any()
    full, _ = dynamic_unroll(cell, data, states, layout='TNC')
    np.testing.assert_allclose(out.asnumpy()[:2], full.asnumpy()[:2], rtol=1e-6)


def test_more_test_utils_helpers():
    from mxnet_b200 import test_utils as tu
    a, (vals, rows) = tu.rand_sparse_ndarray((6, 4), 'row_sparse', density=0.5)
    assert a.stype == 'row_sparse' and vals.shape[0] == len(rows)
    np.testing.assert_allclose(a.asnumpy()[rows], vals)
    c, (indptr, indices, data) = tu.rand_sparse_ndarray((6, 5), 'csr', density=0.4, shuffle_csr_indices=True)
    assert c.stype == 'csr' and indptr[-1] == len(data) == len(indices)
    p = tu.rand_sparse_ndarray((8, 8), 'csr', density=0.3, distribution='powerlaw')[0].asnumpy()
    assert list((p != 0).sum(1)[:3]) == [1, 2, 4]
    assert tu.create_sparse_array_zd((3, 3), 'csr', 0.0).asnumpy().sum() == 0
    assert tu.create_2d_tensor(3, 2).asnumpy().tolist() == [[0, 0], [1, 1], [2, 2]] and tu.create_vector(4).shape == (4,)
    np.testing.assert_allclose(tu.collapse_sum_like(np.ones((2, 3, 4)), (3, 1)), [[8.0]] * 3)
    np.testing.assert_allclose(tu.assign_each2(np.array([1., 2.]), np.array([3., 4.]), lambda x, y: x * y), [3, 8])
    x = nd.ones((3,))
    assert tu.same_array(x, x) and not tu.same_array(x, x.copy())
    s = mx.sym.FullyConnected(mx.sym.var('data'), num_hidden=4)
    assert tu.check_speed(s, data=(8, 16), N=2) > 0 and tu.check_speed(s, data=(8, 16), N=2, typ='forward') > 0
    assert tu.same_symbol_structure(s, s) and os.path.isfile(tu.get_im2rec_path())
    m = tu.new_sym_matrix_with_real_eigvals_nd((2, 3, 3))
    np.testing.assert_allclose(m, m.transpose(0, 2, 1), atol=1e-12)
    q = tu.new_orthonormal_matrix_2d(4)
    np.testing.assert_allclose(q @ q.T, np.eye(4), atol=1e-10)
    assert np.isreal(np.linalg.eigvals(tu.new_matrix_with_real_eigvals_nd((2, 3, 3)))).all()
    tu.compare_optimizer_noise_seeded(mx.optimizer.SGLD(learning_rate=0.1), mx.optimizer.SGLD(learning_rate=0.1), [(3, 4)], 'float32', 7)
    tu.assert_almost_equal_ignore_nan(np.array([1.0, np.nan]), np.array([1.0, 5.0]))
    with pytest.raises(IOError):
        tu.get_mnist_ubyte('/nonexistent-directory')
    with tu.discard_stderr():
        pass
    assert tu.default_numeric_eps()[np.dtype('float32')] == 1.0 / 512 and tu.get_etol() == 0


def test_second_batch_of_api_names(tmp_path):
    from mxnet_b200 import amp as _amp   # noqa: F401
    from mxnet_b200.gluon.block import get_optimization_constraints, set_optimization_constraints
    Flag = mx.gluon.HybridBlock.OptConstraint.Flag
    assert get_optimization_constraints() == Flag(0)
    with mx.gluon.HybridBlock.OptConstraint.disable_amp():
        assert get_optimization_constraints() == Flag.DisableAMP
    assert get_optimization_constraints() == Flag(0)
    prev = set_optimization_constraints(Flag.DisableAMP)
    assert prev == Flag(0)
    set_optimization_constraints(prev)
    s = mx.sym.random.randn(2, 3, loc=1.0, scale=0.0)
    np.testing.assert_allclose(s._bind(mx.cpu(), {}).forward()[0].asnumpy(), np.ones((2, 3)))
    sh = mx.sym.random.shuffle(mx.sym.var('x'))
    out = sh._bind(mx.cpu(), {'x': nd.array(np.arange(6.0))}).forward()[0].asnumpy()
    assert sorted(out.tolist()) == list(range(6))
    cat = mx.sym.random.categorical(mx.sym.var('p'), shape=(50,))
    draws = cat._bind(mx.cpu(), {'p': nd.array([[0.0, 1.0, 0.0]])}).forward()[0].asnumpy()
    assert draws.shape == (1, 50) and (draws == 1).all()
    txt = tmp_path / 't.csv'
    txt.write_text('1,2,3\n4,5,6\n')
    g = mx.np.genfromtxt(str(txt), delimiter=',')
    assert g.shape == (2, 3) and float(g.sum()) == 21
    mx.np.set_printoptions(precision=3)
    np.set_printoptions(precision=8)
    assert mx.base.data_dir().endswith('mxnet') or 'MXNET_HOME' in os.environ
    assert mx.base.c_array(__import__('ctypes').c_int, [1, 2, 3])[2] == 3 and mx.base.c_str('ab').value == b'ab'
    assert 'Parameters' in mx.base.build_param_doc(['a'], ['int'], ['first'])
    assert mx.name.current() is mx.name.NameManager.current() and mx.attribute.current() is mx.attribute.AttrScope.current()
    with pytest.raises(ValueError):
        mx.gluon.model_zoo.model_store.short_hash('no_such_model', root=str(tmp_path))
    (tmp_path / 'resnet18_v1-a0666292.params').write_bytes(b'')
    assert mx.gluon.model_zoo.model_store.short_hash('resnet18_v1', root=str(tmp_path)) == 'a0666292'
    assert mx.gluon.data.dataloader.DataLoaderV1 is mx.gluon.data.DataLoader
    assert mx.library.compiled_with_gcc_cxx11_abi() is True


def test_block_save_load_and_method_additions(tmp_path):
    from mxnet_b200.gluon import nn
    from mxnet_b200.symbol.symbol import NotImplementedForSymbol

    def build():
        net = nn.HybridSequential()
        net.add(nn.Dense(8, activation='relu', in_units=4), nn.Dense(3, in_units=8))
        return net
    net = build()
    net.initialize()
    net.hybridize()
    x = nd.array(np.random.RandomState(0).randn(2, 4))
    net(x)
    ref = net(x).asnumpy()
    prefix = str(tmp_path / 'mymodel')
    net.save(prefix)
    assert os.path.exists(prefix + '-model.json') and os.path.exists(prefix + '-model.params')
    other = build()
    other.load(prefix)
    np.testing.assert_allclose(other(x).asnumpy(), ref, rtol=1e-6)
    assert other._active and other._cached_graph is not None
    wrong = nn.HybridSequential()
    wrong.add(nn.Dense(8, in_units=4))
    wrong_seq = nn.Sequential()
    with pytest.raises(ValueError):
        wrong_seq.load(prefix)
    assert net.generate_arg_names(1) == ['data'] and net.generate_arg_names(2) == ['data0', 'data1']
    s = mx.sym.var('x')
    c = s.astype('float16')
    assert c._bind(mx.cpu(), {'x': nd.ones((2,))}).forward()[0].dtype == np.float16
    assert not s.has_dynamic_shape_op() and mx.sym.contrib.boolean_mask(s, mx.sym.var('m')).has_dynamic_shape_op()
    with pytest.raises(NotImplementedForSymbol):
        s.asnumpy()
    a = nd.ones((3, 4))
    a.attach_grad()
    assert a.grad is not None
    a.drop_grad()
    assert a.grad is None
    a.slice_assign_scalar(5.0, (0, 1), (2, 3), (None, None))
    assert a.asnumpy()[:2, 1:3].sum() == 20 and a.asnumpy().sum() == 28
    m = mx.np.arange(6).reshape(2, 3)
    assert m.mT.shape == (3, 2) and m.diagonal().shape == (2,) and m.reshape_view(3, 2).shape == (3, 2)
    ex = mx.sym.relu(s)._bind(mx.cpu(), {'x': nd.ones((2,))})
    assert ex.get_optimized_symbol().list_arguments() == ['x']


def test_tensor_inspector(tmp_path):
    from mxnet_b200.inspector import CheckerType, TensorInspector
    a = nd.array(np.array([[1.0, -2.0, 0.0], [np.nan, np.inf, -np.inf]], dtype='float32'))
    ti = TensorInspector(a)
    text = ti.to_string()
    assert 'float32 Tensor 2x3' in text and 'nan' in text
    assert ti.check_value(CheckerType.NaNChecker) == [(1, 0)]
    assert ti.check_value(CheckerType.NegativeChecker) == [(0, 1), (1, 2)]
    assert ti.check_value(CheckerType.InfChecker) == [(1, 1), (1, 2)]
    assert ti.check_value(CheckerType.AbnormalChecker) == [(0, 2), (1, 0), (1, 1), (1, 2)]
    assert ti.check_value(lambda v: v == 1.0) == [(0, 0)]
    f1 = ti.dump_to_file('probe', str(tmp_path))
    f2 = ti.dump_to_file('probe', str(tmp_path))
    assert f1.endswith('probe_1.npy') and f2.endswith('probe_2.npy')
    np.testing.assert_array_equal(np.load(f1), a.asnumpy())


def test_reference_import_paths_and_helper_names():
    """Names a reference user reaches by their import paths: ``gluon.nn.HybridBlock``, per-optimizer modules, model-zoo getters,
    symbol helpers, npx interchange helpers, random.binomial / categorical."""
    import numpy as np
    import mxnet_b200 as mx
    from mxnet_b200.gluon import nn
    from mxnet_b200.gluon.model_zoo import vision
    assert nn.HybridBlock is mx.gluon.HybridBlock and nn.Block is mx.gluon.Block and nn.SymbolBlock is mx.gluon.SymbolBlock
    from mxnet_b200.optimizer.sgd import SGD
    from mxnet_b200.optimizer.adamW import AdamW
    from mxnet_b200.optimizer.contrib import GroupAdaGrad
    assert SGD is mx.optimizer.SGD and AdamW is mx.optimizer.AdamW and GroupAdaGrad is mx.optimizer.GroupAdaGrad
    assert type(vision.get_vgg(11)).__name__ == 'VGG' and type(vision.get_mobilenet(0.25)).__name__ == 'MobileNet'
    assert type(vision.get_mobilenet_v2(0.25)).__name__ == 'MobileNetV2'
    x, y = mx.sym.Variable('x'), mx.sym.Variable('y')
    e = mx.sym.maximum(x, 2.0) + mx.sym.minimum(3.0, y) + mx.sym.power(x, y) + mx.sym.pow(2.0, x) + mx.sym.hypot(x, y)
    got = e.bind(mx.cpu(), {'x': mx.nd.array([1., 3.]), 'y': mx.nd.array([2., 4.])}).forward()[0].asnumpy()
    expect = np.maximum([1, 3], 2) + np.minimum(3, [2, 4]) + np.power([1., 3.], [2., 4.]) + np.power(2., [1, 3]) + np.hypot([1, 3], [2, 4])
    np.testing.assert_allclose(got, expect, rtol=1e-6)
    assert mx.sym.maximum(2, 3) == 3 and mx.sym.minimum(2, 3) == 2
    parts = mx.sym.split_v2(x, (1, 3)).bind(mx.cpu(), {'x': mx.nd.array([1., 3., 5., 7.])}).forward()
    assert [p.shape for p in parts] == [(1,), (2,), (1,)]
    assert float(mx.sym.eye(3).bind(mx.cpu(), {}).forward()[0].asnumpy().trace()) == 3.0
    np.testing.assert_allclose(mx.sym.linspace(0, 1, 5).bind(mx.cpu(), {}).forward()[0].asnumpy(), np.linspace(0, 1, 5))
    assert callable(mx.sym.sparse.dot) and callable(mx.sym.sparse.cast_storage)
    a = mx.npx.from_numpy(np.arange(6.).reshape(2, 3))
    b = mx.npx.from_dlpack(mx.npx.to_dlpack_for_read(a))
    assert type(b).__name__ == 'ndarray' and float(b.asnumpy().sum()) == 15.0
    mx.random.seed(3)
    draws = mx.random.binomial(10, 0.3, shape=(4000,))
    assert abs(float(draws.mean().asscalar()) - 3.0) < 0.15
    c, logp = mx.random.categorical(mx.nd.array([[0.1, 0.9]]), get_prob=True)
    assert int(c.asnumpy()[0]) in (0, 1) and logp.shape == (1,)
    assert mx.io.ImageRecordUInt8Iter_v1 is mx.io.ImageRecordUInt8Iter
    from mxnet_b200 import callback, test_utils
    assert callable(callback.save_checkpoint) and test_utils.get_dtype_name(np.float16) == 'float16'


def test_contrib_rand_zipfian_and_multi_tensor_lamb_wrappers():
    import numpy as np
    import mxnet_b200 as mx
    mx.random.seed(5)
    samples, exp_true, exp_sampled = mx.nd.contrib.rand_zipfian(mx.nd.array([3, 0]), 2000, 50)
    s = samples.asnumpy()
    assert s.dtype == np.int64 and s.min() >= 0 and s.max() < 50
    log_range = np.log(51.0)
    np.testing.assert_allclose(exp_true.asnumpy(), np.log(np.array([5 / 4, 2.0])) / log_range * 2000, rtol=1e-10)
    np.testing.assert_allclose(exp_sampled.asnumpy(), np.log((s + 2.0) / (s + 1.0)) / log_range * 2000, rtol=1e-10)
    assert abs((s == 0).mean() - np.log(2.0) / log_range) < 0.04           # the most frequent class
    t = mx.sym.Variable('t')
    outs = mx.sym.Group(list(mx.sym.contrib.rand_zipfian(t, 8, 5))).bind(mx.cpu(), {'t': mx.nd.array([3])}).forward()
    assert outs[0].shape == (8,) and outs[1].shape == (1,) and outs[2].shape == (8,)
    w = [mx.nd.ones((3,)), mx.nd.ones((2, 2))]
    g = [mx.nd.ones((3,)) * 0.1, mx.nd.ones((2, 2)) * 0.2]
    m = [mx.nd.zeros((3,)), mx.nd.zeros((2, 2))]
    v = [mx.nd.zeros((3,)), mx.nd.zeros((2, 2))]
    mx.nd.contrib.multi_lamb_update(w, g, m, v, [1, 1], [0.1, 0.1], [0.0, 0.0])
    np.testing.assert_allclose(w[0].asnumpy(), 0.9, rtol=1e-5)             # unit trust ratio step of size lr
    assert [p.shape for p in mx.nd.split_v2(mx.nd.ones((6, 2)), 3)] == [(2, 2)] * 3
    assert mx.nd.dtype_mx_to_np(mx.nd.dtype_np_to_mx(np.float16)) is np.float16


def test_symbolic_samplers_take_scalars_or_symbols():
    """``mx.sym.random.<dist>``: scalar parameters are attributes (no graph inputs), Symbol parameters are inputs with one
    distribution per element (python/mxnet/symbol/random.py)."""
    import numpy as np
    import mxnet_b200 as mx
    mx.random.seed(11)
    u = mx.sym.random.uniform(2.0, 4.0, shape=(3000,))
    assert u.list_arguments() == []
    vals = u.bind(mx.cpu(), {}).forward()[0].asnumpy()
    assert vals.min() >= 2.0 and vals.max() <= 4.0 and abs(vals.mean() - 3.0) < 0.05
    assert abs(mx.sym.random.exponential(2.0, shape=(6000,)).bind(mx.cpu(), {}).forward()[0].asnumpy().mean() - 2.0) < 0.1
    assert abs(mx.sym.random.poisson(3.0, shape=(6000,)).bind(mx.cpu(), {}).forward()[0].asnumpy().mean() - 3.0) < 0.1
    lo, hi = mx.sym.Variable('lo'), mx.sym.Variable('hi')
    per = mx.sym.random.uniform(lo, hi, shape=(500,))
    assert per.list_arguments() == ['lo', 'hi']
    out = per.bind(mx.cpu(), {'lo': mx.nd.array([0., 10.]), 'hi': mx.nd.array([1., 11.])}).forward()[0].asnumpy()
    assert out.shape == (2, 500) and out[0].max() <= 1.0 and out[1].min() >= 10.0
    with pytest.raises(ValueError):
        mx.sym.random.uniform(lo, 1.0)

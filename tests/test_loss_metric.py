"""Gluon losses and evaluation metrics against NumPy formulas (reference: tests/python/unittest/test_loss.py,
test_metric.py)."""
import numpy as np
import pytest

import mxnet_b200 as mx
from mxnet_b200 import gluon, nd
from mxnet_b200.test_utils import assert_almost_equal

rng = np.random.RandomState(0)


def _softmax(x):
    e = np.exp(x - x.max(-1, keepdims=True))
    return e / e.sum(-1, keepdims=True)


def test_softmax_cross_entropy_variants():
    x = rng.randn(6, 5).astype('float32')
    y = rng.randint(0, 5, (6,))
    ref = -np.log(_softmax(x)[np.arange(6), y])
    out = gluon.loss.SoftmaxCrossEntropyLoss()(nd.array(x), nd.array(y))
    assert_almost_equal(out.asnumpy(), ref, rtol=1e-5, atol=1e-6)
    dense = np.eye(5, dtype='float32')[y]
    out = gluon.loss.SoftmaxCrossEntropyLoss(sparse_label=False)(nd.array(x), nd.array(dense))
    assert_almost_equal(out.asnumpy(), ref, rtol=1e-5, atol=1e-6)
    out = gluon.loss.SoftmaxCrossEntropyLoss(from_logits=True)(nd.array(np.log(_softmax(x))), nd.array(y))
    assert_almost_equal(out.asnumpy(), ref, rtol=1e-5, atol=1e-6)
    w = rng.rand(6, 1).astype('float32')
    out = gluon.loss.SoftmaxCrossEntropyLoss(weight=2.0)(nd.array(x), nd.array(y), nd.array(w))
    assert_almost_equal(out.asnumpy(), ref * 2 * w[:, 0], rtol=1e-5, atol=1e-6)
    x3 = rng.randn(2, 4, 5).astype('float32')
    y3 = rng.randint(0, 5, (2, 4))
    out = gluon.loss.SoftmaxCrossEntropyLoss(axis=-1)(nd.array(x3), nd.array(y3))
    ref3 = -np.log(_softmax(x3)[np.arange(2)[:, None], np.arange(4)[None], y3]).mean(1)
    assert_almost_equal(out.asnumpy(), ref3, rtol=1e-5, atol=1e-6)


def test_regression_losses():
    p, t = rng.randn(4, 3).astype('float32'), rng.randn(4, 3).astype('float32')
    assert_almost_equal(gluon.loss.L2Loss()(nd.array(p), nd.array(t)).asnumpy(), 0.5 * ((p - t) ** 2).mean(1), rtol=1e-5)
    assert_almost_equal(gluon.loss.L1Loss()(nd.array(p), nd.array(t)).asnumpy(), np.abs(p - t).mean(1), rtol=1e-5)
    d = np.abs(p - t)
    hub = np.where(d > 1.0, d - 0.5, 0.5 * d ** 2).mean(1)
    assert_almost_equal(gluon.loss.HuberLoss(rho=1.0)(nd.array(p), nd.array(t)).asnumpy(), hub, rtol=1e-5)
    lab = np.sign(t)
    assert_almost_equal(gluon.loss.HingeLoss()(nd.array(p), nd.array(lab)).asnumpy(), np.maximum(0, 1 - p * lab).mean(1), rtol=1e-5)
    assert_almost_equal(gluon.loss.SquaredHingeLoss()(nd.array(p), nd.array(lab)).asnumpy(),
                        (np.maximum(0, 1 - p * lab) ** 2).mean(1), rtol=1e-5)
    assert_almost_equal(gluon.loss.LogisticLoss()(nd.array(p), nd.array(lab)).asnumpy(), np.log1p(np.exp(-p * lab)).mean(1),
                        rtol=1e-4)


def test_bce_kl_cosine_triplet_poisson():
    z = rng.randn(5, 4).astype('float32')
    y = (rng.rand(5, 4) > 0.5).astype('float32')
    ref = (np.maximum(z, 0) - z * y + np.log1p(np.exp(-np.abs(z)))).mean(1)
    assert_almost_equal(gluon.loss.SigmoidBinaryCrossEntropyLoss()(nd.array(z), nd.array(y)).asnumpy(), ref, rtol=1e-5)
    p = 1 / (1 + np.exp(-z))
    out = gluon.loss.SigmoidBCELoss(from_sigmoid=True)(nd.array(p), nd.array(y))
    assert_almost_equal(out.asnumpy(), ref, rtol=1e-4, atol=1e-5)
    q = _softmax(rng.randn(3, 6)).astype('float32')
    logp = np.log(_softmax(rng.randn(3, 6))).astype('float32')
    kl = (q * (np.log(q + 1e-12) - logp)).mean(1)
    assert_almost_equal(gluon.loss.KLDivLoss()(nd.array(logp), nd.array(q)).asnumpy(), kl, rtol=1e-4, atol=1e-6)
    a, b = rng.randn(4, 8).astype('float32'), rng.randn(4, 8).astype('float32')
    lab = np.array([1, -1, 1, -1], 'float32')
    cos = (a * b).sum(1) / (np.linalg.norm(a, axis=1) * np.linalg.norm(b, axis=1) + 1e-12)
    ref = np.where(lab == 1, 1 - cos, np.maximum(0, cos))
    assert_almost_equal(gluon.loss.CosineEmbeddingLoss()(nd.array(a), nd.array(b), nd.array(lab)).asnumpy().ravel(), ref,
                        rtol=1e-4, atol=1e-6)
    pos, neg = rng.randn(4, 8).astype('float32'), rng.randn(4, 8).astype('float32')
    ref = np.maximum(((a - pos) ** 2 - (a - neg) ** 2).sum(1) + 1.0, 0)
    assert_almost_equal(gluon.loss.TripletLoss(margin=1.0)(nd.array(a), nd.array(pos), nd.array(neg)).asnumpy(), ref, rtol=1e-4)
    rate, tgt = np.abs(rng.randn(4, 3)).astype('float32') + 0.1, rng.poisson(2, (4, 3)).astype('float32')
    out = gluon.loss.PoissonNLLLoss(from_logits=False)(nd.array(rate), nd.array(tgt))
    assert_almost_equal(out.asnumpy(), (rate - tgt * np.log(rate + 1e-8)).mean(1), rtol=1e-4)     # one value per sample


def test_ctc_loss_simple_case():
    # a single time step with a single label: loss = -log softmax(x)[label]
    x = rng.randn(1, 1, 4).astype('float32')          # (N, T, C), blank = last class by default
    out = gluon.loss.CTCLoss(layout='NTC')(nd.array(x), nd.array([[1]]))
    assert_almost_equal(out.asnumpy(), -np.log(_softmax(x[0, 0])[1]), rtol=1e-4)


def test_accuracy_topk_f1_mcc():
    pred = nd.array([[0.3, 0.7], [0.6, 0.4], [0.2, 0.8], [0.9, 0.1]])
    label = nd.array([1, 1, 1, 0])
    acc = mx.metric.Accuracy()
    acc.update([label], [pred])
    assert acc.get() == ('accuracy', 0.75)
    acc.reset()
    assert np.isnan(acc.get()[1])
    topk = mx.metric.TopKAccuracy(top_k=2)
    topk.update([nd.array([2, 0])], [nd.array([[0.1, 0.5, 0.4], [0.2, 0.5, 0.3]])])
    assert topk.get()[1] == 0.5
    f1 = mx.metric.F1()
    f1.update([label], [pred])
    # tp=2 (rows 0,2), fp=0, fn=1
    assert abs(f1.get()[1] - 2 * 1.0 * (2 / 3) / (1.0 + 2 / 3)) < 1e-6
    mcc = mx.metric.MCC()
    mcc.update([label], [pred])
    tp, tn, fp, fn = 2, 1, 0, 1
    ref = (tp * tn - fp * fn) / np.sqrt((tp + fp) * (tp + fn) * (tn + fp) * (tn + fn))
    assert abs(mcc.get()[1] - ref) < 1e-6


def test_regression_and_probabilistic_metrics():
    p, t = rng.rand(8, 1).astype('float32'), rng.rand(8, 1).astype('float32')
    for cls, ref in ((mx.metric.MAE, np.abs(p - t).mean()), (mx.metric.MSE, ((p - t) ** 2).mean()),
                     (mx.metric.RMSE, np.sqrt(((p - t) ** 2).mean()))):
        m = cls()
        m.update([nd.array(t)], [nd.array(p)])
        assert abs(m.get()[1] - ref) < 1e-5
    probs = _softmax(rng.randn(6, 4)).astype('float32')
    lab = rng.randint(0, 4, (6,))
    ce = mx.metric.CrossEntropy()
    ce.update([nd.array(lab)], [nd.array(probs)])
    assert abs(ce.get()[1] - (-np.log(probs[np.arange(6), lab] + 1e-12)).mean()) < 1e-5
    ppl = mx.metric.Perplexity(ignore_label=None)
    ppl.update([nd.array(lab)], [nd.array(probs)])
    assert abs(ppl.get()[1] - np.exp((-np.log(probs[np.arange(6), lab])).mean())) < 1e-3
    pc = mx.metric.PearsonCorrelation()
    pc.update([nd.array(t)], [nd.array(p)])
    assert abs(pc.get()[1] - np.corrcoef(p.ravel(), t.ravel())[0, 1]) < 1e-5


def test_composite_custom_and_create():
    comp = mx.metric.CompositeEvalMetric()
    comp.add(mx.metric.Accuracy())
    comp.add(mx.metric.create('mse'))
    names, _ = comp.get()
    assert names == ['accuracy', 'mse']
    m = mx.metric.create(['acc', 'ce'])
    assert isinstance(m, mx.metric.CompositeEvalMetric)
    cm = mx.metric.np(lambda label, pred: float(np.abs(label - pred).sum()), name='sad')
    cm.update([nd.array([1., 2.])], [nd.array([1.5, 2.5])])
    assert cm.get() == ('sad', 1.0)
    loss = mx.metric.Loss()
    loss.update(None, [nd.array([1., 3.])])
    assert loss.get()[1] == 2.0
    assert dict(mx.metric.Accuracy().get_name_value()).keys() == {'accuracy'}

"""Optimizer update rules against NumPy restatements of the reference formulas
(python/mxnet/optimizer/*.py ``step``; src/operator/optimizer_op-inl.h), plus Updater, multi-precision,
lr schedulers and the registry."""
import math
import pickle

import numpy as np
import pytest

import mxnet_b200 as mx
from mxnet_b200 import nd, optimizer as opt
from mxnet_b200.test_utils import assert_almost_equal

SHAPE = (3, 4)


def _prep(g, w, rescale=1.0, clip=None, wd=0.0):
    g = g * rescale
    if clip is not None:
        g = np.clip(g, -clip, clip)
    return g + wd * w


class _Oracle(object):
    """Each method: (weight, grad, state, t) -> weight, state; all float64 NumPy."""

    @staticmethod
    def sgd(w, g, s, t, lr=0.1, wd=0.01, momentum=0.9, rescale=0.5, clip=0.4):
        g = _prep(g, w, rescale, clip, wd)
        m = s if s is not None else np.zeros_like(w)
        m = momentum * m - lr * g
        return w + m, m

    @staticmethod
    def sgd_nomom(w, g, s, t, lr=0.1, wd=0.01, rescale=0.5):
        return w - lr * _prep(g, w, rescale, None, wd), None

    @staticmethod
    def nag(w, g, s, t, lr=0.1, wd=0.01, momentum=0.9):
        g = _prep(g, w, 1.0, None, wd)
        m = s if s is not None else np.zeros_like(w)
        m = momentum * m - lr * g
        return w + momentum * m - lr * g, m

    @staticmethod
    def adam(w, g, s, t, lr=0.01, wd=0.01, b1=0.9, b2=0.999, eps=1e-8):
        g = _prep(g, w, 1.0, None, wd)
        m, v = s if s is not None else (np.zeros_like(w), np.zeros_like(w))
        lr = lr * math.sqrt(1 - b2 ** t) / (1 - b1 ** t)
        m = b1 * m + (1 - b1) * g
        v = b2 * v + (1 - b2) * g * g
        return w - lr * m / (np.sqrt(v) + eps), (m, v)

    @staticmethod
    def adamw(w, g, s, t, lr=0.01, wd=0.1, b1=0.9, b2=0.999, eps=1e-6):
        m, v = s if s is not None else (np.zeros_like(w), np.zeros_like(w))
        lr = lr * math.sqrt(1 - b2 ** t) / (1 - b1 ** t)
        m = b1 * m + (1 - b1) * g
        v = b2 * v + (1 - b2) * g * g
        w = w - lr * m / (np.sqrt(v) + eps)
        return w - lr * wd * w, (m, v)

    @staticmethod
    def rmsprop(w, g, s, t, lr=0.01, wd=0.0, rho=0.9, eps=1e-8):
        g = _prep(g, w, 1.0, None, wd)
        v = s if s is not None else np.zeros_like(w)
        v = rho * v + (1 - rho) * g * g
        return w - lr * g / (np.sqrt(v) + eps), v

    @staticmethod
    def rmsprop_centered(w, g, s, t, lr=0.01, rho=0.9, momentum=0.9, eps=1e-8):
        mean, var, mom = s if s is not None else (np.zeros_like(w),) * 3
        mean = rho * mean + (1 - rho) * g
        var = rho * var + (1 - rho) * g * g
        mom = momentum * mom - lr * g / np.sqrt(var - mean * mean + eps)
        return w + mom, (mean, var, mom)

    @staticmethod
    def adagrad(w, g, s, t, lr=0.1, wd=0.01, eps=1e-6):
        g = _prep(g, w, 1.0, None, wd)
        h = (s if s is not None else np.zeros_like(w)) + g * g
        return w - lr * g / (np.sqrt(h) + eps), h

    @staticmethod
    def adadelta(w, g, s, t, lr=1.0, rho=0.9, eps=1e-6):
        ag, ad = s if s is not None else (np.zeros_like(w), np.zeros_like(w))
        ag = rho * ag + (1 - rho) * g * g
        d = np.sqrt(ad + eps) / np.sqrt(ag + eps) * g
        ad = rho * ad + (1 - rho) * d * d
        return w - lr * d, (ag, ad)

    @staticmethod
    def signum(w, g, s, t, lr=0.01, wd=0.01, momentum=0.9, wd_lh=0.001):
        g = _prep(g, w, 1.0, None, wd)
        m = s if s is not None else np.zeros_like(w)
        m = momentum * m - (1 - momentum) * g
        return w * (1 - lr * wd_lh) + lr * np.sign(m), m

    @staticmethod
    def ftrl(w, g, s, t, lr=0.1, wd=0.01, lamda1=0.01, beta=1.0):
        z, n = s if s is not None else (np.zeros_like(w), np.zeros_like(w))
        sigma = -np.sqrt(n)
        n = n + g * g
        denom = np.sqrt(n)
        sigma = (sigma + denom) / lr
        z = z + g - sigma * w
        denom = (denom + beta) / lr + wd
        return -np.sign(z) * np.maximum(np.abs(z) - lamda1, 0) / denom, (z, n)

    @staticmethod
    def adamax(w, g, s, t, lr=0.002, wd=0.0, b1=0.9, b2=0.999, eps=1e-8):
        m, u = s if s is not None else (np.zeros_like(w), np.zeros_like(w))
        m = b1 * m + (1 - b1) * g
        u = np.maximum(b2 * u, np.abs(g))
        return w - lr / (1 - b1 ** t) * m / (u + eps), (m, u)

    @staticmethod
    def lamb(w, g, s, t, lr=0.01, wd=0.01, b1=0.9, b2=0.999, eps=1e-6):
        m, v = s if s is not None else (np.zeros_like(w), np.zeros_like(w))
        m = b1 * m + (1 - b1) * g
        v = b2 * v + (1 - b2) * g * g
        mh, vh = m / (1 - b1 ** t), v / (1 - b2 ** t)
        u = mh / (np.sqrt(vh) + eps) + wd * w
        r1, r2 = np.linalg.norm(w), np.linalg.norm(u)
        ratio = r1 / r2 if (r1 > 0 and r2 > 0) else 1.0
        return w - lr * ratio * u, (m, v)


CASES = [
    ('sgd', dict(learning_rate=0.1, wd=0.01, momentum=0.9, rescale_grad=0.5, clip_gradient=0.4), _Oracle.sgd, 1e-5),
    ('sgd', dict(learning_rate=0.1, wd=0.01, rescale_grad=0.5), _Oracle.sgd_nomom, 1e-5),
    ('nag', dict(learning_rate=0.1, wd=0.01, momentum=0.9), _Oracle.nag, 1e-5),
    ('adam', dict(learning_rate=0.01, wd=0.01), _Oracle.adam, 1e-4),
    ('adamw', dict(learning_rate=0.01, wd=0.1), _Oracle.adamw, 1e-4),
    ('rmsprop', dict(learning_rate=0.01), _Oracle.rmsprop, 1e-4),
    ('rmsprop', dict(learning_rate=0.01, centered=True, momentum=0.9), _Oracle.rmsprop_centered, 1e-4),
    ('adagrad', dict(learning_rate=0.1, wd=0.01), _Oracle.adagrad, 1e-5),
    ('adadelta', dict(learning_rate=1.0), _Oracle.adadelta, 1e-4),
    ('signum', dict(learning_rate=0.01, wd=0.01, momentum=0.9, wd_lh=0.001), _Oracle.signum, 1e-5),
    ('ftrl', dict(learning_rate=0.1, wd=0.01), _Oracle.ftrl, 1e-4),
    ('adamax', dict(learning_rate=0.002), _Oracle.adamax, 1e-5),
    ('lamb', dict(learning_rate=0.01, wd=0.01), _Oracle.lamb, 1e-4),
]


@pytest.mark.parametrize('name,kwargs,oracle,tol', CASES, ids=['%s-%d' % (c[0], i) for i, c in enumerate(CASES)])
@pytest.mark.parametrize('aggregate', [False, True])
def test_update_rule(name, kwargs, oracle, tol, aggregate):
    rng = np.random.RandomState(0)
    o = opt.create(name, **kwargs)
    if not aggregate:
        o.aggregate_num = 1
    upd = opt.get_updater(o)
    w_np = [rng.randn(*SHAPE), rng.randn(5)]
    ws = [nd.array(w) for w in w_np]
    states = [None, None]
    for t in range(1, 5):
        gs_np = [rng.randn(*w.shape) for w in w_np]
        upd([0, 1], [nd.array(g) for g in gs_np], ws)
        for i in range(2):
            w_np[i], states[i] = oracle(w_np[i], gs_np[i], states[i], t)
            assert_almost_equal(ws[i].asnumpy(), w_np[i].astype('float32'), rtol=tol * 10, atol=tol)


def test_multi_precision_keeps_fp32_master():
    o = opt.create('sgd', learning_rate=0.1, momentum=0.9, multi_precision=True)
    w = nd.array(np.full((4,), 1.0), dtype='float16')
    state = o.create_state_multi_precision(0, w)
    assert isinstance(state, tuple) and state[0].dtype == np.float32
    master = np.full((4,), 1.0, 'float64')
    mom = np.zeros(4)
    for _ in range(20):
        g = nd.array(np.full((4,), 1e-4), dtype='float16')
        o.update_multi_precision([0], [w], [g], [state])
        mom = 0.9 * mom - 0.1 * float(np.float16(1e-4))
        master = master + mom
    assert_almost_equal(state[0].asnumpy(), master.astype('float32'), rtol=1e-5)
    assert_almost_equal(w.asnumpy(), master.astype('float16'), rtol=1e-3)
    # without a master copy the same tiny steps would be lost to fp16 rounding
    assert abs(float(state[0].asnumpy()[0]) - 1.0) > 1e-4


def test_lr_wd_mult_and_param_dict():
    o = opt.create('sgd', learning_rate=1.0, wd=0.1)
    o.set_lr_mult({0: 0.5})
    o.set_wd_mult({0: 0.0})
    w = nd.ones((2,))
    o.update([0], [w], [nd.ones((2,))], [o.create_state(0, w)])
    assert_almost_equal(w.asnumpy(), np.array([0.5, 0.5]))
    o.set_wd_mult({})
    assert o.wd_mult == {}


def test_update_count_and_lr_scheduler():
    sched = mx.lr_scheduler.FactorScheduler(step=2, factor=0.5, base_lr=1.0)
    o = opt.create('sgd', learning_rate=1.0, lr_scheduler=sched)
    w = nd.zeros((1,))
    lrs = []
    for _ in range(6):
        o.update([0], [w], [nd.zeros((1,))], [None])
        lrs.append(o.learning_rate)
    assert o.num_update == 6
    assert lrs[0] == 1.0 and lrs[-1] == 0.25
    with pytest.raises(UserWarning):
        o.set_learning_rate(0.1)


def test_lr_schedulers_values():
    s = mx.lr_scheduler.MultiFactorScheduler(step=[3, 6], factor=0.1, base_lr=1.0)
    assert [round(s(i), 6) for i in (1, 3, 4, 6, 7)] == [1.0, 1.0, 0.1, 0.1, 0.01]
    s = mx.lr_scheduler.PolyScheduler(max_update=10, base_lr=1.0, pwr=2, final_lr=0.0)
    assert abs(s(5) - 0.25) < 1e-9 and s(10) == 0.0 and s(20) == 0.0
    s = mx.lr_scheduler.CosineScheduler(max_update=10, base_lr=1.0, final_lr=0.0)
    assert abs(s(5) - 0.5) < 1e-9
    s = mx.lr_scheduler.FactorScheduler(step=10, factor=0.5, base_lr=1.0, warmup_steps=4, warmup_begin_lr=0.0)
    assert abs(s(2) - 0.5) < 1e-9


def test_updater_states_round_trip():
    o = opt.create('adam', learning_rate=0.01)
    upd = opt.get_updater(o)
    w = nd.ones((3,))
    upd(0, nd.ones((3,)), w)
    blob = upd.get_states(dump_optimizer=True)
    upd2 = opt.get_updater(opt.create('adam', learning_rate=0.01))
    upd2.set_states(blob)
    assert_almost_equal(upd2.states[0][0].asnumpy(), upd.states[0][0].asnumpy())
    assert upd2.optimizer.num_update == 1
    states, _ = pickle.loads(blob)
    assert 0 in states


def test_registry_and_create_errors():
    assert isinstance(opt.create('SGD'), opt.SGD)
    assert isinstance(opt.Optimizer.create_optimizer('adam'), opt.Adam)
    with pytest.raises(ValueError):
        opt.create('no_such_optimizer')

    @opt.register
    class MyOpt(opt.Optimizer):
        def create_state(self, index, weight):
            return None

        def step(self, indices, weights, grads, states):
            for w, g in zip(weights, grads):
                w[:] = w - g
    o = opt.create('myopt')
    w = nd.ones((2,))
    o.update([0], [w], [nd.ones((2,))], [None])
    assert float(w.sum().asscalar()) == 0


def test_sgld_and_lars_run():
    mx.random.seed(0)
    o = opt.create('sgld', learning_rate=0.01)
    w = nd.zeros((1000,))
    o.update([0], [w], [nd.zeros((1000,))], [o.create_state(0, w)])
    assert 0.05 < float(w.asnumpy().std()) < 0.2          # N(0, sqrt(lr)) noise
    o = opt.create('lars', learning_rate=0.1, momentum=0.9, eta=0.001)
    w = nd.ones((4, 4))
    st = o.create_state(0, w)
    o.update([0], [w], [nd.ones((4, 4))], [st])
    assert float(w.asnumpy().mean()) < 1.0

"""gluon.probability: densities, sampling moments, KL divergences and transformations against closed forms."""
import math

import numpy as np
import pytest

import mxnet_b200 as mx
from mxnet_b200 import autograd, np as mnp
from mxnet_b200.gluon import probability as mgp


def _np(x):
    return x.asnumpy() if hasattr(x, 'asnumpy') else np.asarray(x)


def test_normal_log_prob_cdf_entropy_and_sampling():
    loc, scale = mnp.array([0.0, 1.0]), mnp.array([1.0, 2.0])
    d = mgp.Normal(loc, scale)
    x = mnp.array([0.5, -1.0])
    ref = -0.5 * ((_np(x) - _np(loc)) / _np(scale)) ** 2 - np.log(_np(scale)) - 0.5 * math.log(2 * math.pi)
    np.testing.assert_allclose(_np(d.log_prob(x)), ref, rtol=1e-5)
    np.testing.assert_allclose(_np(d.cdf(loc)), [0.5, 0.5], atol=1e-6)
    np.testing.assert_allclose(_np(d.entropy()), 0.5 * np.log(2 * math.pi * math.e * _np(scale) ** 2), rtol=1e-5)
    mx.random.seed(3)
    s = _np(d.sample((20000,)))
    assert s.shape == (20000, 2)
    np.testing.assert_allclose(s.mean(0), [0.0, 1.0], atol=0.06)
    np.testing.assert_allclose(s.std(0), [1.0, 2.0], rtol=0.05)


def test_reparameterised_sample_carries_gradient():
    loc = mnp.array([0.3])
    scale = mnp.array([1.5])
    loc.attach_grad()
    scale.attach_grad()
    mx.random.seed(0)
    with autograd.record():
        z = mgp.Normal(loc, scale).sample((64,))
        loss = (z * z).mean()
    loss.backward()
    assert abs(float(_np(loc.grad)[0])) > 0 and abs(float(_np(scale.grad)[0])) > 0


@pytest.mark.parametrize('name,kwargs,mean,var', [
    ('Bernoulli', {'prob': 0.3}, 0.3, 0.21),
    ('Exponential', {'scale': 2.0}, 2.0, 4.0),
    ('Gamma', {'shape': 3.0, 'scale': 2.0}, 6.0, 12.0),
    ('Poisson', {'rate': 4.0}, 4.0, 4.0),
    ('Uniform', {'low': -1.0, 'high': 3.0}, 1.0, 16.0 / 12.0),
    ('Laplace', {'loc': 1.0, 'scale': 0.5}, 1.0, 0.5),
    ('Beta', {'alpha': 2.0, 'beta': 5.0}, 2.0 / 7.0, 10.0 / (49.0 * 8.0)),
    ('Geometric', {'prob': 0.25}, 3.0, 12.0),
])
def test_distribution_moments(name, kwargs, mean, var):
    d = getattr(mgp, name)(**{k: mnp.array([v]) for k, v in kwargs.items()})
    np.testing.assert_allclose(_np(d.mean), [mean], rtol=1e-5)
    np.testing.assert_allclose(_np(d.variance), [var], rtol=1e-5)
    mx.random.seed(1)
    s = _np(d.sample((40000,))).astype('float64')
    np.testing.assert_allclose(s.mean(), mean, atol=4 * math.sqrt(var / 40000) + 1e-3)


def test_categorical_and_one_hot():
    p = mnp.array([[0.1, 0.2, 0.7]])
    c = mgp.Categorical(3, prob=p)
    np.testing.assert_allclose(_np(c.log_prob(mnp.array([2]))), [math.log(0.7)], rtol=1e-5)
    mx.random.seed(2)
    s = _np(c.sample((20000,))).reshape(-1)
    np.testing.assert_allclose(np.bincount(s.astype(int), minlength=3) / 20000.0, [0.1, 0.2, 0.7], atol=0.02)
    oh = mgp.OneHotCategorical(3, prob=p)
    v = _np(oh.sample((5,)))
    assert v.shape[-1] == 3 and np.allclose(v.sum(-1), 1.0)


def test_kl_divergence_closed_forms():
    p = mgp.Normal(mnp.array([0.0]), mnp.array([1.0]))
    q = mgp.Normal(mnp.array([1.0]), mnp.array([2.0]))
    ref = math.log(2.0) + (1.0 + 1.0) / (2 * 4.0) - 0.5
    np.testing.assert_allclose(_np(mgp.kl_divergence(p, q)), [ref], rtol=1e-5)
    b1, b2 = mgp.Bernoulli(prob=mnp.array([0.3])), mgp.Bernoulli(prob=mnp.array([0.6]))
    refb = 0.3 * math.log(0.3 / 0.6) + 0.7 * math.log(0.7 / 0.4)
    np.testing.assert_allclose(_np(mgp.kl_divergence(b1, b2)), [refb], rtol=1e-5)


def test_transformed_distribution_log_prob():
    base = mgp.Normal(mnp.array([0.0]), mnp.array([1.0]))
    d = mgp.TransformedDistribution(base, [mgp.ExpTransform()])          # log-normal
    x = mnp.array([1.7])
    ref = -0.5 * math.log(1.7) ** 2 - 0.5 * math.log(2 * math.pi) - math.log(1.7)
    np.testing.assert_allclose(_np(d.log_prob(x)), [ref], rtol=1e-5)
    aff = mgp.TransformedDistribution(base, [mgp.AffineTransform(loc=mnp.array([2.0]), scale=mnp.array([3.0]))])
    ref2 = -0.5 * ((5.0 - 2.0) / 3.0) ** 2 - 0.5 * math.log(2 * math.pi) - math.log(3.0)
    np.testing.assert_allclose(_np(aff.log_prob(mnp.array([5.0]))), [ref2], rtol=1e-5)


def test_multivariate_normal_and_independent():
    cov = np.array([[2.0, 0.3], [0.3, 1.0]], dtype='float32')
    loc = np.array([1.0, -1.0], dtype='float32')
    d = mgp.MultivariateNormal(mnp.array(loc), cov=mnp.array(cov))
    x = np.array([0.5, 0.2], dtype='float32')
    diff = x - loc
    ref = -0.5 * diff @ np.linalg.inv(cov) @ diff - 0.5 * math.log(np.linalg.det(cov)) - math.log(2 * math.pi)
    np.testing.assert_allclose(_np(d.log_prob(mnp.array(x))), ref, rtol=1e-4)
    ind = mgp.Independent(mgp.Normal(mnp.zeros((3, 4)), mnp.ones((3, 4))), 1)
    lp = _np(ind.log_prob(mnp.zeros((3, 4))))
    assert lp.shape == (3,)
    np.testing.assert_allclose(lp, 4 * (-0.5 * math.log(2 * math.pi)), rtol=1e-5)


def test_stochastic_block_collects_losses():
    class VAEish(mgp.StochasticBlock):
        def __init__(self):
            super().__init__()
            self.dense = mx.gluon.nn.Dense(2, in_units=3)

        @mgp.StochasticBlock.collectLoss
        def forward(self, x):
            h = self.dense(x)
            q = mgp.Normal(h, mnp.ones_like(h))
            self.add_loss(mgp.kl_divergence(q, mgp.Normal(mnp.zeros_like(h), mnp.ones_like(h))))
            return h

    net = VAEish()
    net.initialize()
    out = net(mnp.ones((4, 3)))
    assert out.shape == (4, 2) and len(net.losses) == 1 and net.losses[0].shape == (4, 2)


def test_constraints_and_distribution_utils():
    from mxnet_b200.gluon.probability.distributions import constraint as C, utils as U
    import mxnet_b200.gluon.probability.distributions.constraint as C2
    assert C is C2
    mx.npx.set_np()
    try:
        v = mx.np.array([0.2, 0.8])
        assert C.UnitInterval().check(v) is v and C.Simplex().check(v) is v and C.Real().check(v) is v
        bad = [(C.Positive(), [-1.0]), (C.NonNegative(), [-0.5]), (C.IntegerInterval(0, 5), [1.5]), (C.OpenInterval(0, 1), [1.0]),
               (C.HalfOpenInterval(0, 1), [1.0]), (C.LessThan(2), [2.0]), (C.LessThanEq(2), [2.5]), (C.GreaterThanEq(1), [0.5]),
               (C.PositiveInteger(), [0.0]), (C.NonNegativeInteger(), [0.5]), (C.Boolean(), [2.0]), (C.Simplex(), [0.5, 0.6]),
               (C.LowerTriangular(), [[1., 2.], [0., 1.]]), (C.LowerCholesky(), [[-1., 0.], [0., 1.]]),
               (C.PositiveDefinite(), [[1., 2.], [2., 1.]])]
        for c, value in bad:
            with pytest.raises(ValueError, match='Constraint violated'):
                c.check(mx.np.array(value))
        ok = [(C.HalfOpenInterval(0, 1), [0.0]), (C.IntegerGreaterThan(1), [2.0]), (C.IntegerLessThanEq(3), [3.0]),
              (C.LowerCholesky(), [[1., 0.], [2., 3.]]), (C.PositiveDefinite(), [[2., 1.], [1., 2.]])]
        for c, value in ok:
            c.check(mx.np.array(value))
        assert C.Stack([C.Positive(), C.Real()]).check(mx.np.array([1.0, -3.0])).shape == (2,)
        with pytest.raises(ValueError):
            C.Cat([C.Positive(), C.NonNegative()], lengths=[1, 2]).check(mx.np.array([1.0, -1.0, 2.0]))
        assert C.is_dependent(C.dependent) and not C.is_dependent(C.Real())
        np.testing.assert_allclose(U.prob2logit(mx.np.array([0.5])).asnumpy(), [0.0], atol=1e-6)
        np.testing.assert_allclose(U.logit2prob(mx.np.array([[0.0, 0.0]]), False).asnumpy(), [[0.5, 0.5]])
        np.testing.assert_allclose(U.prob2logit(mx.np.array([0.25, 0.75]), False).asnumpy(), np.log([0.25, 0.75]), rtol=1e-6)
        assert U.sample_n_shape_converter(3) == (3,) and U.sample_n_shape_converter(None) == ()
        np.testing.assert_allclose(U.gammaln()(mx.np.array([4.0])).asnumpy(), [np.log(6.0)], rtol=1e-6)

        class Holder(object):
            calls = 0

            @U.cached_property
            def value(self):
                Holder.calls += 1
                return 7
        h = Holder()
        assert h.value == 7 and h.value == 7 and Holder.calls == 1
    finally:
        mx.npx.reset_np()

"""Minimum end-to-end slice on CPU: Gluon MLP 784-256-128-10, SoftmaxCrossEntropy, SGD momentum,
kvstore='local' over two CPU contexts, 100 steps, then a .params round trip."""
import os

import numpy as np

import mxnet_b200 as mx
from mxnet_b200 import autograd, gluon, nd
from mxnet_b200.gluon import nn


def _build():
    net = nn.HybridSequential()
    net.add(nn.Dense(256, activation='relu'), nn.Dense(128, activation='relu'), nn.Dense(10))
    return net


def test_mlp_two_cpu_contexts_trains_and_round_trips(tmp_path):
    mx.random.seed(0)
    np.random.seed(0)
    ctxs = [mx.cpu(0), mx.cpu(1)]
    net = _build()
    net.initialize(mx.init.Xavier(), ctx=ctxs)
    loss_fn = gluon.loss.SoftmaxCrossEntropyLoss()
    trainer = gluon.Trainer(net.collect_params(), 'sgd', {'learning_rate': 0.1, 'momentum': 0.9}, kvstore='local')
    x = np.random.uniform(0, 1, (64, 784)).astype('float32')
    y = np.random.randint(0, 10, (64,)).astype('float32')
    net(nd.array(x[:2]).as_in_context(ctxs[0]))      # finish deferred initialisation
    # independent oracle: the same MLP and update rule written directly against the tensor library
    import torch
    ws = [p.data(ctxs[0])._data.detach().clone().requires_grad_(True) for p in net.collect_params().values()]
    moms = [torch.zeros_like(w) for w in ws]
    xt, yt = torch.tensor(x), torch.tensor(y).long()
    first = last = None
    for step in range(100):
        h = torch.relu(xt @ ws[0].t() + ws[1])
        h = torch.relu(h @ ws[2].t() + ws[3])
        ref_loss = torch.nn.functional.cross_entropy(h @ ws[4].t() + ws[5], yt)
        gs = torch.autograd.grad(ref_loss, ws)
        with torch.no_grad():
            for w, m, g in zip(ws, moms, gs):
                m.mul_(0.9).add_(g, alpha=-0.1)
                w.add_(m)
        xs = gluon.utils.split_and_load(nd.array(x), ctxs)
        ys = gluon.utils.split_and_load(nd.array(y), ctxs)
        with autograd.record():
            losses = [loss_fn(net(a), b) for a, b in zip(xs, ys)]
        for l in losses:
            l.backward()
        trainer.step(64)
        cur = float(sum(l.mean().asscalar() for l in losses) / len(losses))
        if step == 10:
            # the update rule is exact against the oracle while rounding noise is still small (this
            # learning rate makes the problem chaotic later on, so end-of-run weights are not compared)
            for p, w in zip(net.collect_params().values(), ws):
                np.testing.assert_allclose(p.data(ctxs[0]).asnumpy(), w.detach().numpy(), rtol=1e-4, atol=1e-5)
        first = cur if first is None else first
        last = cur
    assert np.isfinite(last), (first, last)
    # replicas stay in sync
    for p in net.collect_params().values():
        a, b = [d.asnumpy() for d in p.list_data()]
        np.testing.assert_allclose(a, b, rtol=1e-6, atol=1e-7)
    f = str(tmp_path / 'mlp.params')
    net.save_parameters(f)
    net2 = _build()
    net2.load_parameters(f, ctx=mx.cpu(0))
    xt = nd.array(x)
    np.testing.assert_allclose(net(xt.as_in_context(ctxs[0])).asnumpy(), net2(xt).asnumpy(), rtol=1e-5, atol=1e-6)
    # the container is the reference's binary format: list magic 0x112 then reserved 0
    with open(f, 'rb') as fh:
        head = fh.read(16)
    assert int.from_bytes(head[:8], 'little') == 0x112 and int.from_bytes(head[8:], 'little') == 0

#!/usr/bin/env python
"""MNIST with Gluon: MLP or LeNet, imperative or hybridized (the flow of example/gluon/mnist/mnist.py in MXNet).

    python example/gluon/mnist/mnist.py --epochs 2 [--gpu] [--hybridize] [--net lenet] [--data-dir DIR]

Without `--data-dir` (the four idx files of MNIST) the script trains on a synthetic, linearly separable stand-in of
the same shape so that it runs with no data set at hand."""
import argparse
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), '..', '..', '..'))
import mxnet_b200 as mx                                    # noqa: E402
from mxnet_b200 import autograd, gluon                     # noqa: E402
from mxnet_b200.gluon import nn                            # noqa: E402


def synthetic(n, rng):
    """28x28 images whose class is readable from ten fixed random templates plus noise."""
    templates = np.random.RandomState(42).rand(10, 28, 28).astype('float32')
    y = rng.randint(0, 10, n)
    x = templates[y] + 0.3 * rng.randn(n, 28, 28).astype('float32')
    return x[:, None], y.astype('float32')


def build(kind):
    net = nn.HybridSequential()
    if kind == 'mlp':
        net.add(nn.Flatten(), nn.Dense(128, activation='relu'), nn.Dense(64, activation='relu'), nn.Dense(10))
    else:
        net.add(nn.Conv2D(20, 5, activation='tanh'), nn.MaxPool2D(2, 2), nn.Conv2D(50, 5, activation='tanh'), nn.MaxPool2D(2, 2),
                nn.Flatten(), nn.Dense(500, activation='tanh'), nn.Dense(10))
    return net


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--epochs', type=int, default=2)
    ap.add_argument('--batch-size', type=int, default=100)
    ap.add_argument('--lr', type=float, default=0.1)
    ap.add_argument('--momentum', type=float, default=0.9)
    ap.add_argument('--net', default='mlp', choices=['mlp', 'lenet'])
    ap.add_argument('--gpu', action='store_true')
    ap.add_argument('--hybridize', action='store_true')
    ap.add_argument('--data-dir', default=None)
    ap.add_argument('--samples', type=int, default=6000, help='size of the synthetic training set')
    args = ap.parse_args(argv)
    ctx = mx.gpu(0) if args.gpu else mx.cpu()
    if args.data_dir:
        tf = lambda d, l: (d.astype('float32').transpose((2, 0, 1)) / 255, np.float32(l))
        train = gluon.data.vision.MNIST(args.data_dir, train=True).transform(tf)
        val = gluon.data.vision.MNIST(args.data_dir, train=False).transform(tf)
    else:
        rng = np.random.RandomState(0)
        train = gluon.data.ArrayDataset(*synthetic(args.samples, rng))
        val = gluon.data.ArrayDataset(*synthetic(args.samples // 6, rng))
    train_data = gluon.data.DataLoader(train, args.batch_size, shuffle=True, last_batch='discard')
    val_data = gluon.data.DataLoader(val, args.batch_size)
    net = build(args.net)
    net.initialize(mx.init.Xavier(magnitude=2.24), ctx=ctx)
    if args.hybridize:
        net.hybridize()
    trainer = gluon.Trainer(net.collect_params(), 'sgd', {'learning_rate': args.lr, 'momentum': args.momentum})
    loss_fn = gluon.loss.SoftmaxCrossEntropyLoss()
    acc = 0.0
    for epoch in range(args.epochs):
        metric = gluon.metric.Accuracy()
        for x, y in train_data:
            x, y = x.as_in_context(ctx), y.as_in_context(ctx)
            with autograd.record():
                out = net(x)
                loss = loss_fn(out, y)
            loss.backward()
            trainer.step(x.shape[0])
            metric.update([y], [out])
        val_metric = gluon.metric.Accuracy()
        for x, y in val_data:
            val_metric.update([y.as_in_context(ctx)], [net(x.as_in_context(ctx))])
        acc = val_metric.get()[1]
        print('epoch %d: train %s=%.4f, validation %s=%.4f' % ((epoch,) + metric.get() + val_metric.get()))
    return acc


if __name__ == '__main__':
    main()

#!/usr/bin/env python
"""Data-parallel training with one process per GPU (the flow of example/distributed_training/cifar10_dist.py in MXNet):
every worker reads its own shard of the data set, gradients are summed through the KVStore.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 example/distributed_training/cifar10_dist.py
    python -m mxnet_b200.parallel.launch -n 2 python example/distributed_training/cifar10_dist.py --cpu

On GPUs `kvstore='device'` makes the Trainer use the fused gradient exchange + optimizer step over NVLink peer memory;
`--cpu` runs the same script over the gloo backend.  CIFAR-10 is replaced by synthetic 32x32 images unless
`--data-dir` holds the binary batches."""
import argparse
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), '..', '..'))
import mxnet_b200 as mx                                    # noqa: E402
from mxnet_b200 import autograd, gluon                     # noqa: E402
from mxnet_b200.gluon import nn                            # noqa: E402


class SplitSampler(gluon.data.sampler.Sampler):
    """Every worker iterates over its own contiguous part of the data set, in a fresh random order per epoch."""

    def __init__(self, length, num_parts=1, part_index=0, seed=0):
        self.part_len = length // num_parts
        self.start = self.part_len * part_index
        self.rng = np.random.RandomState(seed + part_index)

    def __iter__(self):
        order = self.start + self.rng.permutation(self.part_len)
        return iter(order.tolist())

    def __len__(self):
        return self.part_len


def small_resnet(classes):
    net = nn.HybridSequential()
    net.add(nn.Conv2D(32, 3, padding=1), nn.BatchNorm(), nn.Activation('relu'),
            nn.Conv2D(64, 3, strides=2, padding=1), nn.BatchNorm(), nn.Activation('relu'),
            nn.Conv2D(128, 3, strides=2, padding=1), nn.BatchNorm(), nn.Activation('relu'),
            nn.GlobalAvgPool2D(), nn.Flatten(), nn.Dense(classes))
    return net


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--epochs', type=int, default=1)
    ap.add_argument('--batch-size', type=int, default=32, help='per worker')
    ap.add_argument('--lr', type=float, default=0.05)
    ap.add_argument('--samples', type=int, default=1024)
    ap.add_argument('--cpu', action='store_true')
    ap.add_argument('--data-dir', default=None)
    args = ap.parse_args(argv)
    store = mx.kv.create('dist_sync' if args.cpu else 'device')
    rank, world = store.rank, store.num_workers
    ctx = mx.cpu() if args.cpu else mx.gpu(int(os.environ.get('LOCAL_RANK', 0)))
    if args.data_dir:
        ds = gluon.data.vision.CIFAR10(args.data_dir, train=True).transform(
            lambda d, l: (d.astype('float32').transpose((2, 0, 1)) / 255, np.float32(l)))
    else:
        rng = np.random.RandomState(0)                     # the same synthetic set on every worker; each reads its shard
        y = rng.randint(0, 10, args.samples)
        x = rng.rand(args.samples, 3, 32, 32).astype('float32') * 0.1
        x[np.arange(args.samples), y % 3, y, :] += 1.0      # a bright row tells the class
        ds = gluon.data.ArrayDataset(x, y.astype('float32'))
    loader = gluon.data.DataLoader(ds, args.batch_size, sampler=SplitSampler(len(ds), world, rank), last_batch='discard')
    net = small_resnet(10)
    net.initialize(mx.init.Xavier(), ctx=ctx)
    net.hybridize()
    trainer = gluon.Trainer(net.collect_params(), 'sgd', {'learning_rate': args.lr, 'momentum': 0.9}, kvstore=store)
    loss_fn = gluon.loss.SoftmaxCrossEntropyLoss()
    acc = 0.0
    for epoch in range(args.epochs):
        metric = gluon.metric.Accuracy()
        for x, y in loader:
            x, y = x.as_in_context(ctx), y.as_in_context(ctx)
            with autograd.record():
                out = net(x)
                loss = loss_fn(out, y)
            loss.backward()
            trainer.step(args.batch_size * world)           # gradients are summed over the workers
            metric.update([y], [out])
        acc = metric.get()[1]
        print('worker %d/%d epoch %d: training accuracy %.3f' % (rank, world, epoch, acc), flush=True)
    return acc


if __name__ == '__main__':
    main()

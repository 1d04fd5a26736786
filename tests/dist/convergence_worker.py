"""Worker of the multi-GPU convergence check: launched once per GPU by ``torch.distributed.run``.

A small residual convolutional network (NHWC, BatchNorm, fp16 AMP with dynamic loss scaling, hybridized so that the step
runs from CUDA graphs, multi-precision SGD with warm-up through the fused peer-memory step) is trained on a FIXED
synthetic data set whose labels are a function of the images, each rank on its own slice of every batch.  Rank 0 reports
the loss at the start and at the end, the training accuracy at the end, and whether all ranks hold identical weights: the
loss must fall at every world size, which a wrong gradient scale, a missed shard or a stale weight copy would prevent."""
import json
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import mxnet_b200 as mx                                   # noqa: E402
from mxnet_b200 import amp, autograd, gluon, nd           # noqa: E402
from mxnet_b200.gluon import nn                           # noqa: E402
from mxnet_b200.parallel import dist                      # noqa: E402

CLASSES, PER_RANK, SIDE = 8, 16, 16


class Block(gluon.HybridBlock):
    def __init__(self, channels):
        super().__init__()
        self.c1 = nn.Conv2D(channels, 3, padding=1, use_bias=False, layout='NHWC', in_channels=channels)
        self.b1 = nn.BatchNorm(axis=3, in_channels=channels)
        self.c2 = nn.Conv2D(channels, 3, padding=1, use_bias=False, layout='NHWC', in_channels=channels)
        self.b2 = nn.BatchNorm(axis=3, in_channels=channels)

    def forward(self, x):
        y = nd.relu(self.b1(self.c1(x)))
        y = self.b2(self.c2(y))
        return nd.relu(y + x)


def build(ctx):
    mx.random.seed(11)
    np.random.seed(11)
    net = nn.HybridSequential()
    net.add(nn.Conv2D(32, 3, padding=1, use_bias=False, layout='NHWC', in_channels=8), nn.BatchNorm(axis=3, in_channels=32),
            nn.Activation('relu'), Block(32), nn.MaxPool2D(2, 2, layout='NHWC'), Block(32),
            nn.GlobalAvgPool2D(layout='NHWC'), nn.Flatten(), nn.Dense(CLASSES, in_units=32))
    net.initialize(mx.init.Xavier(), ctx=ctx)
    return net


def dataset(world):
    """Fixed images; the label is the arg-max over class templates of the image's correlation with the template."""
    rng = np.random.RandomState(5)
    n = PER_RANK * world * 4                                  # four batches, revisited every epoch
    templates = rng.randn(CLASSES, SIDE, SIDE, 8).astype('float32')
    labels = rng.randint(0, CLASSES, n)
    images = 0.7 * templates[labels] + rng.randn(n, SIDE, SIDE, 8).astype('float32')
    return images, labels


def main():
    dist.ensure_initialized('nccl')
    rank, world = dist.rank(), dist.world_size()
    torch.cuda.set_device(dist.local_rank())
    ctx = mx.gpu(dist.local_rank())
    amp.init(target_dtype='float16')
    net = build(ctx)
    net.hybridize(static_alloc=True, static_shape=True)
    steps = 60
    sched = mx.lr_scheduler.CosineScheduler(steps, base_lr=0.2, final_lr=0.02, warmup_steps=5, warmup_begin_lr=0.02)
    trainer = gluon.Trainer(net.collect_params(), 'sgd', {'learning_rate': 0.2, 'momentum': 0.9, 'wd': 1e-4,
                                                           'multi_precision': True, 'lr_scheduler': sched}, kvstore='device')
    amp.init_trainer(trainer)
    loss_fn = gluon.loss.SoftmaxCrossEntropyLoss()
    images, labels = dataset(world)
    batch = PER_RANK * world
    nbatch = images.shape[0] // batch
    losses = []
    for step in range(steps):
        lo = (step % nbatch) * batch + rank * PER_RANK
        x = nd.array(images[lo:lo + PER_RANK], ctx=ctx, dtype='float16')
        y = nd.array(labels[lo:lo + PER_RANK], ctx=ctx)
        with autograd.record():
            loss = loss_fn(net(x), y)
            with amp.scale_loss(loss, trainer) as scaled:
                autograd.backward(scaled)
        trainer.step(batch)
        mean = float(loss.mean().asnumpy())
        total = dist.all_reduce_sum(torch.tensor([mean], device=ctx.torch_device))
        losses.append(float(total.item()) / world)
    # training accuracy over the whole data set (every rank scores its slice), inference mode
    correct = 0
    for b in range(nbatch):
        lo = b * batch + rank * PER_RANK
        out = net(nd.array(images[lo:lo + PER_RANK], ctx=ctx, dtype='float16'))
        correct += int((out.asnumpy().argmax(1) == labels[lo:lo + PER_RANK]).sum())
    tot = dist.all_reduce_sum(torch.tensor([float(correct)], device=ctx.torch_device))
    # trained parameters only: the moving statistics of BatchNorm follow each rank's own slice of the data
    flat = torch.cat([p.data(ctx)._data.float().reshape(-1) for p in net.collect_params().values() if p.grad_req != 'null'])
    checksum = torch.stack([flat.sum(), flat.abs().sum()])
    sums = dist.all_gather_tensor(checksum)
    identical = all(bool(torch.equal(s, sums[0])) for s in sums)
    if rank == 0:
        print('REPORT ' + json.dumps({'world': world, 'first': float(np.mean(losses[:3])), 'last': float(np.mean(losses[-3:])),
                                      'accuracy': float(tot.item()) / images.shape[0], 'ranks_identical': identical,
                                      'fused': trainer._fused is not None, 'finite': bool(np.isfinite(losses).all())}),
              flush=True)
    dist.barrier()
    dist.destroy()


if __name__ == '__main__':
    main()

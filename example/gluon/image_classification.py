#!/usr/bin/env python
"""Image classification with the model zoo (the flow of example/gluon/image_classification.py in MXNet): any
`gluon.model_zoo.vision` network, SGD with momentum, optional AMP (fp16 with dynamic loss scaling), CUDA-graph
hybridisation on a GPU.

    python example/gluon/image_classification.py --model resnet18_v1 --batch-size 32 --iters 20 [--gpu] [--amp]

Data is synthetic (random images, random labels) at `--image-size`; plug a `gluon.data.DataLoader` over an
`ImageRecordDataset` into `batches()` for real data."""
import argparse
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), '..', '..'))
import mxnet_b200 as mx                                    # noqa: E402
from mxnet_b200 import amp, autograd, gluon                # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='resnet18_v1')
    ap.add_argument('--classes', type=int, default=10)
    ap.add_argument('--batch-size', type=int, default=32)
    ap.add_argument('--image-size', type=int, default=64)
    ap.add_argument('--iters', type=int, default=20)
    ap.add_argument('--lr', type=float, default=0.05)
    ap.add_argument('--gpu', action='store_true')
    ap.add_argument('--amp', action='store_true')
    args = ap.parse_args(argv)
    ctx = mx.gpu(0) if args.gpu else mx.cpu()
    if args.amp:
        amp.init()
    net = gluon.model_zoo.vision.get_model(args.model, classes=args.classes)
    net.initialize(mx.init.Xavier(), ctx=ctx)
    net.hybridize(static_alloc=args.gpu, static_shape=args.gpu)
    trainer = gluon.Trainer(net.collect_params(), 'sgd', {'learning_rate': args.lr, 'momentum': 0.9, 'wd': 1e-4})
    if args.amp:
        amp.init_trainer(trainer)
    loss_fn = gluon.loss.SoftmaxCrossEntropyLoss()
    rng = np.random.RandomState(0)

    def batches():
        for _ in range(args.iters):
            yield (mx.nd.array(rng.rand(args.batch_size, 3, args.image_size, args.image_size), ctx=ctx, dtype='float32'),
                   mx.nd.array(rng.randint(0, args.classes, args.batch_size), ctx=ctx, dtype='float32'))
    tic, seen, last = time.time(), 0, None
    for x, y in batches():
        with autograd.record():
            loss = loss_fn(net(x), y)
            if args.amp:
                with amp.scale_loss(loss, trainer) as scaled:
                    autograd.backward(scaled)
        if not args.amp:
            loss.backward()
        trainer.step(args.batch_size)
        seen += args.batch_size
        last = float(loss.mean().asscalar())
    print('%s: %d images in %.2f s (%.1f img/s), last loss %.4f' % (args.model, seen, time.time() - tic,
                                                                    seen / (time.time() - tic), last))
    return last


if __name__ == '__main__':
    main()

#!/usr/bin/env python
"""Post-training INT8 quantisation of a model-zoo network (the flow of example/quantization in MXNet): calibrate on a
few batches, convert with `mx.contrib.quantization.quantize_net`, compare the outputs with the fp32 network.

    python example/quantization/quantize_model.py --model resnet18_v1 --calib-mode naive [--gpu]

Calibration data is synthetic; pass a DataLoader over real images for a model that is to be deployed."""
import argparse
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), '..', '..'))
import mxnet_b200 as mx                                    # noqa: E402
from mxnet_b200 import gluon                               # noqa: E402
from mxnet_b200.contrib import quantization                # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='resnet18_v1')
    ap.add_argument('--image-size', type=int, default=64)
    ap.add_argument('--batch-size', type=int, default=4)
    ap.add_argument('--calib-batches', type=int, default=2)
    ap.add_argument('--calib-mode', default='naive', choices=['naive', 'entropy', 'none'])
    ap.add_argument('--gpu', action='store_true')
    args = ap.parse_args(argv)
    ctx = mx.gpu(0) if args.gpu else mx.cpu()
    net = gluon.model_zoo.vision.get_model(args.model, classes=10)
    net.initialize(mx.init.Xavier(), ctx=ctx)
    rng = np.random.RandomState(0)
    shape = (args.batch_size, 3, args.image_size, args.image_size)
    calib = [mx.nd.array(rng.rand(*shape), ctx=ctx, dtype='float32') for _ in range(args.calib_batches)]
    x = mx.nd.array(rng.rand(*shape), ctx=ctx, dtype='float32')
    ref = net(x).asnumpy()
    calib_data = gluon.data.DataLoader(gluon.data.ArrayDataset(np.concatenate([c.asnumpy() for c in calib])), args.batch_size)
    qnet = quantization.quantize_net(net, quantized_dtype='int8', calib_mode=args.calib_mode, calib_data=calib_data,
                                     num_calib_batches=args.calib_batches, device=ctx)
    out = qnet(x).asnumpy()
    err = float(np.abs(out - ref).max() / (np.abs(ref).max() + 1e-12))
    agree = float((out.argmax(1) == ref.argmax(1)).mean())
    print('%s int8 (%s calibration): max error relative to the largest logit %.4f, top-1 agreement with fp32 %.2f'
          % (args.model, args.calib_mode, err, agree))
    return err


if __name__ == '__main__':
    main()

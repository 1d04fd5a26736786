"""Inference latency of model-zoo networks as written (NCHW), with and without layout management.

    python -m benchmark.model_zoo_inference [--models resnet50_v1,mobilenet_v2_1_0] [--batches 1,8,64] [--no-library]

Forward pass in predict mode on synthetic data, hybridized with static allocation (CUDA-graph replay), CUDA events over 30
calls after 6 warm-up calls: fp32 as written, fp32 with layout management, fp16 with layout management.  When torchvision is
importable the same architecture in eager tensor-library code is timed beside them (fp32, and fp16 in channels-last memory
format).  Prints one JSON line per network and batch size.
"""
import argparse
import json
import warnings

import numpy as np
import torch

PAIRS = {'resnet18_v1': 'resnet18', 'resnet50_v1': 'resnet50', 'vgg16': 'vgg16', 'mobilenet_v2_1_0': 'mobilenet_v2',
         'densenet121': 'densenet121', 'squeezenet1_1': 'squeezenet1_1', 'alexnet': 'alexnet'}


def _time(fn, warmup=6, reps=30):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return round(a.elapsed_time(b) / reps, 3)


def ours(name, dtype, optimize_layout, batch):
    import mxnet_b200 as mx
    from mxnet_b200.gluon.model_zoo import vision
    from mxnet_b200.symbol import layout
    ctx = mx.gpu(0)
    layout.set_optimize_layout(optimize_layout)
    try:
        net = getattr(vision, name)(classes=1000)
        net.initialize(mx.init.Xavier(), ctx=ctx)
        if dtype != 'float32':
            net.cast(dtype)
        net.hybridize(static_alloc=True, static_shape=True)
        x = mx.nd.array(np.random.uniform(-1, 1, (batch, 3, 224, 224)).astype(dtype), ctx=ctx, dtype=dtype)
        return _time(lambda: net(x))
    finally:
        layout.set_optimize_layout(False)


def library(name, dtype, batch, channels_last):
    import torchvision
    m = getattr(torchvision.models, name)(weights=None).cuda().eval()
    x = torch.randn(batch, 3, 224, 224, device='cuda')
    if dtype == 'float16':
        m, x = m.half(), x.half()
    if channels_last:
        m, x = m.to(memory_format=torch.channels_last), x.to(memory_format=torch.channels_last)
    with torch.no_grad():
        return _time(lambda: m(x))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--models', default='resnet50_v1,mobilenet_v2_1_0')
    ap.add_argument('--batches', default='1,8,64')
    ap.add_argument('--no-library', action='store_true')
    args = ap.parse_args()
    warnings.filterwarnings('ignore')
    try:
        import torchvision  # noqa: F401
        have_tv = not args.no_library
    except ImportError:
        have_tv = False
    for name in args.models.split(','):
        for batch in (int(b) for b in args.batches.split(',')):
            rec = {'model': name, 'batch': batch, 'unit': 'ms per forward pass',
                   'fp32_as_written': ours(name, 'float32', False, batch),
                   'fp32_layout_managed': ours(name, 'float32', True, batch),
                   'fp16_layout_managed': ours(name, 'float16', True, batch)}
            if have_tv and name in PAIRS:
                rec['tensor_library_eager_fp32'] = library(PAIRS[name], 'float32', batch, False)
                rec['tensor_library_eager_fp16_channels_last'] = library(PAIRS[name], 'float16', batch, True)
            print(json.dumps(rec), flush=True)


if __name__ == '__main__':
    main()

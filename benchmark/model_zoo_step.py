"""Training step of the model-zoo networks as a reference user writes them (NCHW), with and without layout management.

    python -m benchmark.model_zoo_step [--batch 32] [--models resnet18_v1,vgg16,...] [--no-library]

For every network: one SGD-momentum training step (forward, softmax cross-entropy, backward, update) on synthetic data,
hybridized with static allocation (CUDA-graph replay), timed with CUDA events over 8 steps after 4 warm-up steps:
fp32 as written; fp32 with layout management (``mx.symbol.layout.set_optimize_layout``); fp16 (multi-precision SGD) with layout
management.  When torchvision is importable the same architecture in plain eager tensor-library code (fp32, its defaults) is
timed beside them as a point of comparison.  Prints one JSON line per network.
"""
import argparse
import json
import warnings

import numpy as np
import torch

PAIRS = [('resnet18_v1', 'resnet18', 224), ('resnet50_v1', 'resnet50', 224), ('vgg16', 'vgg16', 224),
         ('mobilenet_v2_1_0', 'mobilenet_v2', 224), ('densenet121', 'densenet121', 224), ('squeezenet1_1', 'squeezenet1_1', 224),
         ('alexnet', 'alexnet', 224), ('inception_v3', 'inception_v3', 299)]


def _time(step, warmup=4, reps=8):
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        step()
    b.record()
    torch.cuda.synchronize()
    return round(a.elapsed_time(b) / reps, 2)


def ours(name, dtype, optimize_layout, batch, size):
    import mxnet_b200 as mx
    from mxnet_b200 import gluon
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
        trainer = gluon.Trainer(net.collect_params(), 'sgd', {'learning_rate': 0.001, 'momentum': 0.9,
                                                              'multi_precision': dtype != 'float32'})
        x = mx.nd.array(np.random.uniform(-1, 1, (batch, 3, size, size)).astype(dtype), ctx=ctx, dtype=dtype)
        y = mx.nd.array(np.random.randint(0, 1000, (batch,)), ctx=ctx)
        loss_fn = gluon.loss.SoftmaxCrossEntropyLoss()

        def step():
            with mx.autograd.record():
                loss = loss_fn(net(x).astype('float32'), y).mean()
            loss.backward()
            trainer.step(1)
        return _time(step)
    finally:
        layout.set_optimize_layout(False)


def library(name, batch, size):
    import torchvision
    m = getattr(torchvision.models, name)(weights=None).cuda()
    opt = torch.optim.SGD(m.parameters(), lr=0.001, momentum=0.9)
    x = torch.randn(batch, 3, size, size, device='cuda')
    y = torch.randint(0, 1000, (batch,), device='cuda')

    def step():
        opt.zero_grad(set_to_none=True)
        out = m(x)
        if not isinstance(out, torch.Tensor):
            out = out[0]
        torch.nn.functional.cross_entropy(out, y).backward()
        opt.step()
    return _time(step)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--batch', type=int, default=32)
    ap.add_argument('--models', default=','.join(p[0] for p in PAIRS))
    ap.add_argument('--no-library', action='store_true')
    args = ap.parse_args()
    warnings.filterwarnings('ignore')
    wanted = set(args.models.split(','))
    try:
        import torchvision  # noqa: F401
        have_tv = not args.no_library
    except ImportError:
        have_tv = False
    for name, tv_name, size in PAIRS:
        if name not in wanted:
            continue
        rec = {'model': name, 'batch': args.batch, 'image': size, 'unit': 'ms per training step',
               'fp32_as_written': ours(name, 'float32', False, args.batch, size),
               'fp32_layout_managed': ours(name, 'float32', True, args.batch, size),
               'fp16_layout_managed': ours(name, 'float16', True, args.batch, size)}
        if have_tv:
            rec['tensor_library_eager_fp32'] = library(tv_name, args.batch, size)
        print(json.dumps(rec), flush=True)


if __name__ == '__main__':
    main()

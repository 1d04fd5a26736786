#!/usr/bin/env python
"""Headline benchmark: ResNet-50 v1b training throughput (img/s), AMP fp16, NHWC, batch 256 per GPU,
multi-precision SGD momentum 0.9 / wd 1e-4, data parallel over N GPUs of one node.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Prints ONE JSON line (rank 0).  ``value`` is the whole-job img/s with inputs already on the device, timed
with CUDA events (max over ranks).  ``e2e`` is the same training step driven through the public Gluon API
including, every step, the host→device copy of that step's uint8 batch from pinned memory and a
device→host read of the loss.  ``--impl reference`` reports why the reference cannot run here.

The same line carries sub-records measured in the same process after the headline: ``library_path`` (the same training
steps with the in-tree kernels and the fused optimizer step switched off, i.e. library convolutions / GEMMs and one NCCL
all-reduce per parameter), ``bert`` and ``lstm_lm`` (the other two configured models through the shared harness, the
language model in fp32 as configured) and, on two or more GPUs, ``kvstore_pushpull`` (bus bandwidth of the gradient
exchange, fused peer-memory kernels against one NCCL all-reduce per key, at 1 MiB and 64 MiB keys).
"""
import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

BASELINE_IMG_S_1GPU = 363.69      # ResNet-50 training, V100 fp32 batch 128, docs/static_site/.../perf.md:242-253


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--batch', type=int, default=256, help='images per GPU')
    ap.add_argument('--image', type=int, default=224)
    ap.add_argument('--classes', type=int, default=1000)
    ap.add_argument('--graphs', type=int, default=int(os.environ.get('MXB_BENCH_GRAPHS', '1')),
                    help='hybridize(static_alloc, static_shape): CUDA-graph replay of forward/backward')
    ap.add_argument('--no-e2e', action='store_true')
    ap.add_argument('--no-extras', action='store_true',
                    help='skip the sub-records (library path, BERT, LSTM-LM, gradient-exchange bandwidth)')
    return ap.parse_args()


def reference_arm(args):
    print(json.dumps({'impl': 'reference', 'unavailable':
                      'reference is not installable offline: the reference tree has no setup.py/pyproject.toml at its root, '
                      'python/setup.py needs a compiled libmxnet.so and the dmlc-core/tvm(nnvm)/ps-lite/cub submodules '
                      'are empty, so it cannot be built (pip: "Neither setup.py nor pyproject.toml found")'}))
    return 0


def measure_extras(args, ctx, rank, world, measure_resnet, barrier):
    """The sub-records of the JSON line (see the module docstring).  Every rank runs them (they train data-parallel like
    the headline); a sub-record that fails is reported as ``{'error': ...}`` instead of taking the headline down."""
    import types
    import torch
    from mxnet_b200 import amp, env
    bench_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'benchmark')
    if bench_dir not in sys.path:
        sys.path.insert(0, bench_dir)
    out = {}
    steps, warmup = max(5, min(args.steps, 10)), 3

    def guarded(name, fn):
        try:
            out[name] = fn()
        except Exception as e:  # pylint: disable=broad-except
            out[name] = {'error': '%s: %s' % (type(e).__name__, str(e)[:300])}
        barrier()
        torch.cuda.empty_cache()

    # ---- the same ResNet-50 steps on the library path: no in-tree kernels, one NCCL all-reduce per parameter ----------
    def library_path():
        with env.scope('MXNET_B200_KERNELS', '0'), env.scope('MXNET_KVSTORE_FUSED', '0'):
            r = measure_resnet(steps, warmup, False)
        return {'value': r['value'], 'unit': 'img/s', 'ms_per_step': r['ms_per_step'], 'steps': steps,
                'switches': 'MXNET_B200_KERNELS=0 MXNET_KVSTORE_FUSED=0', 'fused_step': r['fused']}
    guarded('library_path', library_path)

    # ---- the other two configured models, through the shared harness ---------------------------------------------------
    def sub_model(module_name, argv, reset_amp):
        import importlib
        import _harness
        mod = importlib.import_module(module_name)
        a = mod.parser().parse_args(argv)
        if reset_amp:
            amp._reset()           # the language model is configured in fp32: no cast policy
        name, unit, items, make_step, cfg = mod.spec(a)
        rec = _harness.measure(name, unit, items, make_step, a, cfg)
        return {k: rec[k] for k in ('metric', 'value', 'unit', 'ms_per_step', 'steps', 'config', 'gpu_launches', 'final_loss')}
    guarded('bert', lambda: sub_model('bert_pretrain', ['--steps', str(steps), '--warmup', str(warmup)], False))
    guarded('lstm_lm', lambda: sub_model('lstm_lm', ['--steps', str(steps), '--warmup', str(warmup), '--dtype', 'float32'], True))

    # the same model with the fp32 GEMMs in the reference's math mode (tf32 operands: src/operator/linalg_impl.h:298 sets
    # CUBLAS_TF32_TENSOR_OP_MATH for fp32 products); reported beside the exact-fp32 record, not instead of it
    def lstm_tf32():
        try:
            return sub_model('lstm_lm', ['--steps', str(steps), '--warmup', str(warmup), '--dtype', 'float32', '--tf32'], True)
        finally:
            env.set('MXNET_CUDA_ALLOW_TF32', False)
    guarded('lstm_lm_tf32', lstm_tf32)

    # ---- gradient-exchange bandwidth (needs peers) -----------------------------------------------------------------------
    if world > 1:
        def pushpull():
            from mxnet_b200.kvstore import bandwidth
            rows = []
            for key_bytes, keys in ((1 << 20, 32), (64 << 20, 8)):
                for path in ('fused', 'nccl'):
                    r = bandwidth.measure(path, keys, key_bytes, 'float16', 10, 3, ctx, rank, world)
                    rows.append({k: r[k] for k in ('path', 'key_bytes', 'num_keys', 'ms', 'busbw_GBps')})
            return {'unit': 'GB/s bus bandwidth = bytes * 2 * (n - 1) / n / t, max time over ranks', 'rows': rows}
        guarded('kvstore_pushpull', pushpull)
    return out


def main():
    args = parse()
    if args.impl == 'reference':
        return reference_arm(args)
    import numpy as np
    import torch
    import mxnet_b200 as mx
    from mxnet_b200 import amp, autograd, gluon
    from mxnet_b200.models import resnet50_v1b
    from mxnet_b200.ops import cuda as kernels
    from mxnet_b200.parallel import dist
    from mxnet_b200.utils import ClockSampler

    world = int(os.environ.get('WORLD_SIZE', '1'))
    if world > 1:
        dist.ensure_initialized('nccl')
    rank, local = dist.rank(), dist.local_rank()
    torch.cuda.set_device(local)
    ctx = mx.gpu(local)
    torch.backends.cudnn.benchmark = True
    mx.random.seed(1234 + rank)
    np.random.seed(1234 + rank)

    amp.init('float16')

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=ctx.torch_device, dtype=torch.float64)
        import torch.distributed as tdist
        tdist.all_reduce(t, op=tdist.ReduceOp.MAX)
        return float(t.item())

    def measure_resnet(steps, warmup, with_e2e):
        """Build the model and its trainer under the current switches, run the device-timed steps and (optionally) the
        end-to-end steps; returns the figures of one arm."""
        B, S, NC = args.batch, args.image, args.classes
        global_batch = B * world
        net = resnet50_v1b(classes=NC, layout='NHWC', fused=True)
        net.initialize(mx.init.Xavier(rnd_type='gaussian', factor_type='out', magnitude=2), ctx=ctx)
        # fp16 weights everywhere (fp32 master copies live in the optimizer); BatchNorm statistics stay fp32
        for p in net.collect_params().values():
            if p.grad_req != 'null':
                p.cast('float16')
        loss_fn = gluon.loss.SoftmaxCrossEntropyLoss()
        # linear-scaling rule with the usual gradual warm-up (5 epochs of ImageNet at this batch size): the first steps of
        # a run from random weights do not diverge at the large-batch learning rate
        base_lr = 0.1 * global_batch / 256.0
        schedule = mx.lr_scheduler.CosineScheduler(max_update=450000, base_lr=base_lr, final_lr=0.0,
                                                   warmup_steps=max(1, 5 * 1281167 // global_batch), warmup_begin_lr=0.0)
        trainer = gluon.Trainer(net.collect_params(), 'sgd',
                                {'learning_rate': base_lr, 'momentum': 0.9, 'wd': 1e-4, 'multi_precision': True,
                                 'lr_scheduler': schedule}, kvstore='device')
        amp.init_trainer(trainer)
        if args.graphs:
            net.hybridize(static_alloc=True, static_shape=True)

        mean = torch.tensor([123.68, 116.28, 103.53], device=ctx.torch_device, dtype=torch.float16)
        inv_std = torch.tensor([1 / 58.4, 1 / 57.12, 1 / 57.38], device=ctx.torch_device, dtype=torch.float16)

        def preprocess(u8):
            """uint8 NHWC batch on the device -> normalised fp16 NHWC."""
            return mx.nd.NDArray._from_tensor((u8.to(torch.float16) - mean) * inv_std, ctx)

        def train_step(x, y):
            with autograd.record():
                out = net(x)
                loss = loss_fn(out, y)
                with amp.scale_loss(loss, trainer) as scaled:
                    autograd.backward(scaled)
            trainer.step(global_batch)
            return loss

        # synthetic data: pixel values from N(0,1) after normalisation, labels uniform in [0, classes)
        n_host = 4
        host_x = [torch.randint(0, 256, (B, S, S, 3), dtype=torch.uint8).pin_memory() for _ in range(n_host)]
        host_y = [torch.randint(0, NC, (B,), dtype=torch.int64).pin_memory() for _ in range(n_host)]
        dev_x = [preprocess(h.to(ctx.torch_device)) for h in host_x[:2]]
        dev_y = [mx.nd.NDArray._from_tensor(h.to(ctx.torch_device), ctx) for h in host_y[:2]]

        def barrier():
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
                torch.cuda.synchronize()

        def max_over_ranks(ms):
            if world == 1:
                return ms
            t = torch.tensor([ms], device=ctx.torch_device, dtype=torch.float64)
            import torch.distributed as tdist
            tdist.all_reduce(t, op=tdist.ReduceOp.MAX)
            return float(t.item())

        # ---------------------------------------------------------------- device-timed steps (inputs resident)
        for i in range(max(warmup, 3)):
            train_step(dev_x[i % 2], dev_y[i % 2])
        barrier()
        sampler = ClockSampler(local).start()
        l0 = kernels.launches()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            loss = train_step(dev_x[i % 2], dev_y[i % 2])
        e1.record()
        barrier()
        launches = kernels.launches() - l0
        clocks = sampler.stop()
        ms = max_over_ranks(e0.elapsed_time(e1))
        value = global_batch * steps / (ms / 1000.0)
        final_loss = float(loss.mean().asscalar())

        # ---------------------------------------------------------------- end to end through the public API
        e2e = None
        if with_e2e:
            copy_stream = torch.cuda.Stream(device=ctx.torch_device)
            loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()
            h2d_bytes = host_x[0].numel() * host_x[0].element_size() + host_y[0].numel() * host_y[0].element_size()
            d2h_bytes = loss_host.numel() * loss_host.element_size()
            staged = [None, None]

            def stage(i):
                """Copy batch i to the device on the copy stream (overlaps the previous step's compute)."""
                with torch.cuda.stream(copy_stream):
                    xb = host_x[i % n_host].to(ctx.torch_device, non_blocking=True)
                    yb = host_y[i % n_host].to(ctx.torch_device, non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(copy_stream)
                staged[i % 2] = (xb, yb, ev)

            def run(n, timed):
                losses = []
                stage(0)
                for i in range(n):
                    xb, yb, ev = staged[i % 2]
                    torch.cuda.current_stream().wait_event(ev)
                    if i + 1 < n:
                        stage(i + 1)
                    x = preprocess(xb)
                    y = mx.nd.NDArray._from_tensor(yb, ctx)
                    loss = train_step(x, y)
                    xb.record_stream(torch.cuda.current_stream())
                    yb.record_stream(torch.cuda.current_stream())
                    loss_host.copy_(loss.mean()._data.float().reshape(1), non_blocking=True)   # device -> host read of the result
                    torch.cuda.current_stream().synchronize() if not timed else None
                    losses.append(loss_host)
                return losses
            run(max(warmup, 3), False)
            barrier()
            t0 = torch.cuda.Event(enable_timing=True)
            t1 = torch.cuda.Event(enable_timing=True)
            t0.record()
            run(steps, True)
            t1.record()
            barrier()
            ms_e2e = max_over_ranks(t0.elapsed_time(t1))
            e2e = {'value': global_batch * steps / (ms_e2e / 1000.0), 'unit': 'img/s', 'ms_per_step': ms_e2e / steps,
                   'h2d_bytes_per_step': int(h2d_bytes), 'd2h_bytes_per_step': int(d2h_bytes),
                   'last_loss': float(loss_host.item())}


        from mxnet_b200.ops.cuda import conv_ops
        tuned = conv_ops.tuned_choices()
        conv_sel = {d: '%d of %d' % (sum(1 for k, v in tuned.items() if k[0] == d and v), sum(1 for k in tuned if k[0] == d))
                    for d in ('fwd', 'dgrad', 'dgrad+skip', 'wgrad')}
        # what the autotuner measured (microseconds with a cold L2: in-tree kernel, library), per direction and layer geometry
        conv_us = {}
        for k, (t_own, t_lib) in sorted(conv_ops.tuned_times().items(), key=lambda kv: (kv[0][0],) + tuple(kv[0][2:])):
            conv_us.setdefault(k[0], {})['%dx%d %d>%d k%d s%d' % (k[3], k[4], k[5], k[6], k[7], k[-1])] = [t_own, t_lib]
        conv_sel['autotune_us'] = conv_us
        res = {'value': value, 'ms_per_step': ms / steps, 'launches': int(launches), 'clocks': clocks, 'final_loss': final_loss,
               'e2e': e2e, 'fused': trainer._fused is not None, 'conv_sel': conv_sel, 'global_batch': global_batch}
        del net, trainer
        torch.cuda.empty_cache()
        return res

    main_arm = measure_resnet(args.steps, args.warmup, not args.no_e2e)
    extras = {} if args.no_extras else measure_extras(args, ctx, rank, world, measure_resnet, barrier)
    B, S = args.batch, args.image
    global_batch = main_arm['global_batch']
    value, ms, launches, clocks = main_arm['value'], main_arm['ms_per_step'] * args.steps, main_arm['launches'], main_arm['clocks']
    final_loss, e2e, conv_sel = main_arm['final_loss'], main_arm['e2e'], main_arm['conv_sel']

    if rank == 0:
        fused = main_arm['fused']
        out = {
            'metric': 'resnet50_train_img_per_s', 'value': value, 'unit': 'img/s', 'n_gpus': world, 'steps': args.steps,
            'warmup': max(args.warmup, 3), 'ms_per_step': ms / args.steps, 'higher_is_better': True, 'scaling': 'weak',
            'vs_baseline': value / (BASELINE_IMG_S_1GPU * world), 'dtype': 'fp16', 'data': 'synthetic',
            'config': {'model': 'resnet50_v1b', 'global_batch': global_batch, 'batch_per_gpu': B, 'image': S, 'layout': 'NHWC',
                       'parallelism': 'dp%d' % world, 'optimizer': 'sgd momentum 0.9 wd 1e-4 multi-precision',
                       'amp': 'fp16 dynamic loss scale (device resident)', 'fused_step': fused, 'cuda_graphs': bool(args.graphs),
                       'conv_in_tree_kernel_chosen': conv_sel,
                       'l2': 'inputs larger than L2 (activations per step >> 126 MB); no explicit flush',
                       'baseline_ref': 'V100 fp32 bs128 363.69 img/s per GPU (perf.md) x n_gpus'},
            'clocks': {k: clocks[k] for k in ('sm_mhz', 'sm_max_mhz', 'reasons')},
            'gpu_launches': int(launches), 'final_loss': final_loss, 'impl': 'ours',
        }
        if e2e is not None:
            out['e2e'] = e2e
        out.update(extras)
        print(json.dumps(out))
    if world > 1:
        barrier()
        dist.destroy()
    return 0


if __name__ == '__main__':
    sys.exit(main())

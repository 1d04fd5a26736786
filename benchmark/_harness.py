"""Shared timing harness of the model benchmarks: warm-up, CUDA-event timing with a barrier and a device
synchronisation on both sides, maximum over ranks, clock sampling during the timed region, one JSON line."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def run(name, unit, items_per_step_per_gpu, make_step, args, config, baseline=None):
    """Measure, print the JSON line on rank 0 and shut the process group down (the stand-alone benchmark scripts)."""
    from mxnet_b200.parallel import dist
    world = int(os.environ.get('WORLD_SIZE', '1'))
    rec = measure(name, unit, items_per_step_per_gpu, make_step, args, config, baseline)
    if dist.rank() == 0:
        print(json.dumps(rec))
    if world > 1:
        import torch
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy()
    return 0


def measure(name, unit, items_per_step_per_gpu, make_step, args, config, baseline=None):
    """``make_step(ctx, rank, world)`` returns ``step()`` which runs one training iteration and returns
    the loss NDArray.  Returns the result record (the same on every rank up to rank-0-only fields)."""
    import torch
    import mxnet_b200 as mx
    from mxnet_b200.ops import cuda as kernels
    from mxnet_b200.parallel import dist
    from mxnet_b200.utils import ClockSampler
    world = int(os.environ.get('WORLD_SIZE', '1'))
    if world > 1:
        dist.ensure_initialized('nccl')
    rank, local = dist.rank(), dist.local_rank()
    torch.cuda.set_device(local)
    ctx = mx.gpu(local)
    mx.random.seed(4321 + rank)
    from mxnet_b200.ops.cuda import gemm_ops
    gemm_seen = set(gemm_ops.tuned_choices())        # products an earlier model of this process already settled
    step = make_step(ctx, rank, world)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
    for _ in range(max(args.warmup, 3)):
        loss = step()
    barrier()
    sampler = ClockSampler(local).start()
    l0 = kernels.launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = step()
    e1.record()
    barrier()
    launches = kernels.launches() - l0
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=ctx.torch_device, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t.item())
    value = items_per_step_per_gpu * world * args.steps / (ms / 1e3)
    cfg = dict(config)
    cfg['parallelism'] = 'dp%d' % world
    tuned = {k: v for k, v in gemm_ops.tuned_choices().items() if k not in gemm_seen}
    if tuned:
        cfg['gemm_in_tree_kernel_chosen'] = {p: '%d of %d' % (sum(1 for k, v in tuned.items() if k[0] == p and v),
                                                              sum(1 for k in tuned if k[0] == p))
                                             for p in ('fwd', 'dgrad', 'wgrad')}
        cfg['gemm_autotune_us'] = {'%s %dx%dx%d' % (k[0], k[2], k[3], k[4]): [v[0], v[1]]
                                   for k, v in sorted(gemm_ops.tuned_times().items(), key=lambda kv: (kv[0][0],) + tuple(kv[0][2:5]))
                                   if k in tuned}
    from mxnet_b200.ops.cuda import rnn_ops
    if rnn_ops.tuned_choices():
        cfg['rnn_in_tree_kernel_chosen'] = {'%s T=%d N=%d I=%d H=%d L=%d %s' % (k[0], k[2], k[3], k[4], k[5], k[6],
                                                                               'train' if k[8] else 'eval'): bool(v)
                                            for k, v in rnn_ops.tuned_choices().items()}
        cfg['rnn_autotune_us'] = {'%s T=%d N=%d H=%d L=%d' % (k[0], k[2], k[3], k[5], k[6]): {'in_tree': v[0], 'library': v[1]}
                                  for k, v in rnn_ops.tuned_times().items()}
    return {'metric': name, 'value': value, 'unit': unit, 'n_gpus': world, 'steps': args.steps,
            'warmup': max(args.warmup, 3), 'ms_per_step': ms / args.steps, 'higher_is_better': True,
            'scaling': 'weak', 'vs_baseline': (value / baseline) if baseline else None, 'data': 'synthetic',
            'config': cfg, 'clocks': {k: clocks[k] for k in ('sm_mhz', 'sm_max_mhz', 'reasons')},
            'gpu_launches': int(launches), 'final_loss': float(loss.mean().asscalar())}

"""All-reduce bandwidth of the gradient exchange (the counterpart of ``tools/bandwidth/measure.py``).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m mxnet_b200.kvstore.bandwidth --num-keys 32 --min-size 4096 --max-size 1073741824 --dtype float16

One process per GPU.  For every key size the tool builds ``--num-keys`` gradients of that size, exchanges
them through ``Trainer.allreduce_grads`` (the public entry point of the data-parallel gradient sum) and
reports, per path:

* ``fused``  : the peer-memory reduce-scatter + all-gather kernels (``ops/cuda/fused_step.cu``);
* ``nccl``   : one ``ncclAllReduce`` per key through the ``nccl`` KVStore (the library baseline).

Bandwidth follows the reference's definition, ``size * 2 * (n - 1) / n / t`` per GPU
(tools/bandwidth/measure.py:138), with ``t`` measured by CUDA events on the launching stream and taken as
the maximum over ranks.  The sum is verified against the expected value on every rank before timing.
"""
import argparse
import json
import os
import sys

import numpy as np
import torch


def measure(path, num_keys, nbytes, dtype, iters, warmup, ctx, rank, world):
    import mxnet_b200 as mx
    from mxnet_b200 import env, gluon, nd
    from mxnet_b200.parallel import dist
    esize = 4 if dtype == 'float32' else 2
    n = max(1, nbytes // esize)
    fused = path in ('fused', 'fused_nvls')
    with env.scope('MXNET_KVSTORE_FUSED', '1' if fused else '0'), env.scope('MXNET_KVSTORE_NVLS', '1' if path == 'fused_nvls' else '0'):
        params = []
        for i in range(num_keys):
            p = gluon.Parameter('key%d' % i, shape=(n,), dtype=dtype)
            p.initialize(mx.init.Zero(), ctx=ctx)
            params.append(p)
        trainer = gluon.Trainer(params, 'sgd', {'learning_rate': 0.0, 'multi_precision': dtype != 'float32'},
                                kvstore='nccl' if path == 'nccl' else 'device', update_on_kvstore=False)
        trainer._init_kvstore()
        if (trainer._fused is not None) != fused:
            raise RuntimeError('path %s was not selected' % path)

        def fill():
            for i, p in enumerate(params):
                p.grad(ctx)._data.fill_(float(rank + 1) * (1 + i % 3))
        # correctness first
        fill()
        trainer.allreduce_grads()
        torch.cuda.synchronize()
        expect = world * (world + 1) / 2
        for i, p in enumerate(params):
            g = p.grad(ctx)._data
            if not bool((g.float() == expect * (1 + i % 3)).all()):
                raise RuntimeError('all-reduce result is wrong on rank %d key %d' % (rank, i))
        # timed exchanges run on zeros: repeated in-place sums of non-zero values would overflow fp16 after a
        # few rounds, and the time does not depend on the values
        for p in params:
            p.grad(ctx)._data.zero_()
        for _ in range(warmup):
            trainer.allreduce_grads()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            trainer.allreduce_grads()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / iters], device=ctx.torch_device, dtype=torch.float64)
        if world > 1:
            torch.distributed.all_reduce(ms, op=torch.distributed.ReduceOp.MAX)
        if trainer._fused is not None:
            trainer._fused._check_status()
        t = float(ms.item()) / 1e3
        total = num_keys * n * esize
        multicast = bool(trainer._fused is not None and getattr(trainer._fused, 'mc_base', 0))
        del trainer, params
        torch.cuda.empty_cache()
        return {'path': path, 'multicast': multicast, 'key_bytes': n * esize, 'num_keys': num_keys, 'total_bytes': total, 'ms': t * 1e3,
                'algbw_GBps': total / t / 1e9, 'busbw_GBps': total * 2 * (world - 1) / world / t / 1e9}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--num-keys', type=int, default=32)
    ap.add_argument('--min-size', type=int, default=4096, help='bytes per key')
    ap.add_argument('--max-size', type=int, default=1 << 30, help='bytes per key')
    ap.add_argument('--max-total', type=int, default=8 << 30, help='cap on bytes exchanged per iteration (fewer keys above it)')
    ap.add_argument('--dtype', default='float16', choices=['float16', 'float32', 'bfloat16'])
    ap.add_argument('--paths', default='fused,nccl', help='comma list of fused, fused_nvls (through the NVLink switch), nccl')
    ap.add_argument('--iters', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    args = ap.parse_args()
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    import mxnet_b200 as mx
    from mxnet_b200.parallel import dist
    dist.ensure_initialized('nccl')
    rank, world = dist.rank(), dist.world_size()
    torch.cuda.set_device(dist.local_rank())
    ctx = mx.gpu(dist.local_rank())
    size = args.min_size
    while size <= args.max_size:
        keys = max(1, min(args.num_keys, args.max_total // size))
        for path in args.paths.split(','):
            res = measure(path, keys, size, args.dtype, args.iters, args.warmup, ctx, rank, world)
            res.update({'n_gpus': world, 'dtype': args.dtype})
            if rank == 0:
                print(json.dumps(res), flush=True)
        size *= 4
    dist.barrier()
    dist.destroy()
    return 0


if __name__ == '__main__':
    sys.exit(main())

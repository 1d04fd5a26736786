"""Worker of the multi-GPU fused-step test: launched once per GPU by ``torch.distributed.run``.

Every rank trains the same small network on its own slice of a fixed batch, once with the fused
peer-memory optimizer step and once with the plain NCCL all-reduce + per-parameter update path, and
rank 0 reports whether both runs agree and whether all ranks hold identical weights."""
import json
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import mxnet_b200 as mx                                   # noqa: E402
from mxnet_b200 import autograd, env, gluon, nd           # noqa: E402
from mxnet_b200.gluon import nn                           # noqa: E402
from mxnet_b200.parallel import dist                      # noqa: E402


_MULTICAST = []          # one entry per fused step that ran through an NVLink-switch multicast mapping


def build(ctx, dtype):
    mx.random.seed(7)
    np.random.seed(7)
    net = nn.HybridSequential()
    net.add(nn.Dense(96, activation='relu', in_units=48), nn.Dense(33, activation='relu', in_units=96),
            nn.Dense(10, in_units=33))
    net.initialize(mx.init.Xavier(), ctx=ctx)
    if dtype != 'float32':
        net.cast(dtype)
    return net


def run(fused, dtype, steps, ctx, rank, world, optimizer='sgd'):
    with env.scope('MXNET_KVSTORE_FUSED', '1' if fused else '0'):
        net = build(ctx, dtype)
        opts = {'sgd': {'learning_rate': 0.05, 'momentum': 0.9, 'wd': 1e-3, 'multi_precision': dtype != 'float32'},
                'lamb': {'learning_rate': 0.01, 'wd': 0.01}, 'adam': {'learning_rate': 0.01, 'wd': 0.01}}[optimizer]
        trainer = gluon.Trainer(net.collect_params(), optimizer, opts, kvstore='device')
        loss_fn = gluon.loss.SoftmaxCrossEntropyLoss()
        rng = np.random.RandomState(123)
        per = 8
        for step in range(steps):
            x_all = rng.randn(per * world, 48).astype('float32')
            y_all = rng.randint(0, 10, (per * world,))
            x = nd.array(x_all[rank * per:(rank + 1) * per], ctx=ctx, dtype=dtype)
            y = nd.array(y_all[rank * per:(rank + 1) * per], ctx=ctx)
            with autograd.record():
                loss = loss_fn(net(x), y)
            loss.backward()
            trainer.step(per * world)
        torch.cuda.synchronize()
        assert (trainer._fused is not None) == fused, 'fused path selection'
        if fused and getattr(trainer._fused, 'mc_base', 0):
            _MULTICAST.append(True)
        if fused:
            trainer._fused._check_status()
            if rank == 0 and optimizer == 'adam':
                # a checkpoint written by ONE rank while the others do nothing: the shards of the other ranks are read
                # through peer copies, so no collective is entered (`if rank == 0: trainer.save_states(...)`)
                import pickle, tempfile
                fname = os.path.join(tempfile.mkdtemp(), 'rank0.states')
                trainer.save_states(fname)
                states = pickle.loads(open(fname, 'rb').read())[0]
                numel = sum(int(np.prod(p.shape)) for p in net.collect_params().values())
                mean_numel = sum(int(st[0].size) for st in states.values())
                assert mean_numel == numel, 'rank 0 did not collect every shard of the Adam state'
                assert all(float(abs(st[0].asnumpy()).sum()) > 0 for st in states.values()), 'an Adam moment is all zero'
        return [p.data(ctx)._data.detach().float().clone() for p in net.collect_params().values()]


def main():
    dist.ensure_initialized('nccl')
    rank, world = dist.rank(), dist.world_size()
    torch.cuda.set_device(dist.local_rank())
    ctx = mx.gpu(dist.local_rank())
    report = {'world': world, 'nvls_requested': bool(env.get('MXNET_KVSTORE_NVLS'))}
    for dtype in ('float32', 'float16'):
        w_fused = run(True, dtype, 6, ctx, rank, world)
        w_plain = run(False, dtype, 6, ctx, rank, world)
        err = max(float((a - b).abs().max()) for a, b in zip(w_fused, w_plain))
        flat = torch.cat([w.reshape(-1) for w in w_fused])
        gathered = [torch.empty_like(flat) for _ in range(world)]
        torch.distributed.all_gather(gathered, flat)
        same = all(bool(torch.equal(gathered[0], g)) for g in gathered)
        report[dtype] = {'max_abs_diff_vs_nccl_path': err, 'ranks_identical': same}
    for optimizer in ('lamb', 'adam'):
        w_fused = run(True, 'float32', 5, ctx, rank, world, optimizer)
        w_plain = run(False, 'float32', 5, ctx, rank, world, optimizer)
        err = max(float((a - b).abs().max()) for a, b in zip(w_fused, w_plain))
        flat = torch.cat([w.reshape(-1) for w in w_fused])
        gathered = [torch.empty_like(flat) for _ in range(world)]
        torch.distributed.all_gather(gathered, flat)
        report[optimizer] = {'max_abs_diff_vs_nccl_path': err,
                             'ranks_identical': all(bool(torch.equal(gathered[0], g)) for g in gathered)}
    report['multicast_steps'] = len(_MULTICAST)
    if rank == 0:
        print('REPORT ' + json.dumps(report))
    dist.barrier()
    dist.destroy()


if __name__ == '__main__':
    main()

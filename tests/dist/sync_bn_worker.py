"""Worker of the multi-GPU SyncBatchNorm test: launched once per GPU by ``torch.distributed.run``.

Checks the peer-memory all-reduce against the library all-reduce, and SyncBatchNorm on per-rank slices of a batch
against plain BatchNorm statistics of the whole batch (output, input gradient, running averages)."""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as tdist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import mxnet_b200 as mx                                   # noqa: E402
from mxnet_b200 import autograd, nd                       # noqa: E402
from mxnet_b200.parallel import dist, peer_reduce         # noqa: E402


def main():
    dist.ensure_initialized('nccl')
    rank, world = dist.rank(), dist.world_size()
    dev = torch.device('cuda', dist.local_rank())
    ctx = mx.gpu(dist.local_rank())
    rep = {'world': world}
    # ---- the collective itself ------------------------------------------------------------------
    assert peer_reduce.available(dev)
    pr = peer_reduce.get(dev)
    worst = 0.0
    for step, n in enumerate((1, 7, 256, 4096, 8192, 33)):
        v = torch.arange(n, device=dev, dtype=torch.float32) * (rank + 1) + step
        got = pr.allreduce(v)
        ref = v.clone()
        tdist.all_reduce(ref)
        worst = max(worst, float((got - ref).abs().max()))
    rep['allreduce_max_abs_diff'] = worst
    rep['status'] = pr.status()
    # ---- SyncBatchNorm ---------------------------------------------------------------------------
    rng = np.random.RandomState(5)
    per, C = 6, 16
    x_all = rng.randn(per * world, C, 5, 5).astype('float32')
    dy_all = rng.randn(per * world, C, 5, 5).astype('float32')
    x = nd.array(x_all[rank * per:(rank + 1) * per], ctx=ctx)
    gamma, beta = nd.array(rng.rand(C).astype('float32') + 0.5, ctx=ctx), nd.array(rng.randn(C).astype('float32'), ctx=ctx)
    mm, mv = nd.zeros((C,), ctx=ctx), nd.ones((C,), ctx=ctx)
    x.attach_grad()
    with autograd.record():
        y = nd.contrib.SyncBatchNorm(x, gamma, beta, mm, mv, fix_gamma=False, eps=1e-5, momentum=0.9, ndev=world, key='t')
    y.backward(nd.array(dy_all[rank * per:(rank + 1) * per], ctx=ctx))
    xt = torch.tensor(x_all, requires_grad=True)
    mean = xt.mean((0, 2, 3), keepdim=True)
    var = xt.var((0, 2, 3), unbiased=False, keepdim=True)
    yt = (xt - mean) / torch.sqrt(var + 1e-5) * torch.tensor(gamma.asnumpy()).reshape(1, C, 1, 1) + \
        torch.tensor(beta.asnumpy()).reshape(1, C, 1, 1)
    yt.backward(torch.tensor(dy_all))
    sl = slice(rank * per, (rank + 1) * per)
    rep['y_diff'] = float(np.abs(y.asnumpy() - yt.detach().numpy()[sl]).max())
    rep['dx_diff'] = float(np.abs(x.grad.asnumpy() - xt.grad.numpy()[sl]).max())
    rep['mean_diff'] = float(np.abs(mm.asnumpy() - 0.1 * mean.detach().numpy().reshape(-1)).max())
    rep['status_after'] = pr.status()
    gathered = dist.all_gather_object(rep)
    if rank == 0:
        merged = {k: max(g[k] for g in gathered) for k in rep}
        print('REPORT ' + json.dumps(merged))
    dist.destroy()


if __name__ == '__main__':
    main()

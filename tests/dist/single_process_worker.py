"""One process, several GPUs: ``Trainer(params over [gpu(0), ...])`` with ``split_and_load`` on the fused peer-memory
kernels, against the same training on one GPU through the generic per-parameter optimizer.  Run as a child process by
``tests/test_gpu_multi.py`` (argument: number of GPUs); prints one ``REPORT {json}`` line."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import numpy as np
import torch

import mxnet_b200 as mx
from mxnet_b200 import autograd, env, gluon, nd
from mxnet_b200.gluon import nn


def build(ctxs, dtype):
    mx.random.seed(11)
    np.random.seed(11)
    net = nn.HybridSequential()
    net.add(nn.Dense(96, activation='relu', in_units=48), nn.Dense(64, activation='relu', in_units=96),
            nn.Dense(10, in_units=64))
    net.initialize(mx.init.Xavier(), ctx=ctxs)
    if dtype != 'float32':
        net.cast(dtype)
    return net


def train(ctxs, fused, dtype, optimizer, steps=6):
    with env.scope('MXNET_KVSTORE_FUSED', '1' if fused else '0'):
        net = build(ctxs, dtype)
        opts = {'learning_rate': 0.05, 'wd': 1e-3, 'multi_precision': dtype != 'float32'}
        if optimizer == 'sgd':
            opts['momentum'] = 0.9
        trainer = gluon.Trainer(net.collect_params(), optimizer, opts, kvstore='device')
        loss_fn = gluon.loss.SoftmaxCrossEntropyLoss()
        rng = np.random.RandomState(5)
        per = 8 * len(ctxs) if len(ctxs) > 1 else 8 * N
        for _ in range(steps):
            x_all = rng.randn(8 * N, 48).astype('float32')
            y_all = rng.randint(0, 10, (8 * N,))
            xs = gluon.utils.split_and_load(nd.array(x_all, dtype=dtype), ctxs)
            ys = gluon.utils.split_and_load(nd.array(y_all), ctxs)
            with autograd.record():
                losses = [loss_fn(net(x), y) for x, y in zip(xs, ys)]
            autograd.backward(losses)
            trainer.step(8 * N)
        nd.waitall()
        from mxnet_b200.parallel import fused as F
        assert isinstance(trainer._fused, F.FusedStepGroup) == (fused and len(ctxs) > 1), type(trainer._fused)
        return [[p.data(c)._data.detach().float().cpu() for c in ctxs] for p in net.collect_params().values()], trainer


N = int(sys.argv[1]) if len(sys.argv) > 1 else 2
ctxs = [mx.gpu(i) for i in range(N)]
report = {'gpus': N}
for dtype, optimizer in (('float32', 'sgd'), ('float16', 'sgd'), ('float32', 'adam'), ('float32', 'lamb')):
    group, tr = train(ctxs, True, dtype, optimizer)
    ref, _ = train([mx.gpu(0)], False, dtype, optimizer)
    same = all(torch.equal(reps[0], r) for reps in group for r in reps[1:])
    diff = max(float((g[0] - r[0]).abs().max()) for g, r in zip(group, ref))
    report['%s_%s' % (dtype, optimizer)] = {'replicas_identical': bool(same), 'max_abs_diff_vs_one_gpu': diff}
# optimizer states written by this process alone and read back
import tempfile
fname = os.path.join(tempfile.mkdtemp(), 'trainer.states')
tr.save_states(fname)
tr.load_states(fname)
report['states_round_trip'] = os.path.getsize(fname) > 0
print('REPORT ' + json.dumps(report), flush=True)

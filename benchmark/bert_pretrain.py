#!/usr/bin/env python
"""BERT-base pre-training throughput (sequences/s): masked LM + next sentence prediction, sequence length 128,
batch 64 per GPU, 20 masked positions per sequence, LAMB, AMP, data parallel.  Synthetic token ids.

    python benchmark/bert_pretrain.py --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 benchmark/bert_pretrain.py
"""
import argparse
import sys

import _harness


def parser():
    ap = argparse.ArgumentParser()
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--batch', type=int, default=64)
    ap.add_argument('--seq-len', type=int, default=128)
    ap.add_argument('--masked', type=int, default=20)
    ap.add_argument('--dtype', default='float16', choices=['float16', 'bfloat16'])
    ap.add_argument('--layers', type=int, default=12)
    ap.add_argument('--graphs', type=int, default=1, help='hybridize(static_alloc, static_shape): CUDA-graph replay')
    return ap


def spec(args):
    """``(metric, unit, items per step and GPU, make_step, config)`` of this benchmark for the shared harness."""
    def make_step(ctx, rank, world):
        import numpy as np
        import mxnet_b200 as mx
        from mxnet_b200 import amp, autograd, gluon, nd
        from mxnet_b200.models.bert import BERTForPretrain
        amp.init(args.dtype)
        net = BERTForPretrain(vocab_size=30522, units=768, hidden_size=3072, num_layers=args.layers, num_heads=12,
                              max_length=512, dropout=0.1)
        net.initialize(mx.init.Normal(0.02), ctx=ctx)
        # low-precision weights, fp32 master copies inside the optimizer: no per-step casts of 110 M parameters
        net.cast(args.dtype)
        trainer = gluon.Trainer(net.collect_params(), 'lamb', {'learning_rate': 1e-4, 'wd': 0.01, 'epsilon': 1e-6,
                                                               'multi_precision': True}, kvstore='device')
        amp.init_trainer(trainer)
        if args.graphs:
            net.hybridize(static_alloc=True, static_shape=True)
        loss_fn = gluon.loss.SoftmaxCrossEntropyLoss()
        B, T, P = args.batch, args.seq_len, args.masked
        rng = np.random.RandomState(rank)
        batches = []
        for _ in range(2):
            batches.append((nd.array(rng.randint(0, 30522, (B, T)), ctx=ctx, dtype='int64'),
                            nd.array(rng.randint(0, 2, (B, T)), ctx=ctx, dtype='int64'),
                            nd.array(np.ones((B, T)), ctx=ctx, dtype='float32'),
                            nd.array(np.sort(rng.rand(B, T).argsort(1)[:, :P], 1), ctx=ctx, dtype='int64'),
                            nd.array(rng.randint(0, 30522, (B * P,)), ctx=ctx, dtype='int64'),
                            nd.array(rng.randint(0, 2, (B,)), ctx=ctx, dtype='int64')))
        it = [0]

        def step():
            ids, tt, mask, pos, mlm_y, nsp_y = batches[it[0] % 2]
            it[0] += 1
            with autograd.record():
                scores, nsp = net(ids, tt, mask, pos)
                loss = loss_fn(scores, mlm_y).mean() + loss_fn(nsp, nsp_y).mean()
                with amp.scale_loss(loss, trainer) as scaled:
                    autograd.backward(scaled)
            trainer.step(1)
            return loss
        return step
    cfg = {'model': 'bert_base' if args.layers == 12 else 'bert_%dL' % args.layers, 'batch_per_gpu': args.batch,
           'seq_len': args.seq_len, 'masked_per_seq': args.masked, 'optimizer': 'lamb (multi-precision)', 'amp': args.dtype, 'cuda_graphs': bool(args.graphs)}
    return 'bert_pretrain_seq_per_s', 'seq/s', args.batch, make_step, cfg


def main():
    args = parser().parse_args()
    name, unit, items, make_step, cfg = spec(args)
    return _harness.run(name, unit, items, make_step, args, cfg)


if __name__ == '__main__':
    sys.exit(main())

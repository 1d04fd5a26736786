#!/usr/bin/env python
"""Word-level LSTM language model throughput (tokens/s): 2 layers x 650 units, tied embedding, vocabulary 33278,
bptt 35, batch 80 per GPU, SGD with global-norm clipping 0.25 (the reference's example/gluon/word_language_model
configuration).  Synthetic token ids.

    python benchmark/lstm_lm.py --steps 20 --warmup 5
"""
import argparse
import sys

import _harness


def parser():
    ap = argparse.ArgumentParser()
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--batch', type=int, default=80)
    ap.add_argument('--bptt', type=int, default=35)
    ap.add_argument('--dtype', default='float32', choices=['float32', 'float16'])
    ap.add_argument('--tf32', action='store_true',
                    help='fp32 GEMMs (the decoder above all) with tf32 operands: MXNET_CUDA_ALLOW_TF32=1, the math mode the '
                         'reference sets for its fp32 cuBLAS calls (src/operator/linalg_impl.h:298)')
    return ap


def spec(args):
    """``(metric, unit, items per step and GPU, make_step, config)`` of this benchmark for the shared harness."""
    def make_step(ctx, rank, world):
        import numpy as np
        import mxnet_b200 as mx
        from mxnet_b200 import autograd, gluon, nd
        from mxnet_b200 import env
        from mxnet_b200.models.lstm_lm import LSTMLanguageModel
        env.set('MXNET_CUDA_ALLOW_TF32', bool(args.tf32))
        net = LSTMLanguageModel(vocab_size=33278, embed_size=650, hidden_size=650, num_layers=2, dropout=0.5)
        net.initialize(mx.init.Xavier(), ctx=ctx)
        if args.dtype != 'float32':
            net.cast(args.dtype)
        trainer = gluon.Trainer(net.collect_params(), 'sgd', {'learning_rate': 20.0 if args.dtype == 'float32' else 1.0,
                                                              'multi_precision': args.dtype != 'float32'}, kvstore='device')
        loss_fn = gluon.loss.SoftmaxCrossEntropyLoss()
        B, T = args.batch, args.bptt
        rng = np.random.RandomState(rank)
        data = [nd.array(rng.randint(0, 33278, (T, B)), ctx=ctx, dtype='int64') for _ in range(2)]
        target = [nd.array(rng.randint(0, 33278, (T * B,)), ctx=ctx, dtype='int64') for _ in range(2)]
        hidden = [net.begin_state(B, ctx=ctx, dtype=args.dtype)]
        params = [p for p in net.collect_params().values() if p.grad_req != 'null']
        it = [0]

        def step():
            x, y = data[it[0] % 2], target[it[0] % 2]
            it[0] += 1
            h = [s.detach() for s in hidden[0]]
            with autograd.record():
                out, h = net(x, h)
                loss = loss_fn(out, y)
            loss.backward()
            hidden[0] = h
            if trainer._fused is not None:
                trainer._fused.set_global_norm_clip(0.25 * T * B * world)
            else:
                gluon.utils.clip_global_norm([p.grad(ctx) for p in params], 0.25 * T * B)
            trainer.step(T * B * world)
            return loss
        return step
    cfg = {'model': 'lstm_lm_2x650', 'batch_per_gpu': args.batch, 'bptt': args.bptt, 'vocab': 33278,
           'optimizer': 'sgd + global-norm clip 0.25', 'dtype': args.dtype,
           'fp32_gemm_math': 'tf32 operands, fp32 accumulation' if args.tf32 else 'fp32'}
    return 'lstm_lm_tokens_per_s', 'tokens/s', args.batch * args.bptt, make_step, cfg


def main():
    args = parser().parse_args()
    name, unit, items, make_step, cfg = spec(args)
    return _harness.run(name, unit, items, make_step, args, cfg)


if __name__ == '__main__':
    sys.exit(main())

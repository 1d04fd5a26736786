#!/usr/bin/env python
"""Word-level language model with a multi-layer LSTM, tied input/output embeddings, dropout, truncated BPTT and global
gradient-norm clipping (the flow of example/gluon/word_language_model in MXNet).

    python example/gluon/word_language_model/train.py --epochs 1 [--gpu] [--data FILE]

`--data` is a plain-text corpus (one sentence per line); without it a synthetic corpus with a learnable bigram
structure is generated."""
import argparse
import math
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), '..', '..', '..'))
import mxnet_b200 as mx                                    # noqa: E402
from mxnet_b200 import autograd, gluon, nd                 # noqa: E402
from mxnet_b200.models.lstm_lm import LSTMLanguageModel    # noqa: E402


def corpus(path, vocab_size, length, rng):
    if path:
        words = open(path).read().replace('\n', ' <eos> ').split()
        vocab = {w: i for i, w in enumerate(sorted(set(words)))}
        return np.array([vocab[w] for w in words], dtype='int64'), len(vocab)
    nxt = rng.randint(0, vocab_size, (vocab_size, 2))          # every word is followed by one of two fixed words
    ids = np.zeros(length, dtype='int64')
    for i in range(1, length):
        ids[i] = nxt[ids[i - 1], rng.randint(0, 2)]
    return ids, vocab_size


def batchify(ids, batch_size):
    n = len(ids) // batch_size
    return ids[:n * batch_size].reshape(batch_size, n).T      # (time, batch)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--data', default=None)
    ap.add_argument('--vocab', type=int, default=200)
    ap.add_argument('--tokens', type=int, default=20000)
    ap.add_argument('--emsize', type=int, default=64)
    ap.add_argument('--nhid', type=int, default=64)
    ap.add_argument('--nlayers', type=int, default=2)
    ap.add_argument('--lr', type=float, default=1.0)
    ap.add_argument('--clip', type=float, default=0.25)
    ap.add_argument('--epochs', type=int, default=1)
    ap.add_argument('--batch-size', type=int, default=20)
    ap.add_argument('--bptt', type=int, default=20)
    ap.add_argument('--dropout', type=float, default=0.2)
    ap.add_argument('--gpu', action='store_true')
    args = ap.parse_args(argv)
    ctx = mx.gpu(0) if args.gpu else mx.cpu()
    ids, vocab = corpus(args.data, args.vocab, args.tokens, np.random.RandomState(0))
    data = batchify(ids, args.batch_size)
    net = LSTMLanguageModel(vocab_size=vocab, embed_size=args.emsize, hidden_size=args.nhid, num_layers=args.nlayers,
                            dropout=args.dropout)
    net.initialize(mx.init.Xavier(), ctx=ctx)
    trainer = gluon.Trainer(net.collect_params(), 'sgd', {'learning_rate': args.lr})
    loss_fn = gluon.loss.SoftmaxCrossEntropyLoss()
    params = [p for p in net.collect_params().values() if p.grad_req != 'null']
    ppl = float('inf')
    for epoch in range(args.epochs):
        hidden = net.begin_state(args.batch_size, ctx=ctx)
        total, count = 0.0, 0
        for i in range(0, data.shape[0] - 1 - args.bptt, args.bptt):
            x = nd.array(data[i:i + args.bptt], ctx=ctx, dtype='int64')
            y = nd.array(data[i + 1:i + 1 + args.bptt].reshape(-1), ctx=ctx, dtype='int64')
            hidden = [h.detach() for h in hidden]
            with autograd.record():
                out, hidden = net(x, hidden)
                loss = loss_fn(out, y)
            loss.backward()
            gluon.utils.clip_global_norm([p.grad(ctx) for p in params], args.clip * args.bptt * args.batch_size)
            trainer.step(args.bptt * args.batch_size)
            total += float(loss.sum().asscalar())
            count += loss.size
        ppl = math.exp(total / count)
        print('epoch %d: training perplexity %.2f (uniform guess: %d)' % (epoch, ppl, vocab))
    return ppl


if __name__ == '__main__':
    main()

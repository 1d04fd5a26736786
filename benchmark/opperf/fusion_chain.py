"""Pointwise fusion on a bias + GELU + scale + residual chain (four operators, three tensors in, one out): the
generated kernel against the same Symbol run operator by operator.

    python benchmark/opperf/fusion_chain.py --rows 32768 --cols 3072 [--dtype float16]

Prints one JSON line: device time of forward and of forward+backward for both modes (CUDA events, median of the timed
iterations, L2 flushed between iterations) and the achieved bandwidth of the fused forward (algorithmic bytes: two
full tensors read, one written)."""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), '..', '..'))


def timed(fn, flush, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return sorted(ts)[len(ts) // 2] * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--rows', type=int, default=32768)
    ap.add_argument('--cols', type=int, default=3072)
    ap.add_argument('--dtype', default='float16')
    ap.add_argument('--iters', type=int, default=10)
    args = ap.parse_args()
    import mxnet_b200 as mx
    from mxnet_b200 import env
    from mxnet_b200.symbol import fusion
    dtype = getattr(torch, args.dtype)
    dev = torch.device('cuda', 0)
    x, b, r = mx.sym.var('x'), mx.sym.var('b'), mx.sym.var('r')
    s = mx.sym.LeakyReLU(mx.sym.broadcast_add(x, b), act_type='gelu') * 0.5 + r
    feed = {'x': torch.randn(args.rows, args.cols, device=dev).to(dtype), 'b': torch.randn(args.cols, device=dev).to(dtype),
            'r': torch.randn(args.rows, args.cols, device=dev).to(dtype)}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    res = {'rows': args.rows, 'cols': args.cols, 'dtype': args.dtype}
    for mode, flag in (('fused', '1'), ('unfused', '0')):
        with env.scope('MXNET_USE_FUSION', flag):
            g = mx.sym.Group([s])

            def fwd():
                with torch.no_grad():
                    return g._run(feed)[0]

            def fwd_bwd():
                f = {k: v.detach().requires_grad_(True) for k, v in feed.items()}
                g._run(f)[0].backward(feed['r'])

            res[mode + '_fwd_us'] = round(timed(fwd, flush, args.iters), 1)
            res[mode + '_fwd_bwd_us'] = round(timed(fwd_bwd, flush, args.iters), 1)
    nbytes = 3 * args.rows * args.cols * feed['x'].element_size()
    res['fused_fwd_gbs'] = round(nbytes / res['fused_fwd_us'] / 1e3, 1)
    res['kernel_calls'] = fusion.stats['kernel_calls']
    print(json.dumps(res))


if __name__ == '__main__':
    main()

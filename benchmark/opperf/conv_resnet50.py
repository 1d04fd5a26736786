"""Per-layer timing of the stride-1 convolutions of ResNet-50 v1b (NHWC, half precision): the tcgen05 implicit-GEMM
kernels against the library convolution, forward / data gradient / weight gradient.

    python benchmark/opperf/conv_resnet50.py --batch 256 --iters 10 [--dtype float16] [--layers 3x3]

One JSON line per layer and direction: device time in microseconds (CUDA events around each launch, L2 flushed by
writing a 256 MiB buffer before every timed launch), the layer's multiplicity in the network, and at the end the
multiplicity-weighted totals."""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), '..', '..'))

# (name, H=W, Cin, Cout, R, count in ResNet-50 v1b)
LAYERS = [
    ('s1_1x1_64_64', 56, 64, 64, 1, 1), ('s1_3x3_64_64', 56, 64, 64, 3, 3), ('s1_1x1_64_256', 56, 64, 256, 1, 4),
    ('s1_1x1_256_64', 56, 256, 64, 1, 2), ('s2_1x1_256_128', 56, 256, 128, 1, 1), ('s2_3x3_128_128', 28, 128, 128, 3, 3),
    ('s2_1x1_128_512', 28, 128, 512, 1, 4), ('s2_1x1_512_128', 28, 512, 128, 1, 3), ('s3_1x1_512_256', 28, 512, 256, 1, 1),
    ('s3_3x3_256_256', 14, 256, 256, 3, 5), ('s3_1x1_256_1024', 14, 256, 1024, 1, 6), ('s3_1x1_1024_256', 14, 1024, 256, 1, 5),
    ('s4_1x1_1024_512', 14, 1024, 512, 1, 1), ('s4_3x3_512_512', 7, 512, 512, 3, 2), ('s4_1x1_512_2048', 7, 512, 2048, 1, 3),
    ('s4_1x1_2048_512', 7, 2048, 512, 1, 2),
]


def timed(fn, flush, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--batch', type=int, default=256)
    ap.add_argument('--iters', type=int, default=10)
    ap.add_argument('--dtype', default='float16')
    ap.add_argument('--layers', default='')
    ap.add_argument('--dirs', default='fwd,dgrad,wgrad')
    ap.add_argument('--profile', action='store_true', help='print the cycle accounting of CTA 0 of the in-tree kernel')
    ap.add_argument('--no-stats', action='store_true', help='forward without the BatchNorm statistics epilogue')
    args = ap.parse_args()
    from mxnet_b200.ops.cuda import conv_ops, gemm_ops
    dtype = getattr(torch, args.dtype)
    dev = torch.device('cuda', 0)
    torch.backends.cudnn.benchmark = True
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    totals = {}
    for name, hw, cin, cout, r, count in LAYERS:
        if args.layers and args.layers not in name:
            continue
        pad = (r // 2, r // 2)
        x = torch.randn(args.batch, hw, hw, cin, device=dev).to(dtype)
        w = (torch.randn(cout, r, r, cin, device=dev) / (r * cin ** 0.5)).to(dtype)
        dy = torch.randn(args.batch, hw, hw, cout, device=dev).to(dtype)
        xc, wc, dyc = x.permute(0, 3, 1, 2), w.permute(0, 3, 1, 2), dy.permute(0, 3, 1, 2)
        flops = 2.0 * args.batch * hw * hw * cin * cout * r * r
        runs = {
            'fwd': (lambda: conv_ops.conv_forward(x, w, None, None, pad, (1, 1), False, not args.no_stats),
                    lambda: torch.nn.functional.conv2d(xc, wc, None, 1, pad, 1)),
            'dgrad': (lambda: conv_ops.conv_dgrad(dy, w, (hw, hw), pad, (1, 1)),
                      lambda: torch.ops.aten.convolution_backward(dyc, xc, wc, None, [1, 1], list(pad), [1, 1], False, [0, 0],
                                                                  1, [True, False, False])),
            'wgrad': (lambda: conv_ops.conv_wgrad(x, dy, (r, r), pad, (1, 1)),
                      lambda: torch.ops.aten.convolution_backward(dyc, xc, wc, None, [1, 1], list(pad), [1, 1], False, [0, 0],
                                                                  1, [False, True, False])),
        }
        for d, (own, libf) in runs.items():
            if d not in args.dirs.split(','):
                continue
            if args.profile and d != 'wgrad':
                import ctypes
                from mxnet_b200.ops import cuda as _cuda
                buf = torch.zeros(16, dtype=torch.int64, device=dev)
                _cuda.lib().mxb_conv_set_profile(ctypes.c_void_p(buf.data_ptr()))
                own()
                torch.cuda.synchronize()
                _cuda.lib().mxb_conv_set_profile(None)
                names = ['prod_wait_stage', 'prod_total', 'ksteps', 'mma_wait_operands', 'mma_wait_accumulator', 'mma_total',
                         'tiles', 'epi_wait', 'epi_total', 'prod_expect_tx', 'prod_tma_issue', 'mma_issue', 'mma_commit',
                         'prod_loop', 'mma_loop']
                print(json.dumps({'layer': name, 'dir': d, 'cycles_cta0': dict(zip(names, buf.tolist()))}), flush=True)
            t_own = timed(own, flush, args.iters)
            t_lib = timed(libf, flush, args.iters)
            gemm_ops.check_errors()
            tot = totals.setdefault(d, [0.0, 0.0])
            tot[0] += t_own * count
            tot[1] += t_lib * count
            print(json.dumps({'layer': name, 'dir': d, 'count': count, 'own_us': round(t_own, 1), 'lib_us': round(t_lib, 1),
                              'own_tflops': round(flops / t_own / 1e6, 1), 'ratio_lib_over_own': round(t_lib / t_own, 3)}),
                  flush=True)
        del x, w, dy
    for d, (a, b) in totals.items():
        print(json.dumps({'total': d, 'own_ms': round(a / 1e3, 3), 'lib_ms': round(b / 1e3, 3)}), flush=True)


if __name__ == '__main__':
    main()

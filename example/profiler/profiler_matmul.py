#!/usr/bin/env python
"""Profile a loop of matrix products (the flow of example/profiler/profiler_matmul.py in MXNet): operator records,
a user scope with a counter and a marker, the Chrome-trace file and the aggregate table.

    python example/profiler/profiler_matmul.py --iters 20 --size 512 [--gpu] [--file profile_matmul.json]

Open the file in chrome://tracing or Perfetto."""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), '..', '..'))
import mxnet_b200 as mx                                    # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument('--iters', type=int, default=20)
    ap.add_argument('--size', type=int, default=512)
    ap.add_argument('--gpu', action='store_true')
    ap.add_argument('--file', default='profile_matmul.json')
    args = ap.parse_args(argv)
    ctx = mx.gpu(0) if args.gpu else mx.cpu()
    mx.profiler.set_config(profile_all=True, aggregate_stats=True, filename=args.file)
    a = mx.nd.random.uniform(-1, 1, (args.size, args.size), ctx=ctx)
    b = mx.nd.random.uniform(-1, 1, (args.size, args.size), ctx=ctx)
    mx.nd.dot(a, b).wait_to_read()                          # warm up outside the profile
    mx.profiler.set_state('run')
    domain = mx.profiler.Domain('example')
    counter = domain.new_counter('products', 0)
    with domain.new_task('matmul loop'):
        for i in range(args.iters):
            c = mx.nd.dot(a, b)
            counter.increment(1)
            if i == args.iters // 2:
                domain.new_marker('half way').mark('process')
        c.wait_to_read()
    mx.profiler.set_state('stop')
    table = mx.profiler.dumps()
    mx.profiler.dump()
    print(table)
    print('trace written to', os.path.abspath(args.file))
    return table


if __name__ == '__main__':
    main()

"""Run one test many times with different seeds to expose flakiness:

    python -m mxnet_b200.tools.flakiness_checker tests/test_gluon.py::test_dense -n 50 [-s SEED]

Each trial runs pytest on the given node with ``MXNET_TEST_SEED`` set (a fixed seed with ``-s``, else a fresh one per
trial) and the failing seeds are reported (reference: tools/flakiness_checker.py)."""
import argparse
import os
import random
import subprocess
import sys


def run_trials(test, trials, seed=None, verbosity=0):
    failed = []
    for i in range(trials):
        s = seed if seed is not None else random.randint(0, 2 ** 31 - 1)
        env = dict(os.environ, MXNET_TEST_SEED=str(s))
        r = subprocess.run([sys.executable, '-m', 'pytest', '-x', '-q', test], env=env, capture_output=True, text=True)
        if r.returncode != 0:
            failed.append(s)
            if verbosity:
                print(r.stdout[-2000:])
        print('trial %d/%d seed %d: %s' % (i + 1, trials, s, 'FAILED' if r.returncode else 'ok'), flush=True)
    return failed


def main(argv=None):
    ap = argparse.ArgumentParser(description='check a test for flakiness')
    ap.add_argument('test', help='pytest node id, e.g. tests/test_gluon.py::test_dense')
    ap.add_argument('-n', '--num-trials', type=int, default=20)
    ap.add_argument('-s', '--seed', type=int, default=None)
    ap.add_argument('-v', '--verbosity', type=int, default=0)
    args = ap.parse_args(argv)
    failed = run_trials(args.test, args.num_trials, args.seed, args.verbosity)
    print('%d of %d trials failed%s' % (len(failed), args.num_trials, (': seeds %s' % failed) if failed else ''))
    return 1 if failed else 0


if __name__ == '__main__':
    sys.exit(main())

"""Tabulate a training log:  python -m mxnet_b200.tools.parse_log train.log [--format markdown|none] [--metric-names accuracy]

Understands the lines written by ``callback.Speedometer`` / ``model.fit`` / the estimator's LoggingHandler:
``Epoch[3] Train-accuracy=0.91``, ``Epoch[3] Validation-accuracy=0.88``, ``Epoch[3] Time cost=12.3``
(reference: tools/parse_log.py)."""
import argparse
import re
import sys


def parse(lines, metric_names=('accuracy',)):
    """{epoch: {'train-<m>': v, 'val-<m>': v, 'time': v}} with the last value seen per epoch."""
    pats = [(re.compile(r'Epoch\[(\d+)\].*?Train-' + re.escape(m) + r'.*?=([.\deE+-]+)'), 'train-' + m) for m in metric_names]
    pats += [(re.compile(r'Epoch\[(\d+)\].*?Validation-' + re.escape(m) + r'.*?=([.\deE+-]+)'), 'val-' + m) for m in metric_names]
    pats.append((re.compile(r'Epoch\[(\d+)\].*?Time cost=([.\deE+-]+)'), 'time'))
    table = {}
    for line in lines:
        for pat, name in pats:
            m = pat.search(line)
            if m:
                table.setdefault(int(m.group(1)), {})[name] = float(m.group(2))
    return table


def render(table, metric_names, fmt='markdown'):
    cols = ['train-' + m for m in metric_names] + ['val-' + m for m in metric_names] + ['time']
    out = []
    if fmt == 'markdown':
        out.append('| epoch | ' + ' | '.join(cols) + ' |')
        out.append('| --- | ' + ' | '.join('---' for _ in cols) + ' |')
    for ep in sorted(table):
        vals = ['%.6g' % table[ep][c] if c in table[ep] else '' for c in cols]
        out.append(('| %d | ' % ep + ' | '.join(vals) + ' |') if fmt == 'markdown' else ' '.join([str(ep)] + vals))
    return '\n'.join(out)


def main(argv=None):
    ap = argparse.ArgumentParser(description='parse a training log')
    ap.add_argument('logfile')
    ap.add_argument('--format', default='markdown', choices=['markdown', 'none'])
    ap.add_argument('--metric-names', nargs='+', default=['accuracy'])
    args = ap.parse_args(argv)
    with open(args.logfile) as f:
        table = parse(f, args.metric_names)
    print(render(table, args.metric_names, args.format))
    return 0


if __name__ == '__main__':
    sys.exit(main())

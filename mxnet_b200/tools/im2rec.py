"""Create image lists and RecordIO packs from a folder of images.

    python -m mxnet_b200.tools.im2rec PREFIX ROOT --list [--recursive] [--train-ratio 0.9] [--no-shuffle]
    python -m mxnet_b200.tools.im2rec PREFIX ROOT [--resize 256] [--quality 95] [--encoding .jpg] [--num-thread 8]

The first form writes ``PREFIX.lst`` (or ``PREFIX_train.lst`` / ``PREFIX_val.lst`` / ``PREFIX_test.lst``) with lines
``index<TAB>label<TAB>relative/path``; with ``--recursive`` every sub-folder of ROOT is one class.  The second form reads
every ``PREFIX*.lst`` and writes ``.rec`` + ``.idx`` files of packed, optionally resized and centre-cropped images.
Same list format, record format and options as the reference's tools/im2rec.py."""
import argparse
import os
import random
import sys
from concurrent.futures import ThreadPoolExecutor

import numpy as np

EXTS = ('.jpeg', '.jpg', '.png', '.bmp')


def list_images(root, recursive, exts=EXTS):
    """Yield (index, relative path, label); labels follow the sorted order of class folders."""
    i = 0
    if recursive:
        cat = {}
        for path, dirs, files in os.walk(root, followlinks=True):
            dirs.sort()
            for fname in sorted(files):
                if os.path.splitext(fname)[1].lower() not in exts:
                    continue
                label_dir = os.path.relpath(path, root)
                if label_dir not in cat:
                    cat[label_dir] = len(cat)
                yield i, os.path.join(label_dir, fname) if label_dir != '.' else fname, cat[label_dir]
                i += 1
    else:
        for fname in sorted(os.listdir(root)):
            if os.path.isfile(os.path.join(root, fname)) and os.path.splitext(fname)[1].lower() in exts:
                yield i, fname, 0
                i += 1


def write_list(path, items):
    with open(path, 'w') as f:
        for idx, rel, label in items:
            f.write('%d\t%f\t%s\n' % (idx, label, rel))


def make_list(args):
    items = list(list_images(args.root, args.recursive))
    if args.shuffle:
        random.seed(100)
        random.shuffle(items)
    n = len(items)
    chunk = (n + args.chunks - 1) // args.chunks
    for c in range(args.chunks):
        part = items[c * chunk:(c + 1) * chunk]
        suffix = '_%d' % c if args.chunks > 1 else ''
        n_test = int(len(part) * args.test_ratio)
        n_train = int(len(part) * args.train_ratio)
        if args.train_ratio == 1.0 and n_test == 0:
            write_list(args.prefix + suffix + '.lst', part)
            continue
        if n_test:
            write_list(args.prefix + suffix + '_test.lst', part[:n_test])
        write_list(args.prefix + suffix + '_train.lst', part[n_test:n_test + n_train])
        if args.train_ratio + args.test_ratio < 1.0:
            write_list(args.prefix + suffix + '_val.lst', part[n_test + n_train:])


def read_list(path):
    with open(path) as f:
        for line in f:
            parts = line.rstrip('\n').split('\t')
            if len(parts) < 3:
                continue
            yield int(parts[0]), parts[-1], [float(x) for x in parts[1:-1]]


def _load(fullpath, args):
    from PIL import Image
    if args.pass_through:
        with open(fullpath, 'rb') as f:
            return f.read()
    im = Image.open(fullpath)
    im = im.convert('L' if args.color == 0 else 'RGB')
    if args.center_crop:
        w, h = im.size
        m = min(w, h)
        im = im.crop(((w - m) // 2, (h - m) // 2, (w - m) // 2 + m, (h - m) // 2 + m))
    if args.resize:
        w, h = im.size
        if w > h:
            im = im.resize((max(1, w * args.resize // h), args.resize))
        else:
            im = im.resize((args.resize, max(1, h * args.resize // w)))
    arr = np.asarray(im)
    return arr[..., ::-1] if arr.ndim == 3 else arr          # BGR, the order pack_img expects


def pack_list(lst_path, args):
    from .. import recordio
    base = os.path.splitext(lst_path)[0]
    items = list(read_list(lst_path))
    rec = recordio.MXIndexedRecordIO(base + '.idx', base + '.rec', 'w')

    def encode(item):
        idx, rel, labels = item
        try:
            data = _load(os.path.join(args.root, rel), args)
        except Exception as e:                      # unreadable image: skip it, like the reference
            print('skipping %s: %s' % (rel, e), file=sys.stderr)
            return idx, None
        label = labels[0] if len(labels) == 1 and not args.pack_label else np.asarray(labels, dtype='float32')
        header = recordio.IRHeader(0, label, idx, 0)
        if args.pass_through:
            return idx, recordio.pack(header, data)
        return idx, recordio.pack_img(header, data, quality=args.quality, img_fmt=args.encoding)

    count = 0
    with ThreadPoolExecutor(max_workers=max(1, args.num_thread)) as ex:
        for idx, buf in ex.map(encode, items):       # map keeps list order, so the pack is reproducible
            if buf is None:
                continue
            rec.write_idx(idx, buf)
            count += 1
    rec.close()
    return count


def main(argv=None):
    ap = argparse.ArgumentParser(description='make an image list or pack images into RecordIO')
    ap.add_argument('prefix')
    ap.add_argument('root')
    ap.add_argument('--list', action='store_true')
    ap.add_argument('--exts', nargs='+', default=list(EXTS))
    ap.add_argument('--chunks', type=int, default=1)
    ap.add_argument('--train-ratio', type=float, default=1.0)
    ap.add_argument('--test-ratio', type=float, default=0.0)
    ap.add_argument('--recursive', action='store_true')
    ap.add_argument('--no-shuffle', dest='shuffle', action='store_false')
    ap.add_argument('--pass-through', action='store_true')
    ap.add_argument('--resize', type=int, default=0)
    ap.add_argument('--center-crop', action='store_true')
    ap.add_argument('--quality', type=int, default=95)
    ap.add_argument('--num-thread', type=int, default=1)
    ap.add_argument('--color', type=int, default=1, choices=[-1, 0, 1])
    ap.add_argument('--encoding', default='.jpg', choices=['.jpg', '.png'])
    ap.add_argument('--pack-label', action='store_true')
    args = ap.parse_args(argv)
    if args.list:
        make_list(args)
        return 0
    d = os.path.dirname(os.path.abspath(args.prefix))
    stem = os.path.basename(args.prefix)
    lists = sorted(os.path.join(d, f) for f in os.listdir(d) if f.startswith(stem) and f.endswith('.lst'))
    if not lists:
        print('no .lst file with prefix %s' % args.prefix, file=sys.stderr)
        return 1
    for lst in lists:
        print('%s: %d records' % (lst, pack_list(lst, args)))
    return 0


if __name__ == '__main__':
    sys.exit(main())

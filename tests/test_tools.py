"""The command-line tools: image list / RecordIO packing, index rebuild, log parsing, environment report."""
import os

import numpy as np

from mxnet_b200 import recordio
from mxnet_b200.tools import diagnose, im2rec, parse_log, rec2idx


def _make_images(root):
    from PIL import Image
    rng = np.random.RandomState(0)
    for cls in ('cat', 'dog'):
        os.makedirs(os.path.join(root, cls))
        for i in range(3):
            Image.fromarray(rng.randint(0, 255, (20 + i, 30, 3), dtype=np.uint8)).save(os.path.join(root, cls, '%d.png' % i))


def test_im2rec_list_pack_and_rec2idx(tmp_path):
    root = str(tmp_path / 'imgs')
    _make_images(root)
    prefix = str(tmp_path / 'data')
    assert im2rec.main([prefix, root, '--list', '--recursive', '--no-shuffle']) == 0
    items = list(im2rec.read_list(prefix + '.lst'))
    assert len(items) == 6 and [l[0] for _, _, l in items] == [0.0] * 3 + [1.0] * 3
    assert im2rec.main([prefix, root, '--resize', '16', '--encoding', '.png', '--num-thread', '2']) == 0
    rec = recordio.MXIndexedRecordIO(prefix + '.idx', prefix + '.rec', 'r')
    assert sorted(rec.keys) == list(range(6))
    header, img = recordio.unpack_img(rec.read_idx(4))
    assert header.label == 1.0 and min(img.shape[:2]) == 16 and img.shape[2] == 3
    rec.close()
    # rebuilding the index from the .rec alone gives the same offsets
    assert rec2idx.main([prefix + '.rec', prefix + '.idx2']) == 0
    a = [l.split('\t')[1] for l in open(prefix + '.idx').read().strip().split('\n')]
    b = [l.split('\t')[1] for l in open(prefix + '.idx2').read().strip().split('\n')]
    assert a == b


def test_im2rec_train_val_split(tmp_path):
    root = str(tmp_path / 'imgs')
    _make_images(root)
    prefix = str(tmp_path / 'split')
    im2rec.main([prefix, root, '--list', '--recursive', '--train-ratio', '0.5'])
    n_train = len(list(im2rec.read_list(prefix + '_train.lst')))
    n_val = len(list(im2rec.read_list(prefix + '_val.lst')))
    assert n_train == 3 and n_val == 3


def test_parse_log(tmp_path, capsys):
    log = tmp_path / 'train.log'
    log.write_text('INFO Epoch[0] Batch [20] Speed: 100 samples/sec accuracy=0.1\n'
                   'INFO Epoch[0] Train-accuracy=0.50\nINFO Epoch[0] Time cost=12.5\nINFO Epoch[0] Validation-accuracy=0.40\n'
                   'INFO Epoch[1] Train-accuracy=0.75\nINFO Epoch[1] Time cost=11.0\nINFO Epoch[1] Validation-accuracy=0.70\n')
    table = parse_log.parse(open(str(log)))
    assert table[1] == {'train-accuracy': 0.75, 'val-accuracy': 0.70, 'time': 11.0}
    assert parse_log.main([str(log)]) == 0
    out = capsys.readouterr().out
    assert '| 0 | 0.5 | 0.4 | 12.5 |' in out


def test_diagnose_reports_sections():
    text = diagnose.report()
    for title in ('Platform', 'Python', 'Framework', 'Native libraries', 'GPUs'):
        assert title in text
    assert 'libmxb200_rt.so' in text

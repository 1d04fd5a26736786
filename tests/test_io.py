"""Data iterators, RecordIO and image helpers (reference: tests/python/unittest/test_io.py, test_recordio.py,
test_image.py, test_gluon_data.py)."""
import os
import struct

import numpy as np
import pytest

import mxnet_b200 as mx
from mxnet_b200 import gluon, nd, recordio
from mxnet_b200.test_utils import assert_almost_equal, same


def test_recordio_sequential_and_magic(tmp_path):
    f = str(tmp_path / 'a.rec')
    w = recordio.MXRecordIO(f, 'w')
    payloads = [b'x' * n for n in (1, 3, 4, 5, 1000)] + [bytes(range(256))]
    for p in payloads:
        w.write(p)
    w.close()
    raw = open(f, 'rb').read()
    magic, lrec = struct.unpack('<II', raw[:8])
    assert magic == 0xced7230a and (lrec & ((1 << 29) - 1)) == 1 and len(raw) % 4 == 0
    r = recordio.MXRecordIO(f, 'r')
    got = []
    while True:
        item = r.read()
        if item is None:
            break
        got.append(item)
    assert got == payloads
    r.reset()
    assert r.read() == payloads[0]
    r.close()


def test_recordio_payload_containing_magic(tmp_path):
    """A payload that contains the magic word is split into continuation records and reassembled."""
    f = str(tmp_path / 'm.rec')
    magic = struct.pack('<I', 0xced7230a)
    payload = b'abcd' + magic + b'efgh' + magic + magic + b'ij'
    w = recordio.MXRecordIO(f, 'w')
    w.write(payload)
    w.write(b'next')
    w.close()
    r = recordio.MXRecordIO(f, 'r')
    assert r.read() == payload and r.read() == b'next' and r.read() is None


def test_indexed_recordio_and_pack(tmp_path):
    rec, idx = str(tmp_path / 'a.rec'), str(tmp_path / 'a.idx')
    w = recordio.MXIndexedRecordIO(idx, rec, 'w')
    for i in range(10):
        header = recordio.IRHeader(0, float(i), i, 0)
        w.write_idx(i, recordio.pack(header, ('payload%d' % i).encode()))
    w.close()
    r = recordio.MXIndexedRecordIO(idx, rec, 'r')
    assert sorted(r.keys) == list(range(10))
    for i in (7, 2, 9, 0):
        h, s = recordio.unpack(r.read_idx(i))
        assert h.label == float(i) and h.id == i and s == ('payload%d' % i).encode()
    h = recordio.IRHeader(0, np.array([1., 2., 3.], 'float32'), 5, 0)
    h2, s2 = recordio.unpack(recordio.pack(h, b'zz'))
    assert h2.flag == 3 and same(h2.label, np.array([1., 2., 3.], 'float32')) and s2 == b'zz'


def test_pack_img_round_trip():
    img = (np.random.rand(16, 20, 3) * 255).astype('uint8')
    s = recordio.pack_img(recordio.IRHeader(0, 1.0, 0, 0), img, img_fmt='.png')
    h, back = recordio.unpack_img(s)
    assert h.label == 1.0 and back.shape == (16, 20, 3) and same(back, img)


def test_ndarray_iter_padding_and_shuffle():
    data = np.arange(50, dtype='float32').reshape(10, 5)
    label = np.arange(10, dtype='float32')
    it = mx.io.NDArrayIter(data, label, batch_size=4, last_batch_handle='pad')
    assert it.provide_data[0].shape == (4, 5) and it.provide_label[0].name == 'softmax_label'
    batches = list(it)
    assert len(batches) == 3 and batches[-1].pad == 2
    assert same(batches[0].data[0].asnumpy(), data[:4])
    it = mx.io.NDArrayIter(data, label, batch_size=4, last_batch_handle='discard')
    assert len(list(it)) == 2
    it = mx.io.NDArrayIter({'a': data, 'b': data * 2}, {'l': label}, batch_size=5, shuffle=True)
    seen = []
    for b in it:
        assert_almost_equal(b.data[1].asnumpy(), b.data[0].asnumpy() * 2)
        seen.extend(b.label[0].asnumpy().tolist())
    assert sorted(seen) == label.tolist()
    it.reset()
    assert len(list(it)) == 2
    it = mx.io.NDArrayIter(data, label, batch_size=4, last_batch_handle='roll_over')
    assert len(list(it)) == 2
    it.reset()
    assert len(list(it)) == 3


def test_csv_and_libsvm_iters(tmp_path):
    d, l = str(tmp_path / 'd.csv'), str(tmp_path / 'l.csv')
    x = np.random.rand(7, 6).astype('float32')
    y = np.arange(7, dtype='float32')
    np.savetxt(d, x, delimiter=',')
    np.savetxt(l, y, delimiter=',')
    it = mx.io.CSVIter(data_csv=d, data_shape=(2, 3), label_csv=l, batch_size=3)
    got = [b for b in it]
    assert len(got) == 3 and got[0].data[0].shape == (3, 2, 3)
    assert_almost_equal(got[0].data[0].asnumpy().reshape(3, 6), x[:3], rtol=1e-5)
    assert got[-1].pad == 2
    f = str(tmp_path / 'a.libsvm')
    open(f, 'w').write('1 0:1.5 3:2.0\n0 1:0.5\n1 2:3.0 4:1.0\n')
    it = mx.io.LibSVMIter(data_libsvm=f, data_shape=(5,), batch_size=3)
    b = next(iter(it))
    dense = b.data[0].tostype('default').asnumpy() if hasattr(b.data[0], 'tostype') else b.data[0].asnumpy()
    assert same(dense, np.array([[1.5, 0, 0, 2.0, 0], [0, 0.5, 0, 0, 0], [0, 0, 3.0, 0, 1.0]], 'float32'))
    assert same(b.label[0].asnumpy(), np.array([1, 0, 1], 'float32'))


def test_image_record_iter(tmp_path):
    rec, idx = str(tmp_path / 'img.rec'), str(tmp_path / 'img.idx')
    w = recordio.MXIndexedRecordIO(idx, rec, 'w')
    rng = np.random.RandomState(0)
    for i in range(12):
        img = (rng.rand(40, 48, 3) * 255).astype('uint8')
        w.write_idx(i, recordio.pack_img(recordio.IRHeader(0, float(i % 3), i, 0), img, img_fmt='.png'))
    w.close()
    it = mx.io.ImageRecordIter(path_imgrec=rec, path_imgidx=idx, data_shape=(3, 32, 32), batch_size=5, rand_crop=True,
                               rand_mirror=True, mean_r=127, mean_g=127, mean_b=127, preprocess_threads=2, shuffle=True)
    n, labels = 0, []
    for b in it:
        assert b.data[0].shape == (5, 3, 32, 32) and b.data[0].dtype == np.float32
        n += 5 - b.pad
        labels.extend(b.label[0].asnumpy()[:5 - b.pad].tolist())
    assert n == 12 and sorted(labels) == sorted([float(i % 3) for i in range(12)])
    it.reset()
    assert sum(5 - b.pad for b in it) == 12


def test_prefetching_and_resize_iter():
    data = np.arange(40, dtype='float32').reshape(20, 2)
    base = mx.io.NDArrayIter(data, np.zeros(20), batch_size=4)
    it = mx.io.PrefetchingIter(base)
    assert sum(1 for _ in it) == 5
    it.reset()
    assert sum(1 for _ in it) == 5
    rs = mx.io.ResizeIter(mx.io.NDArrayIter(data, np.zeros(20), batch_size=4), 8)
    assert sum(1 for _ in rs) == 8


def test_gluon_dataset_dataloader():
    x, y = np.arange(30, dtype='float32').reshape(10, 3), np.arange(10)
    ds = gluon.data.ArrayDataset(x, y)
    assert len(ds) == 10 and same(ds[3][0], x[3])
    dl = gluon.data.DataLoader(ds, batch_size=4, shuffle=False, last_batch='keep')
    shapes = [b[0].shape for b in dl]
    assert shapes == [(4, 3), (4, 3), (2, 3)]
    dl = gluon.data.DataLoader(ds.transform_first(lambda a: a * 2), batch_size=5, num_workers=2)
    total = sum(float(b[0].sum().asscalar()) for b in dl)
    assert total == float(x.sum() * 2)
    sampler = gluon.data.BatchSampler(gluon.data.RandomSampler(10), 3, 'discard')
    assert len(list(sampler)) == 3
    f = gluon.data.SimpleDataset(list(range(10))).filter(lambda v: v % 2 == 0).take(3)
    assert list(f) == [0, 2, 4]


def test_image_module_ops():
    img = (np.random.rand(30, 40, 3) * 255).astype('uint8')
    a = nd.array(img, dtype='uint8')
    r = mx.image.imresize(a, 20, 10)
    assert r.shape == (10, 20, 3)
    c, rect = mx.image.center_crop(a, (16, 12))
    assert c.shape == (12, 16, 3) and rect == (12, 9, 16, 12)
    rs = mx.image.resize_short(a, 15)
    assert min(rs.shape[:2]) == 15
    n = mx.image.color_normalize(a.astype('float32'), nd.array([1., 2., 3.]), nd.array([2., 2., 2.]))
    assert_almost_equal(n.asnumpy(), (img.astype('float32') - [1, 2, 3]) / 2, rtol=1e-5)
    augs = mx.image.CreateAugmenter(data_shape=(3, 24, 24), rand_crop=True, rand_mirror=True, brightness=0.1, mean=True,
                                    std=True)
    out = a.astype('float32')
    for aug in augs:
        out = aug(out)
    assert out.shape == (24, 24, 3)
    t = gluon.data.vision.transforms.Compose([gluon.data.vision.transforms.Resize(16),
                                              gluon.data.vision.transforms.ToTensor(),
                                              gluon.data.vision.transforms.Normalize(0.5, 0.25)])
    o = t(a)
    assert o.shape == (3, 16, 16) and o.dtype == np.float32


def test_image_record_iter_random_resized_crop(tmp_path):
    """``random_resized_crop`` (image_aug_default.cc): every sample is a rectangle of random area and aspect ratio resampled to
    ``data_shape``; shapes, label order and value range are checked, and two epochs differ (the crops are random)."""
    import io as _io
    from PIL import Image
    import mxnet_b200 as mx
    from mxnet_b200 import recordio
    rng = np.random.RandomState(0)
    path = str(tmp_path / 'rrc.rec')
    w = recordio.MXRecordIO(path, 'w')
    for i in range(6):
        img = (rng.rand(40 + i, 60, 3) * 255).astype('uint8')
        b = _io.BytesIO()
        Image.fromarray(img).save(b, format='PNG')
        w.write(recordio.pack(recordio.IRHeader(0, float(i), i, 0), b.getvalue()))
    w.close()
    it = mx.io.ImageRecordIter(path_imgrec=path, data_shape=(3, 24, 32), batch_size=3, random_resized_crop=True, rand_mirror=True,
                               min_random_area=0.3, max_random_area=1.0)
    first = [b.data[0].asnumpy().copy() for b in it]
    it.reset()
    second = [b.data[0].asnumpy().copy() for b in it]
    assert len(first) == 2 and first[0].shape == (3, 3, 24, 32)
    assert 0 <= first[0].min() and first[0].max() <= 255
    assert any(not np.array_equal(a, b) for a, b in zip(first, second))

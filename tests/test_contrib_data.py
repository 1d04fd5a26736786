"""gluon.contrib.data.vision: box arithmetic, box-aware transforms and the one-call loaders."""
import io
import os
import random

import numpy as np
import pytest

import mxnet_b200 as mx
from mxnet_b200 import nd, recordio
from mxnet_b200.gluon.contrib.data.vision import (ImageBboxDataLoader, ImageDataLoader, BboxLabelTransform, create_bbox_augment,
                                                 create_image_augment)
from mxnet_b200.gluon.contrib.data.vision.transforms import bbox as B


def test_box_arithmetic():
    boxes = np.array([[10., 10., 30., 40., 1.], [50., 20., 80., 60., 2.], [0., 0., 5., 5., 3.]])
    cropped = B.bbox_crop(boxes, (5, 5, 50, 50), allow_outside_center=False)
    np.testing.assert_allclose(cropped, [[5, 5, 25, 35, 1]])                      # box 2: centre outside, box 3: emptied
    kept = B.bbox_crop(boxes, (5, 5, 50, 50), allow_outside_center=True)
    assert kept.shape[0] == 2 and kept[1, 4] == 2
    np.testing.assert_allclose(B.bbox_flip(boxes, (100, 80), flip_x=True)[0, :4], [70, 10, 90, 40])
    np.testing.assert_allclose(B.bbox_flip(boxes, (100, 80), flip_y=True)[0, :4], [10, 40, 30, 70])
    np.testing.assert_allclose(B.bbox_resize(boxes, (100, 80), (50, 160))[0, :4], [5, 20, 15, 80])
    np.testing.assert_allclose(B.bbox_translate(boxes, 3, -2)[0, :4], [13, 8, 33, 38])
    iou = B.bbox_iou(boxes[:, :4], np.array([[10., 10., 30., 40.], [20., 10., 40., 40.]]))
    np.testing.assert_allclose(iou[0], [1.0, 1 / 3], rtol=1e-6)
    assert B.bbox_xywh_to_xyxy((10, 20, 5, 6)) == (10, 20, 14, 25) and B.bbox_xyxy_to_xywh((10, 20, 14, 25)) == (10, 20, 5, 6)
    np.testing.assert_allclose(B.bbox_xyxy_to_xywh(B.bbox_xywh_to_xyxy(np.array([[1., 2., 3., 4.]]))), [[1, 2, 3, 4]])
    np.testing.assert_allclose(B.bbox_clip_xyxy(np.array([[-5., 3., 120., 90.]]), 100, 80), [[0, 3, 99, 79]])
    random.seed(0)
    new, crop = B.bbox_random_crop_with_constraints(boxes, (100, 80))
    x, y, w, h = crop
    assert 0 <= x and 0 <= y and x + w <= 100 and y + h <= 80 and len(new) >= 1
    assert (new[:, :2] >= 0).all() and (new[:, 2] <= w).all() and (new[:, 3] <= h).all()


def test_box_transforms_move_image_and_boxes_together():
    img = nd.array(np.arange(40 * 60 * 3).reshape(40, 60, 3) % 255, dtype='uint8')
    boxes = nd.array([[10., 5., 30., 25., 0.], [40., 10., 55., 35., 1.]])
    fi, fb = B.ImageBboxRandomFlipLeftRight(p=1.0)(img, boxes)
    np.testing.assert_array_equal(fi.asnumpy(), img.asnumpy()[:, ::-1])
    np.testing.assert_allclose(fb.asnumpy()[0, :4], [30, 5, 50, 25])
    ci, cb = B.ImageBboxCrop((5, 0, 40, 30))(img, boxes)
    assert ci.shape == (30, 40, 3) and cb.shape == (1, 5)
    np.testing.assert_allclose(cb.asnumpy()[0, :4], [5, 5, 25, 25])
    ri, rb = B.ImageBboxResize(120, 20)(img, boxes)
    assert ri.shape == (20, 120, 3)
    np.testing.assert_allclose(rb.asnumpy()[0, :4], [20, 2.5, 60, 12.5])
    random.seed(1)
    ei, eb = B.ImageBboxRandomExpand(p=1.0, max_ratio=3, fill=(1, 2, 3))(img, boxes)
    dx, dy = eb.asnumpy()[0, 0] - 10, eb.asnumpy()[0, 1] - 5
    assert ei.shape[0] >= 40 and ei.shape[1] >= 60
    np.testing.assert_array_equal(ei.asnumpy()[int(dy):int(dy) + 40, int(dx):int(dx) + 60], img.asnumpy())
    ki, kb = B.ImageBboxRandomCropWithConstraints(p=1.0)(img, boxes)
    assert ki.shape[2] == 3 and kb.shape[1] == 5 and kb.shape[0] >= 1


def _write_rec(tmp_path, detection):
    from PIL import Image
    rec, idx = str(tmp_path / 'd.rec'), str(tmp_path / 'd.idx')
    w = recordio.MXIndexedRecordIO(idx, rec, 'w')
    rng = np.random.RandomState(0)
    for i in range(6):
        arr = rng.randint(0, 255, (32 + 4 * i, 48, 3)).astype('uint8')
        buf = io.BytesIO()
        Image.fromarray(arr).save(buf, format='PNG')
        if detection:
            label = [2, 5] + [i % 3, 0.1, 0.2, 0.6, 0.8] + ([1, 0.5, 0.5, 0.9, 0.9] if i % 2 else [])
        else:
            label = float(i % 3)
        w.write_idx(i, recordio.pack(recordio.IRHeader(0, label, i, 0), buf.getvalue()))
    w.close()
    return rec


def test_image_data_loader_from_record_file(tmp_path):
    rec = _write_rec(tmp_path, detection=False)
    loader = ImageDataLoader(4, (3, 24, 24), path_imgrec=rec, rand_crop=True, rand_mirror=True, mean=True, std=True, brightness=0.1)
    batches = list(loader)
    assert len(loader) == 2 and batches[0][0].shape == (4, 3, 24, 24) and batches[0][1].shape == (4,)
    assert batches[0][0].dtype == np.float32 and abs(float(batches[0][0].mean().asscalar())) < 3.0
    aug = create_image_augment((3, 16, 16), resize=20)
    out = aug(nd.array(np.zeros((30, 40, 3)), dtype='uint8'))
    assert out.shape == (3, 16, 16)


def test_image_bbox_data_loader_pads_labels(tmp_path):
    rec = _write_rec(tmp_path, detection=True)
    loader = ImageBboxDataLoader(3, (3, 32, 32), path_imgrec=rec, rand_mirror=True, rand_crop=0.5, rand_pad=0.5, mean=True)
    data, label = next(iter(loader))
    assert data.shape == (3, 3, 32, 32) and label.shape[0] == 3 and label.shape[2] == 5
    lab = label.asnumpy()
    valid = lab[lab[:, :, 4] >= 0]
    assert len(valid) >= 3 and (valid[:, :4] >= -1e-3).all() and (valid[:, :4] <= 32 + 1e-3).all()
    img, boxes = BboxLabelTransform(coord_normalized=True)(np.zeros((50, 100, 3)), np.array([2, 5, 7, 0.1, 0.2, 0.6, 0.8]))
    np.testing.assert_allclose(boxes, [[10, 10, 60, 40, 7]])
    pair = create_bbox_augment((3, 20, 20))(nd.array(np.zeros((40, 60, 3)), dtype='uint8'), boxes)
    assert pair[0].shape == (3, 20, 20)
    np.testing.assert_allclose(np.asarray(pair[1]), [[10 / 3, 5, 20, 20, 7]], rtol=1e-5)

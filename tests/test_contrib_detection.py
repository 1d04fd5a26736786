"""Region-proposal, position-sensitive pooling, deformable convolution and mask-target operators (CPU)."""
import numpy as np
import pytest

import mxnet_b200 as mx
from mxnet_b200 import autograd, nd


def _iou_plus1(a, b):
    x1, y1, x2, y2 = max(a[0], b[0]), max(a[1], b[1]), min(a[2], b[2]), min(a[3], b[3])
    inter = max(0.0, x2 - x1 + 1) * max(0.0, y2 - y1 + 1)
    area = lambda r: (r[2] - r[0] + 1) * (r[3] - r[1] + 1)
    return inter / (area(a) + area(b) - inter)


def test_proposal_outputs_clipped_sorted_and_suppressed():
    rng = np.random.RandomState(0)
    A = 12
    cls = nd.array(rng.rand(2, 2 * A, 6, 8).astype('float32'))
    box = nd.array((rng.randn(2, 4 * A, 6, 8) * 0.2).astype('float32'))
    info = nd.array([[96, 128, 1.0], [80, 100, 1.0]])
    rois, scores = nd.contrib.MultiProposal(cls, box, info, rpn_pre_nms_top_n=300, rpn_post_nms_top_n=16, threshold=0.5,
                                            rpn_min_size=8, output_score=True)
    rois, scores = rois.asnumpy(), scores.asnumpy()[:, 0]
    assert rois.shape == (32, 5) and (rois[:16, 0] == 0).all() and (rois[16:, 0] == 1).all()
    for b, (h, w) in enumerate(((96, 128), (80, 100))):
        r, s = rois[b * 16:(b + 1) * 16, 1:], scores[b * 16:(b + 1) * 16]
        assert (r[:, 0] >= 0).all() and (r[:, 2] <= w - 1).all() and (r[:, 1] >= 0).all() and (r[:, 3] <= h - 1).all()
        assert (np.diff(s) <= 1e-6).all()                    # descending scores
        for i in range(16):
            for j in range(i + 1, 16):
                assert _iou_plus1(r[i], r[j]) <= 0.5 + 1e-5
    single = nd.contrib.Proposal(cls[0:1], box[0:1], info[0:1], rpn_pre_nms_top_n=300, rpn_post_nms_top_n=16, threshold=0.5,
                                 rpn_min_size=8).asnumpy()
    np.testing.assert_allclose(single, rois[:16])


def test_proposal_pads_by_cycling_kept_boxes():
    # one anchor, identical scores everywhere and zero deltas: heavy suppression leaves fewer boxes than requested
    cls = nd.array(np.concatenate([np.zeros((1, 1, 2, 2)), np.full((1, 1, 2, 2), 0.9)], 1).astype('float32'))
    box = nd.zeros((1, 4, 2, 2))
    rois = nd.contrib.Proposal(cls, box, nd.array([[32, 32, 1.0]]), rpn_post_nms_top_n=6, threshold=0.1, rpn_min_size=1,
                               scales=(8.0,), ratios=(1.0,), feature_stride=16).asnumpy()
    assert rois.shape == (6, 5)
    uniq = np.unique(rois, axis=0)
    assert len(uniq) < 6
    np.testing.assert_allclose(rois[len(uniq):], np.concatenate([rois[:len(uniq)]] * 6)[:6 - len(uniq)])


def test_psroi_pooling_matches_direct_evaluation():
    rng = np.random.RandomState(1)
    D, G, P = 2, 3, 3
    data = rng.randn(2, D * G * G, 12, 10).astype('float32')
    rois = np.array([[0, 1, 2, 7, 9], [1, 0, 0, 9, 11], [1, 3.4, 2.6, 5.2, 4.9]], dtype='float32')
    out = nd.contrib.PSROIPooling(nd.array(data), nd.array(rois), spatial_scale=0.5, output_dim=D, pooled_size=P,
                                  group_size=G).asnumpy()
    ref = np.zeros_like(out)
    for n, r in enumerate(rois):
        b = int(r[0])
        x1, y1 = np.round(r[1]) * 0.5, np.round(r[2]) * 0.5
        x2, y2 = (np.round(r[3]) + 1) * 0.5, (np.round(r[4]) + 1) * 0.5
        bw, bh = max(x2 - x1, 0.1) / P, max(y2 - y1, 0.1) / P
        for c in range(D):
            for ph in range(P):
                for pw in range(P):
                    hs, he = int(np.floor(ph * bh + y1)), int(np.ceil((ph + 1) * bh + y1))
                    ws, we = int(np.floor(pw * bw + x1)), int(np.ceil((pw + 1) * bw + x1))
                    hs, he, ws, we = max(hs, 0), min(he, 12), max(ws, 0), min(we, 10)
                    if he > hs and we > ws:
                        ref[n, c, ph, pw] = data[b, (c * G + ph) * G + pw, hs:he, ws:we].mean()
    np.testing.assert_allclose(out, ref, rtol=1e-5, atol=1e-6)


def test_deformable_psroi_pooling_without_offsets_is_sampled_psroi():
    rng = np.random.RandomState(2)
    data = nd.array(rng.randn(1, 2 * 2 * 2, 8, 8).astype('float32'))
    rois = nd.array([[0, 0, 0, 7, 7]])
    a = nd.contrib.DeformablePSROIPooling(data, rois, spatial_scale=1.0, output_dim=2, group_size=2, pooled_size=2,
                                          sample_per_part=4, no_trans=True).asnumpy()
    zero = nd.zeros((1, 2, 2, 2))
    b = nd.contrib.DeformablePSROIPooling(data, rois, zero, spatial_scale=1.0, output_dim=2, group_size=2, pooled_size=2,
                                          part_size=2, sample_per_part=4, trans_std=0.1).asnumpy()
    np.testing.assert_allclose(a, b, rtol=1e-6)
    shifted = nd.contrib.DeformablePSROIPooling(data, rois, nd.ones((1, 2, 2, 2)), spatial_scale=1.0, output_dim=2, group_size=2,
                                                pooled_size=2, part_size=2, sample_per_part=4, trans_std=0.1).asnumpy()
    assert np.abs(shifted - a).max() > 1e-3


def test_deformable_convolution_zero_offsets_equals_convolution_and_has_gradients():
    rng = np.random.RandomState(3)
    x = nd.array(rng.randn(2, 4, 7, 7).astype('float32'))
    w = nd.array(rng.randn(6, 4, 3, 3).astype('float32'))
    off = nd.zeros((2, 18, 7, 7))
    for t in (x, w, off):
        t.attach_grad()
    with autograd.record():
        y = nd.contrib.DeformableConvolution(x, off, w, kernel=(3, 3), pad=(1, 1), num_filter=6, no_bias=True)
        (y * y).sum().backward()
    ref = nd.Convolution(x, w, kernel=(3, 3), pad=(1, 1), num_filter=6, no_bias=True)
    np.testing.assert_allclose(y.asnumpy(), ref.asnumpy(), rtol=1e-4, atol=1e-4)
    assert np.abs(off.grad.asnumpy()).max() > 0 and np.abs(w.grad.asnumpy()).max() > 0
    m = nd.contrib.ModulatedDeformableConvolution(x, off, nd.ones((2, 9, 7, 7)) * 0.25, w, kernel=(3, 3), pad=(1, 1),
                                                  num_filter=6, no_bias=True)
    np.testing.assert_allclose(m.asnumpy(), 0.25 * ref.asnumpy(), rtol=1e-4, atol=1e-4)


def test_mrcnn_mask_target_shapes_and_class_weights():
    rng = np.random.RandomState(4)
    masks = np.zeros((1, 2, 16, 16), dtype='float32')
    masks[0, 0, :8] = 1.0            # upper half
    masks[0, 1] = 1.0
    rois = nd.array([[[0, 0, 15, 15], [0, 0, 15, 7], [4, 4, 11, 11]]])
    t, w = nd.contrib.mrcnn_mask_target(rois, nd.array(masks), nd.array([[0, 0, 1]]), nd.array([[2, 0, 1]]), num_rois=3,
                                        num_classes=3, mask_size=(4, 4))
    t, w = t.asnumpy(), w.asnumpy()
    assert t.shape == (1, 3, 3, 4, 4) and w.shape == t.shape
    np.testing.assert_allclose(t[0, 0, 0, :2], 1.0, atol=1e-5)      # rows inside the upper half
    np.testing.assert_allclose(t[0, 0, 0, 3], 0.0, atol=1e-5)
    np.testing.assert_allclose(t[0, 1], 1.0, atol=1e-5)
    np.testing.assert_allclose(t[0, 2], 1.0, atol=1e-5)
    np.testing.assert_array_equal(w[0, :, :, 0, 0], [[0, 0, 1], [1, 0, 0], [0, 1, 0]])


# ---------------------------------------------------------------------------------------- ROIAlign, box_nms
def _roi_align_scalar(data, rois, pooled, scale, sample_ratio, position_sensitive, aligned):
    """Loop restatement of the operator's rules (roi_align.cc): samples more than one pixel outside the map are zero,
    samples in the border are clamped to the edge, bins average sample_ratio^2 (or ceil(roi/bin)^2) samples."""
    N, CI, H, W = data.shape
    ph, pw = pooled
    C = CI // (ph * pw) if position_sensitive else CI
    out = np.zeros((len(rois), C, ph, pw), dtype=np.float64)

    def sample(plane, y, x):
        if y < -1.0 or y > H or x < -1.0 or x > W:
            return 0.0
        y, x = max(y, 0.0), max(x, 0.0)
        y0, x0 = int(y), int(x)
        if y0 >= H - 1:
            y1 = y0 = H - 1
            y = float(y0)
        else:
            y1 = y0 + 1
        if x0 >= W - 1:
            x1 = x0 = W - 1
            x = float(x0)
        else:
            x1 = x0 + 1
        ly, lx = y - y0, x - x0
        return ((1 - ly) * (1 - lx) * plane[y0, x0] + (1 - ly) * lx * plane[y0, x1] + ly * (1 - lx) * plane[y1, x0] +
                ly * lx * plane[y1, x1])
    off = 0.5 if aligned else 0.0
    for r, roi in enumerate(rois):
        b = int(roi[0])
        if b < 0:
            continue
        x1, y1, x2, y2 = [v * scale - off for v in roi[1:]]
        rw, rh = x2 - x1, y2 - y1
        if not aligned:
            rw, rh = max(rw, 1.0), max(rh, 1.0)
        gh = sample_ratio if sample_ratio > 0 else max(int(np.ceil(rh / ph)), 1)
        gw = sample_ratio if sample_ratio > 0 else max(int(np.ceil(rw / pw)), 1)
        for c in range(C):
            for i in range(ph):
                for j in range(pw):
                    ci = (c * ph + i) * pw + j if position_sensitive else c
                    acc = 0.0
                    for iy in range(gh):
                        for ix in range(gw):
                            acc += sample(data[b, ci], y1 + i * rh / ph + (iy + 0.5) * rh / ph / gh,
                                          x1 + j * rw / pw + (ix + 0.5) * rw / pw / gw)
                    out[r, c, i, j] = acc / (gh * gw)
    return out


_ROI_CASES = [dict(pooled=(2, 2), scale=1.0, sample_ratio=2, position_sensitive=False, aligned=False),
              dict(pooled=(3, 2), scale=0.5, sample_ratio=-1, position_sensitive=False, aligned=True),
              dict(pooled=(2, 2), scale=1.0, sample_ratio=2, position_sensitive=True, aligned=False)]
_ROIS = np.array([[0, 1.0, 1.5, 6.0, 7.0], [1, -3.0, -2.0, 4.0, 5.0], [0, 5.0, 5.0, 12.0, 11.0], [-1, 0, 0, 4, 4],
                  [1, 2.2, 3.1, 2.4, 3.3]], dtype='float32')


@pytest.mark.parametrize('case', _ROI_CASES)
def test_roi_align_follows_the_boundary_rules(case):
    rng = np.random.RandomState(0)
    data = rng.randn(2, 8, 9, 10).astype('float32')
    out = mx.nd.contrib.ROIAlign(mx.nd.array(data), mx.nd.array(_ROIS), pooled_size=case['pooled'], spatial_scale=case['scale'],
                                 sample_ratio=case['sample_ratio'], position_sensitive=case['position_sensitive'],
                                 aligned=case['aligned'])
    ref = _roi_align_scalar(data, _ROIS, **case)
    assert out.shape == ref.shape
    np.testing.assert_allclose(out.asnumpy(), ref, rtol=1e-4, atol=1e-5)


def _nms_input(rng, n, classes=3):
    xy = rng.uniform(0, 50, (n, 2))
    wh = rng.uniform(5, 25, (n, 2))
    return np.concatenate([rng.randint(0, classes, (n, 1)).astype('float64'), rng.uniform(0, 1, (n, 1)), xy, xy + wh],
                          1).astype('float32')


def _nms_scalar(rows, thresh, valid, topk, force):
    order = [i for i in np.argsort(-rows[:, 1], kind='stable') if rows[i, 1] > valid]
    if topk > 0:
        order = order[:topk]
    kept = []
    for i in order:
        ok = True
        for k in kept:
            if not force and rows[k, 0] != rows[i, 0]:
                continue
            a, b = rows[k, 2:6], rows[i, 2:6]
            w, h = max(min(a[2], b[2]) - max(a[0], b[0]), 0), max(min(a[3], b[3]) - max(a[1], b[1]), 0)
            inter = w * h
            if inter / ((a[2] - a[0]) * (a[3] - a[1]) + (b[2] - b[0]) * (b[3] - b[1]) - inter) > thresh:
                ok = False
                break
        if ok:
            kept.append(i)
    out = np.full_like(rows, -1.0)
    out[:len(kept)] = rows[kept]
    return out


@pytest.mark.parametrize('force,topk', [(False, -1), (True, -1), (False, 20)])
def test_box_nms_keeps_the_greedy_selection(force, topk):
    rows = _nms_input(np.random.RandomState(2), 60)
    out = mx.nd.contrib.box_nms(mx.nd.array(rows[None]), overlap_thresh=0.4, valid_thresh=0.1, topk=topk, coord_start=2,
                                score_index=1, id_index=0, force_suppress=force)
    np.testing.assert_allclose(out.asnumpy()[0], _nms_scalar(rows, 0.4, 0.1, topk, force), rtol=1e-6)


def test_rotated_roi_align_reduces_to_roi_align_at_zero_angle_and_rotates_by_ninety_degrees():
    rng = np.random.RandomState(4)
    data = rng.randn(1, 3, 12, 12).astype('float32')
    # an axis-aligned box given by corners and the same box given by centre / size / angle 0
    corner = np.array([[0, 2.0, 3.0, 8.0, 9.0]], dtype='float32')
    rotated = np.array([[0, 5.0, 6.0, 6.0, 6.0, 0.0]], dtype='float32')
    a = mx.nd.contrib.ROIAlign(mx.nd.array(data), mx.nd.array(corner), pooled_size=(3, 3), spatial_scale=1.0, sample_ratio=2).asnumpy()
    b = mx.nd.contrib.RROIAlign(mx.nd.array(data), mx.nd.array(rotated), pooled_size=(3, 3), spatial_scale=1.0, sampling_ratio=2).asnumpy()
    np.testing.assert_allclose(b, a, rtol=1e-5, atol=1e-6)
    # a quarter turn of the sampling grid equals sampling the map turned the other way
    turned = np.array([[0, 5.5, 5.5, 6.0, 6.0, 90.0]], dtype='float32')
    straight = np.array([[0, 5.5, 5.5, 6.0, 6.0, 0.0]], dtype='float32')
    c = mx.nd.contrib.RROIAlign(mx.nd.array(data), mx.nd.array(turned), pooled_size=(2, 2), sampling_ratio=2).asnumpy()
    d = mx.nd.contrib.RROIAlign(mx.nd.array(np.rot90(data, k=-1, axes=(2, 3)).copy()), mx.nd.array(straight), pooled_size=(2, 2),
                                sampling_ratio=2).asnumpy()
    np.testing.assert_allclose(c, d, rtol=1e-4, atol=1e-5)

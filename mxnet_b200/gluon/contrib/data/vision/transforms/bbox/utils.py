"""Bounding-box arithmetic on NumPy arrays of shape (N, 4+): columns 0..3 are x_min, y_min, x_max, y_max, further
columns (class, difficulty ...) ride along unchanged (``gluon/contrib/data/vision/transforms/bbox/utils.py``)."""
import random

import numpy as np

__all__ = ['bbox_crop', 'bbox_flip', 'bbox_resize', 'bbox_translate', 'bbox_iou', 'bbox_xywh_to_xyxy', 'bbox_xyxy_to_xywh',
           'bbox_clip_xyxy', 'bbox_random_crop_with_constraints']


def _check(bbox):
    if bbox.ndim != 2 or bbox.shape[1] < 4:
        raise ValueError('Bounding boxes must have shape (N, 4+), got %s' % (bbox.shape,))


def bbox_crop(bbox, crop_box=None, allow_outside_center=True):
    """Boxes expressed in the coordinates of the crop (x, y, width, height), clipped to it; boxes that end up empty are
    dropped, and with ``allow_outside_center=False`` also boxes whose centre lies outside the crop."""
    bbox = bbox.copy()
    if crop_box is None:
        return bbox
    if len(crop_box) != 4:
        raise ValueError('Invalid crop_box parameter, requires length 4, given %s' % (crop_box,))
    if all(c is None for c in crop_box):
        return bbox
    left, top = crop_box[0] or 0, crop_box[1] or 0
    right = left + (crop_box[2] if crop_box[2] else np.inf)
    bottom = top + (crop_box[3] if crop_box[3] else np.inf)
    lo, hi = np.array((left, top)), np.array((right, bottom))
    keep = np.ones(bbox.shape[0], dtype=bool)
    if not allow_outside_center:
        centre = (bbox[:, :2] + bbox[:, 2:4]) / 2
        keep = ((lo <= centre) & (centre < hi)).all(axis=1)
    bbox[:, :2] = np.maximum(bbox[:, :2], lo) - lo
    bbox[:, 2:4] = np.minimum(bbox[:, 2:4], hi) - lo
    keep &= (bbox[:, :2] < bbox[:, 2:4]).all(axis=1)
    return bbox[keep]


def bbox_flip(bbox, size, flip_x=False, flip_y=False):
    """Mirror boxes inside an image of ``size`` (width, height)."""
    if len(size) != 2:
        raise ValueError('size requires length 2 tuple, given %d' % len(size))
    width, height = size
    bbox = bbox.copy()
    if flip_y:
        bbox[:, 1], bbox[:, 3] = height - bbox[:, 3], height - bbox[:, 1].copy()
    if flip_x:
        bbox[:, 0], bbox[:, 2] = width - bbox[:, 2], width - bbox[:, 0].copy()
    return bbox


def bbox_resize(bbox, in_size, out_size):
    """Scale boxes from an image of ``in_size`` (width, height) to ``out_size``."""
    if len(in_size) != 2 or len(out_size) != 2:
        raise ValueError('in_size and out_size require length 2 tuples')
    bbox = bbox.copy().astype(float)
    sx, sy = out_size[0] / in_size[0], out_size[1] / in_size[1]
    bbox[:, [0, 2]] *= sx
    bbox[:, [1, 3]] *= sy
    return bbox


def bbox_translate(bbox, x_offset=0, y_offset=0):
    bbox = bbox.copy()
    bbox[:, [0, 2]] += x_offset
    bbox[:, [1, 3]] += y_offset
    return bbox


def bbox_iou(bbox_a, bbox_b, offset=0):
    """Intersection over union of every box of ``bbox_a`` (N, 4) with every box of ``bbox_b`` (M, 4); ``offset=1`` for
    inclusive pixel coordinates."""
    if bbox_a.shape[1] < 4 or bbox_b.shape[1] < 4:
        raise IndexError('Bounding boxes axis 1 must have at least length 4')
    tl = np.maximum(bbox_a[:, None, :2], bbox_b[:, :2])
    br = np.minimum(bbox_a[:, None, 2:4], bbox_b[:, 2:4])
    inter = np.prod(br - tl + offset, axis=2) * (tl < br).all(axis=2)
    area_a = np.prod(bbox_a[:, 2:4] - bbox_a[:, :2] + offset, axis=1)
    area_b = np.prod(bbox_b[:, 2:4] - bbox_b[:, :2] + offset, axis=1)
    return inter / (area_a[:, None] + area_b - inter)


def bbox_xywh_to_xyxy(xywh):
    """(x, y, width, height) -> (x_min, y_min, x_max, y_max) with inclusive pixel coordinates (x_max = x + width - 1)."""
    if isinstance(xywh, (tuple, list)):
        if len(xywh) != 4:
            raise IndexError('Bounding boxes must have 4 elements, given %d' % len(xywh))
        w, h = max(xywh[2] - 1, 0), max(xywh[3] - 1, 0)
        return xywh[0], xywh[1], xywh[0] + w, xywh[1] + h
    if isinstance(xywh, np.ndarray):
        if xywh.size % 4:
            raise IndexError('Bounding boxes must have n * 4 elements, given %s' % (xywh.shape,))
        return np.hstack((xywh[:, :2], xywh[:, :2] + np.maximum(0, xywh[:, 2:4] - 1)))
    raise TypeError('Expect input xywh a list, tuple or numpy.ndarray, given %s' % type(xywh))


def bbox_xyxy_to_xywh(xyxy):
    if isinstance(xyxy, (tuple, list)):
        if len(xyxy) != 4:
            raise IndexError('Bounding boxes must have 4 elements, given %d' % len(xyxy))
        return xyxy[0], xyxy[1], xyxy[2] - xyxy[0] + 1, xyxy[3] - xyxy[1] + 1
    if isinstance(xyxy, np.ndarray):
        if xyxy.size % 4:
            raise IndexError('Bounding boxes must have n * 4 elements, given %s' % (xyxy.shape,))
        return np.hstack((xyxy[:, :2], xyxy[:, 2:4] - xyxy[:, :2] + 1))
    raise TypeError('Expect input xyxy a list, tuple or numpy.ndarray, given %s' % type(xyxy))


def bbox_clip_xyxy(xyxy, width, height):
    """Clip corner boxes to the image [0, width - 1] x [0, height - 1]."""
    if isinstance(xyxy, (tuple, list)):
        if len(xyxy) != 4:
            raise IndexError('Bounding boxes must have 4 elements, given %d' % len(xyxy))
        return (min(max(xyxy[0], 0), width - 1), min(max(xyxy[1], 0), height - 1),
                min(max(xyxy[2], 0), width - 1), min(max(xyxy[3], 0), height - 1))
    if isinstance(xyxy, np.ndarray):
        if xyxy.size % 4:
            raise IndexError('Bounding boxes must have n * 4 elements, given %s' % (xyxy.shape,))
        out = xyxy.copy()
        out[:, [0, 2]] = np.clip(out[:, [0, 2]], 0, width - 1)
        out[:, [1, 3]] = np.clip(out[:, [1, 3]], 0, height - 1)
        return out
    raise TypeError('Expect input xyxy a list, tuple or numpy.ndarray, given %s' % type(xyxy))


def bbox_random_crop_with_constraints(bbox, size, min_scale=0.3, max_scale=1, max_aspect_ratio=2, constraints=None, max_trial=50):
    """The random crop of the SSD paper: for every (min_iou, max_iou) constraint try up to ``max_trial`` crops of random
    scale and aspect ratio and keep the first whose overlap with every box satisfies the constraint; one of the kept
    candidates (the whole image is always one) is then drawn, skipping crops that would lose every box.
    Returns (boxes in crop coordinates, (x, y, width, height))."""
    if constraints is None:
        constraints = ((0.1, None), (0.3, None), (0.5, None), (0.7, None), (0.9, None), (None, 1))
    w, h = size
    candidates = [(0, 0, w, h)]
    for min_iou, max_iou in constraints:
        lo = -np.inf if min_iou is None else min_iou
        hi = np.inf if max_iou is None else max_iou
        for _ in range(max_trial):
            scale = random.uniform(min_scale, max_scale)
            ratio = random.uniform(max(1 / max_aspect_ratio, scale * scale), min(max_aspect_ratio, 1 / (scale * scale)))
            ch, cw = int(h * scale / np.sqrt(ratio)), int(w * scale * np.sqrt(ratio))
            if ch <= 0 or cw <= 0 or ch >= h or cw >= w:
                if ch == h and cw == w:
                    ct = cl = 0
                else:
                    continue
            else:
                ct, cl = random.randrange(h - ch), random.randrange(w - cw)
            if len(bbox) == 0:
                return bbox, (cl, ct, cw, ch)
            iou = bbox_iou(bbox, np.array([[cl, ct, cl + cw, ct + ch]], dtype=float))
            if lo <= iou.min() and iou.max() <= hi:
                candidates.append((cl, ct, cw, ch))
                break
    while candidates:
        crop = candidates.pop(random.randrange(len(candidates)))
        new_bbox = bbox_crop(bbox, crop, allow_outside_center=False)
        if new_bbox.size < 1:
            continue
        return new_bbox, crop
    return bbox, (0, 0, w, h)

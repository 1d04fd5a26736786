"""Blocks that transform an (image, boxes) pair (``gluon/contrib/data/vision/transforms/bbox/bbox.py``).  Images are
(H, W, C) arrays, boxes (N, 4+) arrays in corner format; both come back as arrays of the image's class."""
import random

import numpy as np

from mxnet_b200.ndarray.ndarray import NDArray
from mxnet_b200.gluon import block as _block
from mxnet_b200 import image as _image
from .utils import bbox_crop, bbox_flip, bbox_random_crop_with_constraints, bbox_resize, bbox_translate

__all__ = ['ImageBboxRandomFlipLeftRight', 'ImageBboxCrop', 'ImageBboxRandomCropWithConstraints', 'ImageBboxRandomExpand',
           'ImageBboxResize']


def _np(x):
    return x.asnumpy() if isinstance(x, NDArray) else np.asarray(x)


def _like(arr, ref, dtype=None):
    """A framework array of the class of ``ref`` (legacy or NumPy-semantics) holding ``arr``."""
    if not isinstance(ref, NDArray):
        return arr
    from mxnet_b200 import nd
    out = nd.array(arr, dtype=dtype or arr.dtype)
    return out.as_np_ndarray() if type(ref).__name__ == 'ndarray' else out


class ImageBboxRandomFlipLeftRight(_block.Block):
    """Mirror image and boxes horizontally with probability ``p``."""

    def __init__(self, p=0.5):
        super().__init__()
        self.p = p

    def forward(self, img, bbox):
        if self.p <= 0 or (self.p < 1 and random.random() >= self.p):
            return img, bbox
        im = _np(img)
        width = im.shape[-2]
        return _like(np.ascontiguousarray(im[..., ::-1, :]), img), _like(bbox_flip(_np(bbox), (width, im.shape[-3]), flip_x=True), bbox)


class ImageBboxCrop(_block.Block):
    """Crop (x, y, width, height) of the image; boxes are clipped to it and emptied boxes dropped."""

    def __init__(self, crop, allow_outside_center=False):
        super().__init__()
        if len(crop) != 4:
            raise ValueError('expected crop as (x, y, width, height), got %s' % (crop,))
        self._crop, self._allow = tuple(crop), allow_outside_center

    def forward(self, img, bbox):
        x, y, w, h = self._crop
        im = _np(img)
        if x + w > im.shape[-2] or y + h > im.shape[-3]:
            return img, bbox                      # the crop does not fit: leave the pair unchanged
        new_bbox = bbox_crop(_np(bbox), self._crop, self._allow)
        return _like(np.ascontiguousarray(im[..., y:y + h, x:x + w, :]), img), _like(new_bbox, bbox)


class ImageBboxRandomCropWithConstraints(_block.Block):
    """The overlap-constrained random crop used to train SSD-style detectors, applied with probability ``p``."""

    def __init__(self, p=0.5, min_scale=0.3, max_scale=1, max_aspect_ratio=2, constraints=None, max_trial=50):
        super().__init__()
        self.p = p
        self._args = dict(min_scale=min_scale, max_scale=max_scale, max_aspect_ratio=max_aspect_ratio, constraints=constraints,
                          max_trial=max_trial)

    def forward(self, img, bbox):
        if random.random() > self.p:
            return img, bbox
        im = _np(img)
        new_bbox, (x, y, w, h) = bbox_random_crop_with_constraints(_np(bbox), (im.shape[-2], im.shape[-3]), **self._args)
        return _like(np.ascontiguousarray(im[..., y:y + h, x:x + w, :]), img), _like(new_bbox, bbox)


class ImageBboxRandomExpand(_block.Block):
    """Place the image at a random position on a larger canvas (up to ``max_ratio`` times each side) filled with ``fill``;
    boxes move with it.  Makes small objects out of large ones."""

    def __init__(self, p=0.5, max_ratio=4, fill=0, keep_ratio=True):
        super().__init__()
        self.p, self._max_ratio, self._fill, self._keep_ratio = p, max_ratio, fill, keep_ratio

    def forward(self, img, bbox):
        if self._max_ratio <= 1 or random.random() > self.p:
            return img, bbox
        im = _np(img)
        if im.ndim != 3:
            raise NotImplementedError('ImageBboxRandomExpand expects (H, W, C) images')
        h, w, c = im.shape
        rx = random.uniform(1, self._max_ratio)
        ry = rx if self._keep_ratio else random.uniform(1, self._max_ratio)
        oh, ow = int(h * ry), int(w * rx)
        off_y, off_x = random.randint(0, oh - h), random.randint(0, ow - w)
        canvas = np.empty((oh, ow, c), dtype=im.dtype)
        canvas[...] = np.asarray(self._fill, dtype=im.dtype)
        canvas[off_y:off_y + h, off_x:off_x + w] = im
        return _like(canvas, img), _like(bbox_translate(_np(bbox), off_x, off_y), bbox)


class ImageBboxResize(_block.Block):
    """Resize the image to ``width`` x ``height`` and scale the boxes accordingly."""

    def __init__(self, width, height, interp=1):
        super().__init__()
        self._size, self._interp = (width, height), interp

    def forward(self, img, bbox):
        im = _np(img)
        from mxnet_b200 import nd
        interp = self._interp if self._interp != 10 else random.randint(0, 4)
        resized = _image.imresize(nd.array(im, dtype=im.dtype), self._size[0], self._size[1], interp=interp).asnumpy()
        return _like(resized, img), _like(bbox_resize(_np(bbox), (im.shape[-2], im.shape[-3]), self._size), bbox)

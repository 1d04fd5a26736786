"""Image loading, geometric and colour helpers, the ``Augmenter`` family and ``ImageIter`` (API of
``python/mxnet/image/image.py``).

Images are HxWxC arrays (uint8 after decoding, float32 after ``CastAug``); sizes are given as ``(width, height)`` the way
the reference does.  Decoding goes through Pillow, resizing and border padding through the ``_cvimresize`` /
``_cvcopyMakeBorder`` operators.  Randomness comes from Python's ``random`` module (and NumPy's for the PCA noise), so
``mx.random.seed`` makes augmentation repeatable.
"""
import io
import json
import logging
import os
import random

import numpy as np

from ..ndarray.ndarray import NDArray
from ..ops import registry as _reg

__all__ = ['imread', 'imdecode', 'imresize', 'scale_down', 'copyMakeBorder', 'resize_short', 'fixed_crop',
           'random_crop', 'center_crop', 'color_normalize', 'random_size_crop', 'Augmenter', 'SequentialAug',
           'ResizeAug', 'ForceResizeAug', 'RandomCropAug', 'RandomSizedCropAug', 'CenterCropAug', 'RandomOrderAug',
           'BrightnessJitterAug', 'ContrastJitterAug', 'SaturationJitterAug', 'HueJitterAug', 'ColorJitterAug',
           'LightingAug', 'ColorNormalizeAug', 'RandomGrayAug', 'HorizontalFlipAug', 'CastAug', 'CreateAugmenter',
           'ImageIter']

# ITU-R 601 luma weights (RGB order), used by the contrast / saturation jitters
_LUMA = (0.299, 0.587, 0.114)


# ---- decoding ---------------------------------------------------------------------------------------------------------
def _decode_to_numpy(buf, flag=1, to_rgb=True):
    """Encoded image bytes -> contiguous uint8 array: HxWx3 (RGB, or BGR with ``to_rgb=False``) or HxWx1 for ``flag=0``."""
    from PIL import Image
    picture = Image.open(io.BytesIO(bytes(buf)))
    if flag == 0:
        pixels = np.asarray(picture.convert('L'))[:, :, None]
    else:
        pixels = np.asarray(picture.convert('RGB'))
        if not to_rgb:
            pixels = pixels[:, :, ::-1]
    return np.ascontiguousarray(pixels)


def _to_array(pixels):
    """A NumPy image as the array type of the active front end (``mx.np`` inside ``npx.set_np()``, else ``mx.nd``)."""
    from ..util import is_np_array
    if is_np_array():
        from .. import numpy as front
    else:
        from .. import ndarray as front
    return front.array(pixels, dtype=pixels.dtype)


def imdecode(buf, flag=1, to_rgb=True, out=None, **kwargs):
    """Decode a JPEG/PNG byte string (or a uint8 array holding one).  ``flag=0`` gives one grey channel."""
    raw = buf.asnumpy().tobytes() if isinstance(buf, NDArray) else buf
    image = _to_array(_decode_to_numpy(raw, flag, to_rgb))
    if out is None:
        return image
    out._data.copy_(image._data)
    return out


def imread(filename, flag=1, to_rgb=True, **kwargs):
    with open(filename, 'rb') as f:
        return imdecode(f.read(), flag, to_rgb)


# ---- geometry ---------------------------------------------------------------------------------------------------------
def imresize(src, w, h, interp=1, out=None):
    return _reg.invoke('_cvimresize', [src], {'w': w, 'h': h, 'interp': interp}, out=out)


def copyMakeBorder(src, top, bot, left, right, type=0, value=0.0, **kwargs):  # pylint: disable=redefined-builtin
    params = {'top': top, 'bot': bot, 'left': left, 'right': right, 'type': type, 'value': value}
    return _reg.invoke('_cvcopyMakeBorder', [src], params)


def scale_down(src_size, size):
    """Shrink the crop ``size`` (w, h), keeping its aspect ratio, until it fits into ``src_size`` (w, h)."""
    w, h = size
    src_w, src_h = src_size
    if src_h < h:
        w, h = w * src_h / float(h), src_h
    if src_w < w:
        w, h = src_w, h * src_w / float(w)
    return int(w), int(h)


def _get_interp_method(interp, sizes=()):
    """Interpolation code for a resize: 9 = by direction (cubic when enlarging, area when shrinking, else bilinear; cubic
    when the sizes are unknown), 10 = a random method, anything else as given.  ``sizes`` = (old_h, old_w, new_h, new_w)."""
    if interp == 10:
        return random.randint(0, 4)
    if interp != 9:
        return interp
    if not sizes:
        return 2
    old_h, old_w, new_h, new_w = sizes
    if new_h > old_h and new_w > old_w:
        return 2
    if new_h < old_h and new_w < old_w:
        return 3
    return 1


def resize_short(src, size, interp=2):
    """Resize so that the shorter side becomes ``size`` (aspect ratio kept, integer arithmetic as in the reference)."""
    h, w = src.shape[0], src.shape[1]
    new_h, new_w = (size * h // w, size) if h > w else (size, size * w // h)
    return imresize(src, new_w, new_h, interp=_get_interp_method(interp, (h, w, new_h, new_w)))


def fixed_crop(src, x0, y0, w, h, size=None, interp=2):
    """The ``w`` x ``h`` window at ``(x0, y0)``, resized to ``size`` (w, h) if that differs."""
    window = src[y0:y0 + h, x0:x0 + w]
    if size is None or tuple(size) == (w, h):
        return window
    return imresize(window, size[0], size[1], interp=_get_interp_method(interp, (h, w, size[1], size[0])))


def _crop_at(src, size, interp, place):
    """Crop of (scaled-down) ``size`` whose corner ``place(free_w, free_h)`` picks; returns (image, (x0, y0, w, h))."""
    h, w = src.shape[0], src.shape[1]
    crop_w, crop_h = scale_down((w, h), size)
    x0, y0 = place(w - crop_w, h - crop_h)
    return fixed_crop(src, x0, y0, crop_w, crop_h, size, interp), (x0, y0, crop_w, crop_h)


def random_crop(src, size, interp=2):
    return _crop_at(src, size, interp, lambda fw, fh: (random.randint(0, fw), random.randint(0, fh)))


def center_crop(src, size, interp=2):
    return _crop_at(src, size, interp, lambda fw, fh: (int(fw / 2), int(fh / 2)))


def color_normalize(src, mean, std=None):
    out = src if mean is None else src - mean
    return out if std is None else out / std


def random_size_crop(src, size, area, ratio, interp=2, **kwargs):
    """Inception-style crop: a window covering a random share ``area`` (a lower bound or a (low, high) pair) of the image
    with a random aspect ratio from ``ratio`` (drawn log-uniformly), resized to ``size``; after ten windows that do not
    fit, the centre crop."""
    h, w = src.shape[0], src.shape[1]
    area = kwargs.pop('min_area', area)
    lo, hi = (area, 1.0) if isinstance(area, (int, float)) else area
    log_lo, log_hi = np.log(ratio[0]), np.log(ratio[1])
    for _ in range(10):
        pixels = random.uniform(lo, hi) * h * w
        aspect = np.exp(random.uniform(log_lo, log_hi))
        crop_w, crop_h = int(round(np.sqrt(pixels * aspect))), int(round(np.sqrt(pixels / aspect)))
        if crop_w <= w and crop_h <= h:
            x0, y0 = random.randint(0, w - crop_w), random.randint(0, h - crop_h)
            return fixed_crop(src, x0, y0, crop_w, crop_h, size, interp), (x0, y0, crop_w, crop_h)
    return center_crop(src, size, interp)


# ---- augmenters -------------------------------------------------------------------------------------------------------
class Augmenter(object):
    """An image -> image callable that can describe itself as JSON (``dumps``): ``[lower-cased class name, kwargs]``."""

    def __init__(self, **kwargs):
        self._kwargs = {k: (v.asnumpy().tolist() if isinstance(v, NDArray) else v) for k, v in kwargs.items()}

    def dumps(self):
        return json.dumps([type(self).__name__.lower(), self._kwargs])

    def __call__(self, src):
        raise NotImplementedError('Must override implementation.')


class _Chain(Augmenter):
    """Shared part of the augmenters that hold a list ``ts`` of other augmenters."""

    def __init__(self, ts):
        super().__init__()
        self.ts = ts

    def dumps(self):
        return [type(self).__name__.lower(), [t.dumps() for t in self.ts]]

    def _run(self, src):
        for t in self.ts:
            src = t(src)
        return src


class SequentialAug(_Chain):
    """Apply the augmenters in order."""

    def __call__(self, src):
        return self._run(src)


class RandomOrderAug(_Chain):
    """Apply the augmenters in a fresh random order each time."""

    def __call__(self, src):
        random.shuffle(self.ts)
        return self._run(src)


class _SizedAug(Augmenter):
    """Augmenters configured by a target ``size`` and an interpolation code."""

    def __init__(self, size, interp=2, **extra):
        super().__init__(size=size, interp=interp, **extra)
        self.size = size
        self.interp = interp


class ResizeAug(_SizedAug):
    """Shorter side to ``size``."""

    def __call__(self, src):
        return resize_short(src, self.size, self.interp)


class ForceResizeAug(_SizedAug):
    """To exactly ``size`` = (w, h), ignoring the aspect ratio."""

    def __call__(self, src):
        return imresize(src, self.size[0], self.size[1], interp=_get_interp_method(self.interp))


class RandomCropAug(_SizedAug):
    def __call__(self, src):
        return random_crop(src, self.size, self.interp)[0]


class CenterCropAug(_SizedAug):
    def __call__(self, src):
        return center_crop(src, self.size, self.interp)[0]


class RandomSizedCropAug(_SizedAug):
    """``random_size_crop`` with fixed ``area`` and ``ratio`` ranges (``min_area`` is the older name of ``area``)."""

    def __init__(self, size, area, ratio, interp=2, **kwargs):
        super().__init__(size, interp, area=area, ratio=ratio)
        self.area = kwargs.pop('min_area', area)
        self.ratio = ratio

    def __call__(self, src):
        return random_size_crop(src, self.size, self.area, self.ratio, self.interp)[0]


def _const_like(src, values):
    """A float32 constant on the device and of the array class of ``src``."""
    return type(src)(np.asarray(values, dtype='float32'), ctx=src.context)


def _jitter(strength):
    return 1.0 + random.uniform(-strength, strength)


class BrightnessJitterAug(Augmenter):
    """Scale all pixels by a factor from ``[1 - brightness, 1 + brightness]``."""

    def __init__(self, brightness):
        super().__init__(brightness=brightness)
        self.brightness = brightness

    def __call__(self, src):
        return src * _jitter(self.brightness)


class ContrastJitterAug(Augmenter):
    """Blend with the image's mean luma: ``alpha * src + (1 - alpha) * mean_luma``."""

    def __init__(self, contrast):
        super().__init__(contrast=contrast)
        self.contrast = contrast

    def __call__(self, src):
        alpha = _jitter(self.contrast)
        luma_sum = (src * _const_like(src, [[_LUMA]])).sum()
        mean_luma = luma_sum * (3.0 / src.size)          # src.size counts the three channels
        return src * alpha + mean_luma * (1.0 - alpha)


class SaturationJitterAug(Augmenter):
    """Blend every pixel with its own luma."""

    def __init__(self, saturation):
        super().__init__(saturation=saturation)
        self.saturation = saturation

    def __call__(self, src):
        alpha = _jitter(self.saturation)
        luma = (src * _const_like(src, [[_LUMA]])).sum(axis=2, keepdims=True)
        return src * alpha + luma * (1.0 - alpha)


class HueJitterAug(Augmenter):
    """Rotate the chroma plane of the YIQ representation by an angle from ``[-hue, hue]`` half-turns."""

    def __init__(self, hue):
        super().__init__(hue=hue)
        self.hue = hue
        self.tyiq = np.array([[0.299, 0.587, 0.114], [0.596, -0.274, -0.321], [0.211, -0.523, 0.311]])
        self.ityiq = np.array([[1.0, 0.956, 0.621], [1.0, -0.272, -0.647], [1.0, -1.107, 1.705]])

    def __call__(self, src):
        angle = random.uniform(-self.hue, self.hue) * np.pi
        c, s = np.cos(angle), np.sin(angle)
        rotate = np.array([[1.0, 0.0, 0.0], [0.0, c, -s], [0.0, s, c]])
        rgb_to_rgb = self.ityiq @ rotate @ self.tyiq
        return _reg.invoke('dot', [src, _const_like(src, rgb_to_rgb.T)], {})


class ColorJitterAug(RandomOrderAug):
    """Brightness, contrast and saturation jitter (those with a positive strength) in random order."""

    def __init__(self, brightness, contrast, saturation):
        parts = ((brightness, BrightnessJitterAug), (contrast, ContrastJitterAug), (saturation, SaturationJitterAug))
        super().__init__([cls(strength) for strength, cls in parts if strength > 0])


class LightingAug(Augmenter):
    """AlexNet-style PCA noise: add ``eigvec @ (alpha * eigval)`` with ``alpha ~ N(0, alphastd)`` per component."""

    def __init__(self, alphastd, eigval, eigvec):
        super().__init__(alphastd=alphastd, eigval=eigval, eigvec=eigvec)
        self.alphastd = alphastd
        self.eigval = np.asarray(eigval)
        self.eigvec = np.asarray(eigvec)

    def __call__(self, src):
        alpha = np.random.normal(0, self.alphastd, size=(3,))
        return src + _const_like(src, (self.eigvec * alpha) @ self.eigval)


class ColorNormalizeAug(Augmenter):
    """``(src - mean) / std`` per channel."""

    def __init__(self, mean, std):
        super().__init__(mean=mean, std=std)
        self.mean = self._constant(mean)
        self.std = self._constant(std)

    @staticmethod
    def _constant(v):
        if v is None or isinstance(v, NDArray):
            return v
        from .. import ndarray as nd
        return nd.array(np.asarray(v, dtype='float32'))

    def __call__(self, src):
        return color_normalize(src, self.mean, self.std)


class _WithProbability(Augmenter):
    def __init__(self, p):
        super().__init__(p=p)
        self.p = p

    def _apply(self, src):
        raise NotImplementedError

    def __call__(self, src):
        return self._apply(src) if random.random() < self.p else src


class RandomGrayAug(_WithProbability):
    """With probability ``p`` replace the three channels by their (0.21, 0.72, 0.07) grey value."""

    def __init__(self, p):
        super().__init__(p)
        self.mat = np.tile(np.array([[0.21], [0.72], [0.07]], dtype='float32'), (1, 3))

    def _apply(self, src):
        return _reg.invoke('dot', [src, _const_like(src, self.mat)], {})


class HorizontalFlipAug(_WithProbability):
    """With probability ``p`` mirror left-right."""

    def _apply(self, src):
        return _reg.invoke('reverse', [src], {'axis': 1})


class CastAug(Augmenter):
    def __init__(self, typ='float32'):
        super().__init__(type=typ)
        self.typ = typ

    def __call__(self, src):
        return src.astype(self.typ)


# ImageNet statistics used when `mean=True` / `std=True`, and the PCA of its RGB values for the lighting noise
_IMAGENET_MEAN = (123.68, 116.28, 103.53)
_IMAGENET_STD = (58.395, 57.12, 57.375)
_PCA_EIGVAL = (55.46, 4.794, 1.148)
_PCA_EIGVEC = ((-0.5675, 0.7192, 0.4009), (-0.5808, -0.0045, -0.8140), (-0.5836, -0.6948, 0.4203))


def CreateAugmenter(data_shape, resize=0, rand_crop=False, rand_resize=False, rand_mirror=False, mean=None, std=None,
                    brightness=0, contrast=0, saturation=0, hue=0, pca_noise=0, rand_gray=0, inter_method=2):
    """The standard training / evaluation chain for images of ``data_shape`` = (C, H, W): optional short-side resize, one
    crop (random-sized, random or centre), optional mirror, cast to float32, colour jitters, PCA noise, random grey, and
    normalisation, in this order."""
    crop = (data_shape[2], data_shape[1])
    chain = [ResizeAug(resize, inter_method)] if resize > 0 else []
    if rand_resize:
        if not rand_crop:
            raise AssertionError('rand_resize requires rand_crop')
        chain.append(RandomSizedCropAug(crop, 0.08, (3.0 / 4.0, 4.0 / 3.0), inter_method))
    elif rand_crop:
        chain.append(RandomCropAug(crop, inter_method))
    else:
        chain.append(CenterCropAug(crop, inter_method))
    if rand_mirror:
        chain.append(HorizontalFlipAug(0.5))
    chain.append(CastAug())
    if brightness or contrast or saturation:
        chain.append(ColorJitterAug(brightness, contrast, saturation))
    if hue:
        chain.append(HueJitterAug(hue))
    if pca_noise > 0:
        chain.append(LightingAug(pca_noise, np.array(_PCA_EIGVAL), np.array(_PCA_EIGVEC)))
    if rand_gray > 0:
        chain.append(RandomGrayAug(rand_gray))
    mean = np.array(_IMAGENET_MEAN) if mean is True else mean
    std = np.array(_IMAGENET_STD) if std is True else std
    if mean is not None or std is not None:
        chain.append(ColorNormalizeAug(mean, std))
    return chain


# ---- iterator ---------------------------------------------------------------------------------------------------------
def _parse_list_file(path, dtype):
    """``index<TAB>label...<TAB>relative path`` per line -> ({index: (label array, path)}, [indices in file order])."""
    table, order = {}, []
    with open(path) as f:
        for line in f:
            fields = line.strip().split('\t')
            if len(fields) < 2:
                continue
            key = int(fields[0])
            table[key] = (np.array(fields[1:-1], dtype=dtype), fields[-1])
            order.append(key)
    return table, order


def _parse_list_arg(entries, dtype):
    """``[(label or labels, path), ...]`` -> the same structures, keyed '1', '2', ..."""
    table, order = {}, []
    for pos, (label, path) in enumerate(((e[0], e[1]) for e in entries), 1):
        key = str(pos)
        label = np.array([label] if isinstance(label, (int, float)) else label, dtype=dtype)
        table[key] = (label, path)
        order.append(key)
    return table, order


class ImageIter(object):
    """Batches of augmented images in NCHW ``dtype`` from an image RecordIO file (sequential, or random access with its
    ``.idx``), from a ``.lst`` file naming image files under ``path_root``, or from an in-memory ``imglist``.  Labels come
    from the list when there is one, else from the record headers.

    ``last_batch_handle``: ``pad`` fills the last batch from the start of the data and reports ``pad``; ``discard`` drops
    it; ``roll_over`` keeps it for the next epoch.  ``num_parts`` / ``part_index`` give every worker its share of a list
    or index.  Subclasses customise ``imdecode``, ``read_image``, ``check_valid_image``, ``augmentation_transform`` and
    ``postprocess_data``."""

    def __init__(self, batch_size, data_shape, label_width=1, path_imgrec=None, path_imglist=None, path_root=None,
                 path_imgidx=None, shuffle=False, part_index=0, num_parts=1, aug_list=None, imglist=None,
                 data_name='data', label_name='softmax_label', dtype='float32', last_batch_handle='pad', **kwargs):
        from .. import recordio
        from ..io import DataDesc
        if not (path_imgrec or path_imglist or isinstance(imglist, list)):
            raise AssertionError('one of path_imgrec, path_imglist and imglist is required')
        self.check_data_shape(data_shape)
        self.batch_size = batch_size
        self.data_shape = tuple(data_shape)
        self.label_width = label_width
        self.shuffle = shuffle
        self.dtype = dtype
        self.path_root = path_root
        self.last_batch_handle = last_batch_handle
        # ---- where samples come from ---------------------------------------------------------------------
        self.imgrec = self.imgidx = self.imglist = self.seq = None
        if path_imgrec and path_imgidx:
            self.imgrec = recordio.MXIndexedRecordIO(path_imgidx, path_imgrec, 'r')
            self.imgidx = list(self.imgrec.keys)
        elif path_imgrec:
            self.imgrec = recordio.MXRecordIO(path_imgrec, 'r')
        if path_imglist:
            self.imglist, self.seq = _parse_list_file(path_imglist, dtype)
        elif isinstance(imglist, list):
            self.imglist, self.seq = _parse_list_arg(imglist, dtype)
        elif self.imgidx is not None:
            self.seq = self.imgidx
        if self.seq is not None and num_parts > 1:
            share = len(self.seq) // num_parts
            self.seq = self.seq[part_index * share:(part_index + 1) * share]
        # ---- what a batch looks like -----------------------------------------------------------------------
        label_shape = (batch_size, label_width) if label_width > 1 else (batch_size,)
        self.provide_data = [DataDesc(data_name, (batch_size,) + self.data_shape, dtype)]
        self.provide_label = [DataDesc(label_name, label_shape, dtype)]
        self.auglist = aug_list if aug_list is not None else CreateAugmenter(data_shape, **kwargs)
        self.cur = 0
        self._allow_read = True
        self._carry = None           # (data, label, filled) of an unfinished batch kept by 'roll_over'
        self.reset()

    # the three attributes the reference exposes for the carried-over batch
    @property
    def _cache_data(self):
        return self._carry[0] if self._carry else None

    @property
    def _cache_label(self):
        return self._carry[1] if self._carry else None

    @property
    def _cache_idx(self):
        return self._carry[2] if self._carry else None

    # ---- epoch control --------------------------------------------------------------------------------------
    def _rewind(self):
        if self.imgrec is not None:
            self.imgrec.reset()
        self.cur = 0
        self._allow_read = True

    def reset(self):
        """Start the next epoch (a batch carried over by ``roll_over`` is kept and completed first)."""
        if self.shuffle and self.seq is not None:
            random.shuffle(self.seq)
        if self.last_batch_handle != 'roll_over' or self._carry is None:
            self._rewind()

    def hard_reset(self):
        """Start over and forget a carried-over batch."""
        if self.shuffle and self.seq is not None:
            random.shuffle(self.seq)
        self._carry = None
        self._rewind()

    # ---- one sample -----------------------------------------------------------------------------------------
    def next_sample(self):
        """``(label, encoded image bytes)`` of the next sample; ``StopIteration`` at the end of the data."""
        from .. import recordio
        if not self._allow_read:
            raise StopIteration
        if self.seq is None:                       # sequential record file
            record = self.imgrec.read()
            if record is None:
                if self.last_batch_handle != 'discard':
                    self.imgrec.reset()
                raise StopIteration
            header, payload = recordio.unpack(record)
            return header.label, payload
        if self.cur >= len(self.seq):
            if self.last_batch_handle != 'discard':
                self.cur = 0
            raise StopIteration
        key = self.seq[self.cur]
        self.cur += 1
        if self.imgrec is None:                    # files named by the list
            label, fname = self.imglist[key]
            return label, self.read_image(fname)
        header, payload = recordio.unpack(self.imgrec.read_idx(key))
        return (header.label if self.imglist is None else self.imglist[key][0]), payload

    def _batchify(self, batch_data, batch_label, start=0):
        """Fill rows ``start ..`` of the batch; returns the number of rows filled in total.  Undecodable or invalid
        images are skipped."""
        filled = start
        try:
            while filled < self.batch_size:
                label, raw = self.next_sample()
                image = self.imdecode(raw)
                try:
                    self.check_valid_image(image)
                except RuntimeError as e:
                    logging.debug('Invalid image, skipping:  %s', str(e))
                    continue
                image = self.augmentation_transform(image)
                batch_data[filled] = self.postprocess_data(image)
                batch_label[filled] = label
                filled += 1
        except StopIteration:
            if filled == 0:
                raise
        return filled

    def next(self):
        from ..io import DataBatch
        from .. import ndarray as nd
        if self._carry is not None:
            # 'roll_over': the short batch kept from the last epoch is completed with the first samples of this one
            batch_data, batch_label, filled = self._carry
            self._carry = None
            filled = self._batchify(batch_data, batch_label, filled)
        else:
            batch_data = nd.zeros((self.batch_size,) + self.data_shape, dtype=self.dtype)
            batch_label = nd.zeros(self.provide_label[0][1], dtype=self.dtype)
            filled = self._batchify(batch_data, batch_label)
        pad = self.batch_size - filled
        if pad:
            if self.last_batch_handle == 'discard':
                raise StopIteration
            if self.last_batch_handle == 'roll_over':
                self._carry = (batch_data, batch_label, filled)
                raise StopIteration
            self._batchify(batch_data, batch_label, filled)      # 'pad': wrap around to the start of the data
            self._allow_read = False
        return DataBatch([batch_data], [batch_label], pad=pad)

    __next__ = next

    def __iter__(self):
        return self

    # ---- hooks ----------------------------------------------------------------------------------------------
    def check_data_shape(self, data_shape):
        if len(data_shape) != 3:
            raise ValueError('data_shape should have length 3, with dimensions CxHxW')
        if data_shape[0] not in (1, 3):
            raise ValueError('This iterator expects inputs to have 3 or 1 channels.')

    def check_valid_image(self, data):
        if len(data[0].shape) == 0:
            raise RuntimeError('Data shape is wrong')

    def imdecode(self, s):
        return imdecode(s)

    def read_image(self, fname):
        path = os.path.join(self.path_root, fname) if self.path_root else fname
        with open(path, 'rb') as f:
            return f.read()

    def augmentation_transform(self, data):
        for aug in self.auglist:
            data = aug(data)
        return data

    def postprocess_data(self, datum):
        """HWC -> CHW."""
        return _reg.invoke('transpose', [datum], {'axes': (2, 0, 1)})


def imrotate(src, rotation_degrees, zoom_in=False, zoom_out=False):
    """Rotate a float32 image (C, H, W) or batch (N, C, H, W) counter-clockwise by ``rotation_degrees`` (a scalar, or one
    angle per image) around its centre with bilinear sampling and zero padding.  ``zoom_in`` scales so that no padding
    shows, ``zoom_out`` so that the whole source stays visible."""
    import math
    import torch
    import torch.nn.functional as F
    if zoom_in and zoom_out:
        raise ValueError('`zoom_in` and `zoom_out` cannot be both True')
    t = src._data
    if t.dtype != torch.float32:
        raise TypeError('Only `float32` images are supported by this function')
    single = t.dim() == 3
    if not single and t.dim() != 4:
        raise TypeError('Only 3D (CHW) or 4D (NCHW) images are supported')
    batch = t[None] if single else t
    n, _, h, w = batch.shape
    if isinstance(rotation_degrees, NDArray):
        if single:
            raise TypeError('When a single image is passed the rotation angle is required to be a scalar.')
        ang = rotation_degrees._data.float().to(t.device)
        if ang.numel() != n:
            raise ValueError('The number of images must be equal to the number of rotation angles')
    else:
        ang = torch.full((n,), float(rotation_degrees), device=t.device)
    rad = ang * (math.pi / 180.0)
    cos, sin = torch.cos(rad), torch.sin(rad)
    scale = torch.ones_like(rad)
    ac, as_ = cos.abs(), sin.abs()
    if zoom_out:          # the bounding box of the rotated image, relative to the frame: sample a larger source area
        scale = torch.maximum((w * ac + h * as_) / w, (w * as_ + h * ac) / h)
    elif zoom_in:         # the largest rectangle of the frame's aspect ratio inside the rotated image
        scale = 1.0 / (ac + as_ * max(h / w, w / h))
        scale = scale * ((min(h, w) - 1.0) / min(h, w))      # outermost samples at pixel centres: no blend with padding
    # normalised sampling grid: output pixel -> source location (inverse rotation), aspect corrected
    theta = torch.zeros(n, 2, 3, device=t.device)
    theta[:, 0, 0], theta[:, 0, 1] = cos * scale, -sin * scale * (h / w)
    theta[:, 1, 0], theta[:, 1, 1] = sin * scale * (w / h), cos * scale
    grid = F.affine_grid(theta, list(batch.shape), align_corners=False)
    out = F.grid_sample(batch, grid, mode='bilinear', padding_mode='zeros', align_corners=False)
    return src.__class__._from_tensor(out[0] if single else out, src.context)


def random_rotate(src, angle_limits, zoom_in=False, zoom_out=False):
    """:func:`imrotate` by an angle drawn uniformly from ``angle_limits`` (one draw per image of a batch)."""
    import numpy as _np
    if src.ndim == 3:
        degrees = float(_np.random.uniform(*angle_limits))
    else:
        from .. import ndarray as nd
        degrees = nd.array(_np.random.uniform(*angle_limits, size=src.shape[0]), ctx=src.context, dtype='float32')
    return imrotate(src, degrees, zoom_in=zoom_in, zoom_out=zoom_out)


__all__ += ['imrotate', 'random_rotate']

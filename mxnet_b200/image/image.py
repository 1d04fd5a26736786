"""Image decode/resize helpers, augmenters and ``ImageIter`` (``python/mxnet/image/image.py``)."""
import io
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


def _decode_to_numpy(buf, flag=1, to_rgb=True):
    from PIL import Image
    im = Image.open(io.BytesIO(bytes(buf)))
    if flag == 0:
        a = np.asarray(im.convert('L'))[:, :, None]
    else:
        a = np.asarray(im.convert('RGB'))
        if not to_rgb:
            a = a[:, :, ::-1]
    return np.ascontiguousarray(a)


def _wrap(a, like=None):
    from ..util import is_np_array
    if is_np_array():
        from .. import numpy as mnp
        return mnp.array(a, dtype=a.dtype)
    from .. import ndarray as nd
    return nd.array(a, dtype=a.dtype)


def imdecode(buf, flag=1, to_rgb=True, out=None, **kwargs):
    if isinstance(buf, NDArray):
        buf = buf.asnumpy().tobytes()
    res = _wrap(_decode_to_numpy(buf, flag, to_rgb))
    if out is not None:
        out._data.copy_(res._data)
        return out
    return res


def imread(filename, flag=1, to_rgb=True, **kwargs):
    with open(filename, 'rb') as f:
        return imdecode(f.read(), flag, to_rgb)


def imresize(src, w, h, interp=1, out=None):
    return _reg.invoke('_cvimresize', [src], {'w': w, 'h': h, 'interp': interp}, out=out)


def copyMakeBorder(src, top, bot, left, right, type=0, value=0.0, **kwargs):  # pylint: disable=redefined-builtin
    return _reg.invoke('_cvcopyMakeBorder', [src], {'top': top, 'bot': bot, 'left': left, 'right': right, 'type': type,
                                                    'value': value})


def scale_down(src_size, size):
    w, h = size
    sw, sh = src_size
    if sh < h:
        w, h = float(w * sh) / h, sh
    if sw < w:
        w, h = sw, float(h * sw) / w
    return int(w), int(h)


def _get_interp_method(interp, sizes=()):
    if interp == 9:
        if sizes:
            oh, ow, nh, nw = sizes
            return 2 if nh > oh and nw > ow else (3 if nh < oh and nw < ow else 1)
        return 2
    if interp == 10:
        return random.randint(0, 4)
    return interp


def resize_short(src, size, interp=2):
    h, w, _ = src.shape
    if h > w:
        new_h, new_w = size * h // w, size
    else:
        new_h, new_w = size, size * w // h
    return imresize(src, new_w, new_h, interp=_get_interp_method(interp, (h, w, new_h, new_w)))


def fixed_crop(src, x0, y0, w, h, size=None, interp=2):
    out = src[y0:y0 + h, x0:x0 + w]
    if size is not None and (w, h) != size:
        out = imresize(out, size[0], size[1], interp=_get_interp_method(interp, (h, w, size[1], size[0])))
    return out


def random_crop(src, size, interp=2):
    h, w, _ = src.shape
    new_w, new_h = scale_down((w, h), size)
    x0, y0 = random.randint(0, w - new_w), random.randint(0, h - new_h)
    return fixed_crop(src, x0, y0, new_w, new_h, size, interp), (x0, y0, new_w, new_h)


def center_crop(src, size, interp=2):
    h, w, _ = src.shape
    new_w, new_h = scale_down((w, h), size)
    x0, y0 = int((w - new_w) / 2), int((h - new_h) / 2)
    return fixed_crop(src, x0, y0, new_w, new_h, size, interp), (x0, y0, new_w, new_h)


def color_normalize(src, mean, std=None):
    if mean is not None:
        src = src - mean
    if std is not None:
        src = src / std
    return src


def random_size_crop(src, size, area, ratio, interp=2, **kwargs):
    h, w, _ = src.shape
    src_area = h * w
    if 'min_area' in kwargs:
        area = kwargs.pop('min_area')
    if isinstance(area, (int, float)):
        area = (area, 1.0)
    for _ in range(10):
        target_area = random.uniform(area[0], area[1]) * src_area
        log_ratio = (np.log(ratio[0]), np.log(ratio[1]))
        new_ratio = np.exp(random.uniform(*log_ratio))
        new_w = int(round(np.sqrt(target_area * new_ratio)))
        new_h = int(round(np.sqrt(target_area / new_ratio)))
        if new_w <= w and new_h <= h:
            x0, y0 = random.randint(0, w - new_w), random.randint(0, h - new_h)
            return fixed_crop(src, x0, y0, new_w, new_h, size, interp), (x0, y0, new_w, new_h)
    return center_crop(src, size, interp)


class Augmenter(object):
    def __init__(self, **kwargs):
        self._kwargs = kwargs
        for k, v in self._kwargs.items():
            if isinstance(v, NDArray):
                self._kwargs[k] = v.asnumpy().tolist()

    def dumps(self):
        import json
        return json.dumps([self.__class__.__name__.lower(), self._kwargs])

    def __call__(self, src):
        raise NotImplementedError('Must override implementation.')


class SequentialAug(Augmenter):
    def __init__(self, ts):
        super().__init__()
        self.ts = ts

    def dumps(self):
        return [self.__class__.__name__.lower(), [x.dumps() for x in self.ts]]

    def __call__(self, src):
        for aug in self.ts:
            src = aug(src)
        return src


class ResizeAug(Augmenter):
    def __init__(self, size, interp=2):
        super().__init__(size=size, interp=interp)
        self.size, self.interp = size, interp

    def __call__(self, src):
        return resize_short(src, self.size, self.interp)


class ForceResizeAug(Augmenter):
    def __init__(self, size, interp=2):
        super().__init__(size=size, interp=interp)
        self.size, self.interp = size, interp

    def __call__(self, src):
        return imresize(src, self.size[0], self.size[1], interp=_get_interp_method(self.interp))


class RandomCropAug(Augmenter):
    def __init__(self, size, interp=2):
        super().__init__(size=size, interp=interp)
        self.size, self.interp = size, interp

    def __call__(self, src):
        return random_crop(src, self.size, self.interp)[0]


class RandomSizedCropAug(Augmenter):
    def __init__(self, size, area, ratio, interp=2, **kwargs):
        super().__init__(size=size, area=area, ratio=ratio, interp=interp)
        self.size, self.area, self.ratio, self.interp = size, kwargs.pop('min_area', area), ratio, interp

    def __call__(self, src):
        return random_size_crop(src, self.size, self.area, self.ratio, self.interp)[0]


class CenterCropAug(Augmenter):
    def __init__(self, size, interp=2):
        super().__init__(size=size, interp=interp)
        self.size, self.interp = size, interp

    def __call__(self, src):
        return center_crop(src, self.size, self.interp)[0]


class RandomOrderAug(Augmenter):
    def __init__(self, ts):
        super().__init__()
        self.ts = ts

    def dumps(self):
        return [self.__class__.__name__.lower(), [x.dumps() for x in self.ts]]

    def __call__(self, src):
        random.shuffle(self.ts)
        for t in self.ts:
            src = t(src)
        return src


def _coef(like):
    return like.__class__(np.array([[[0.299, 0.587, 0.114]]], dtype='float32'), ctx=like.context)


class BrightnessJitterAug(Augmenter):
    def __init__(self, brightness):
        super().__init__(brightness=brightness)
        self.brightness = brightness

    def __call__(self, src):
        alpha = 1.0 + random.uniform(-self.brightness, self.brightness)
        return src * alpha


class ContrastJitterAug(Augmenter):
    def __init__(self, contrast):
        super().__init__(contrast=contrast)
        self.contrast = contrast

    def __call__(self, src):
        alpha = 1.0 + random.uniform(-self.contrast, self.contrast)
        gray = src * _coef(src)
        gray = (3.0 * (1.0 - alpha) / gray.size) * gray.sum()
        return src * alpha + gray


class SaturationJitterAug(Augmenter):
    def __init__(self, saturation):
        super().__init__(saturation=saturation)
        self.saturation = saturation

    def __call__(self, src):
        alpha = 1.0 + random.uniform(-self.saturation, self.saturation)
        gray = (src * _coef(src)).sum(axis=2, keepdims=True) * (1.0 - alpha)
        return src * alpha + gray


class HueJitterAug(Augmenter):
    def __init__(self, hue):
        super().__init__(hue=hue)
        self.hue = hue
        self.tyiq = np.array([[0.299, 0.587, 0.114], [0.596, -0.274, -0.321], [0.211, -0.523, 0.311]])
        self.ityiq = np.array([[1.0, 0.956, 0.621], [1.0, -0.272, -0.647], [1.0, -1.107, 1.705]])

    def __call__(self, src):
        alpha = random.uniform(-self.hue, self.hue)
        u, w = np.cos(alpha * np.pi), np.sin(alpha * np.pi)
        bt = np.array([[1.0, 0.0, 0.0], [0.0, u, -w], [0.0, w, u]])
        t = np.dot(np.dot(self.ityiq, bt), self.tyiq).T
        return _reg.invoke('dot', [src, src.__class__(t.astype('float32'), ctx=src.context)], {})


class ColorJitterAug(RandomOrderAug):
    def __init__(self, brightness, contrast, saturation):
        ts = []
        if brightness > 0:
            ts.append(BrightnessJitterAug(brightness))
        if contrast > 0:
            ts.append(ContrastJitterAug(contrast))
        if saturation > 0:
            ts.append(SaturationJitterAug(saturation))
        super().__init__(ts)


class LightingAug(Augmenter):
    def __init__(self, alphastd, eigval, eigvec):
        super().__init__(alphastd=alphastd, eigval=eigval, eigvec=eigvec)
        self.alphastd, self.eigval, self.eigvec = alphastd, np.asarray(eigval), np.asarray(eigvec)

    def __call__(self, src):
        alpha = np.random.normal(0, self.alphastd, size=(3,))
        rgb = np.dot(self.eigvec * alpha, self.eigval)
        return src + src.__class__(rgb.astype('float32'), ctx=src.context)


class ColorNormalizeAug(Augmenter):
    def __init__(self, mean, std):
        super().__init__(mean=mean, std=std)
        from .. import ndarray as nd
        self.mean = mean if mean is None or isinstance(mean, NDArray) else nd.array(np.asarray(mean, dtype='float32'))
        self.std = std if std is None or isinstance(std, NDArray) else nd.array(np.asarray(std, dtype='float32'))

    def __call__(self, src):
        return color_normalize(src, self.mean, self.std)


class RandomGrayAug(Augmenter):
    def __init__(self, p):
        super().__init__(p=p)
        self.p = p
        self.mat = np.array([[0.21, 0.21, 0.21], [0.72, 0.72, 0.72], [0.07, 0.07, 0.07]], dtype='float32')

    def __call__(self, src):
        if random.random() < self.p:
            src = _reg.invoke('dot', [src, src.__class__(self.mat, ctx=src.context)], {})
        return src


class HorizontalFlipAug(Augmenter):
    def __init__(self, p):
        super().__init__(p=p)
        self.p = p

    def __call__(self, src):
        if random.random() < self.p:
            src = _reg.invoke('reverse', [src], {'axis': 1})
        return src


class CastAug(Augmenter):
    def __init__(self, typ='float32'):
        super().__init__(type=typ)
        self.typ = typ

    def __call__(self, src):
        return src.astype(self.typ)


def CreateAugmenter(data_shape, resize=0, rand_crop=False, rand_resize=False, rand_mirror=False, mean=None, std=None,
                    brightness=0, contrast=0, saturation=0, hue=0, pca_noise=0, rand_gray=0, inter_method=2):
    auglist = []
    if resize > 0:
        auglist.append(ResizeAug(resize, inter_method))
    crop_size = (data_shape[2], data_shape[1])
    if rand_resize:
        assert rand_crop
        auglist.append(RandomSizedCropAug(crop_size, 0.08, (3.0 / 4.0, 4.0 / 3.0), inter_method))
    elif rand_crop:
        auglist.append(RandomCropAug(crop_size, inter_method))
    else:
        auglist.append(CenterCropAug(crop_size, inter_method))
    if rand_mirror:
        auglist.append(HorizontalFlipAug(0.5))
    auglist.append(CastAug())
    if brightness or contrast or saturation:
        auglist.append(ColorJitterAug(brightness, contrast, saturation))
    if hue:
        auglist.append(HueJitterAug(hue))
    if pca_noise > 0:
        eigval = np.array([55.46, 4.794, 1.148])
        eigvec = np.array([[-0.5675, 0.7192, 0.4009], [-0.5808, -0.0045, -0.8140], [-0.5836, -0.6948, 0.4203]])
        auglist.append(LightingAug(pca_noise, eigval, eigvec))
    if rand_gray > 0:
        auglist.append(RandomGrayAug(rand_gray))
    if mean is True:
        mean = np.array([123.68, 116.28, 103.53])
    if std is True:
        std = np.array([58.395, 57.12, 57.375])
    if mean is not None or std is not None:
        auglist.append(ColorNormalizeAug(mean, std))
    return auglist


class ImageIter(object):
    """Image iterator over a RecordIO file or an image list with a chain of augmenters."""

    def __init__(self, batch_size, data_shape, label_width=1, path_imgrec=None, path_imglist=None, path_root=None,
                 path_imgidx=None, shuffle=False, part_index=0, num_parts=1, aug_list=None, imglist=None,
                 data_name='data', label_name='softmax_label', dtype='float32', last_batch_handle='pad', **kwargs):
        from .. import recordio
        from ..io import DataDesc
        assert path_imgrec or path_imglist or (isinstance(imglist, list))
        self.imgrec = self.imgidx = self.imglist = None
        self.seq = None
        if path_imgrec:
            if path_imgidx:
                self.imgrec = recordio.MXIndexedRecordIO(path_imgidx, path_imgrec, 'r')
                self.imgidx = list(self.imgrec.keys)
            else:
                self.imgrec = recordio.MXRecordIO(path_imgrec, 'r')
        if path_imglist:
            with open(path_imglist) as fin:
                imglist_d, keys = {}, []
                for line in iter(fin.readline, ''):
                    line = line.strip().split('\t')
                    label = np.array(line[1:-1], dtype=dtype)
                    key = int(line[0])
                    imglist_d[key] = (label, line[-1])
                    keys.append(key)
                self.imglist, self.seq = imglist_d, keys
        elif isinstance(imglist, list):
            result, keys = {}, []
            for index, img in enumerate(imglist, 1):
                key = str(index)
                label = np.array(img[0], dtype=dtype) if not isinstance(img[0], (int, float)) else np.array([img[0]], dtype=dtype)
                result[key] = (label, img[1])
                keys.append(key)
            self.imglist, self.seq = result, keys
        elif self.imgidx is not None:
            self.seq = self.imgidx
        self.path_root = path_root
        self.check_data_shape(data_shape)
        self.provide_data = [DataDesc(data_name, (batch_size,) + tuple(data_shape), dtype)]
        self.provide_label = [DataDesc(label_name, (batch_size, label_width) if label_width > 1 else (batch_size,), dtype)]
        self.batch_size, self.data_shape, self.label_width, self.shuffle, self.dtype = \
            batch_size, tuple(data_shape), label_width, shuffle, dtype
        if self.seq is not None and num_parts > 1:
            C = len(self.seq) // num_parts
            self.seq = self.seq[part_index * C:(part_index + 1) * C]
        self.auglist = CreateAugmenter(data_shape, **kwargs) if aug_list is None else aug_list
        self.cur = 0
        self._allow_read = True
        self.last_batch_handle = last_batch_handle
        self._cache_data = self._cache_label = self._cache_idx = None
        self.reset()

    def reset(self):
        if self.seq is not None and self.shuffle:
            random.shuffle(self.seq)
        if self.last_batch_handle != 'roll_over' or self._cache_data is None:
            if self.imgrec is not None:
                self.imgrec.reset()
            self.cur = 0
            if self._allow_read is False:
                self._allow_read = True

    def hard_reset(self):
        if self.seq is not None and self.shuffle:
            random.shuffle(self.seq)
        if self.imgrec is not None:
            self.imgrec.reset()
        self.cur = 0
        self._allow_read = True
        self._cache_data = self._cache_label = self._cache_idx = None

    def next_sample(self):
        from .. import recordio
        if self._allow_read is False:
            raise StopIteration
        if self.seq is not None:
            if self.cur < len(self.seq):
                idx = self.seq[self.cur]
            else:
                if self.last_batch_handle != 'discard':
                    self.cur = 0
                raise StopIteration
            self.cur += 1
            if self.imgrec is not None:
                s = self.imgrec.read_idx(idx)
                header, img = recordio.unpack(s)
                if self.imglist is None:
                    return header.label, img
                return self.imglist[idx][0], img
            label, fname = self.imglist[idx]
            return label, self.read_image(fname)
        s = self.imgrec.read()
        if s is None:
            if self.last_batch_handle != 'discard':
                self.imgrec.reset()
            raise StopIteration
        header, img = recordio.unpack(s)
        return header.label, img

    def _batchify(self, batch_data, batch_label, start=0):
        i = start
        batch_size = self.batch_size
        try:
            while i < batch_size:
                label, s = self.next_sample()
                data = self.imdecode(s)
                try:
                    self.check_valid_image(data)
                except RuntimeError as e:
                    logging.debug('Invalid image, skipping:  %s', str(e))
                    continue
                data = self.augmentation_transform(data)
                assert i < batch_size, 'Batch size must be multiples of augmenter output length'
                batch_data[i] = self.postprocess_data(data)
                batch_label[i] = label
                i += 1
        except StopIteration:
            if not i:
                raise StopIteration
        return i

    def next(self):
        from ..io import DataBatch
        from .. import ndarray as nd
        batch_size = self.batch_size
        c, h, w = self.data_shape
        if self._cache_data is not None:
            batch_data, batch_label, i = self._cache_data, self._cache_label, self._cache_idx
            self._cache_data = self._cache_label = self._cache_idx = None
        else:
            batch_data = nd.zeros((batch_size, c, h, w), dtype=self.dtype)
            batch_label = nd.zeros(self.provide_label[0][1], dtype=self.dtype)
            i = self._batchify(batch_data, batch_label)
        pad = batch_size - i
        if pad != 0:
            if self.last_batch_handle == 'discard':
                raise StopIteration
            if self.last_batch_handle == 'roll_over' and self._cache_data is None:
                self._cache_data, self._cache_label, self._cache_idx = batch_data, batch_label, i
                raise StopIteration
            _ = self._batchify(batch_data, batch_label, i)
            if self.last_batch_handle == 'pad':
                self._allow_read = False
            else:
                self._cache_data = self._cache_label = self._cache_idx = None
        return DataBatch([batch_data], [batch_label], pad=pad)

    __next__ = next

    def __iter__(self):
        return self

    def check_data_shape(self, data_shape):
        if not len(data_shape) == 3:
            raise ValueError('data_shape should have length 3, with dimensions CxHxW')
        if not data_shape[0] == 3 and not data_shape[0] == 1:
            raise ValueError('This iterator expects inputs to have 3 or 1 channels.')

    def check_valid_image(self, data):
        if len(data[0].shape) == 0:
            raise RuntimeError('Data shape is wrong')

    def imdecode(self, s):
        return imdecode(s)

    def read_image(self, fname):
        with open(os.path.join(self.path_root, fname) if self.path_root else fname, 'rb') as fin:
            return fin.read()

    def augmentation_transform(self, data):
        for aug in self.auglist:
            data = aug(data)
        return data

    def postprocess_data(self, datum):
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

"""Detection augmenters and ``ImageDetIter`` (``python/mxnet/image/detection.py``)."""
import random

import numpy as np

from .image import Augmenter, ImageIter, imresize, fixed_crop, CastAug, ColorJitterAug, HueJitterAug, LightingAug, \
    RandomGrayAug, ColorNormalizeAug, ResizeAug, ForceResizeAug

__all__ = ['DetAugmenter', 'DetBorrowAug', 'DetRandomSelectAug', 'DetHorizontalFlipAug', 'DetRandomCropAug',
           'DetRandomPadAug', 'CreateDetAugmenter', 'ImageDetIter']


class DetAugmenter(object):
    def __init__(self, **kwargs):
        self._kwargs = kwargs

    def dumps(self):
        import json
        return json.dumps([self.__class__.__name__.lower(), self._kwargs])

    def __call__(self, src, label):
        raise NotImplementedError('Must override implementation.')


class DetBorrowAug(DetAugmenter):
    def __init__(self, augmenter):
        if not isinstance(augmenter, Augmenter):
            raise TypeError('Borrowing from invalid Augmenter')
        super().__init__(augmenter=augmenter.dumps())
        self.augmenter = augmenter

    def __call__(self, src, label):
        return self.augmenter(src), label


class DetRandomSelectAug(DetAugmenter):
    def __init__(self, aug_list, skip_prob=0):
        super().__init__(skip_prob=skip_prob)
        self.aug_list = aug_list if isinstance(aug_list, (list, tuple)) else [aug_list]
        self.skip_prob = skip_prob

    def __call__(self, src, label):
        if random.random() < self.skip_prob or not self.aug_list:
            return src, label
        return random.choice(self.aug_list)(src, label)


class DetHorizontalFlipAug(DetAugmenter):
    def __init__(self, p):
        super().__init__(p=p)
        self.p = p

    def __call__(self, src, label):
        if random.random() < self.p:
            from ..ops import registry as _reg
            src = _reg.invoke('reverse', [src], {'axis': 1})
            tmp = 1.0 - label[:, 1]
            label[:, 1] = 1.0 - label[:, 3]
            label[:, 3] = tmp
        return src, label


class DetRandomCropAug(DetAugmenter):
    def __init__(self, min_object_covered=0.1, aspect_ratio_range=(0.75, 1.33), area_range=(0.05, 1.0),
                 min_eject_coverage=0.3, max_attempts=50):
        super().__init__(min_object_covered=min_object_covered, aspect_ratio_range=aspect_ratio_range,
                         area_range=area_range, min_eject_coverage=min_eject_coverage, max_attempts=max_attempts)
        self.min_object_covered, self.aspect_ratio_range, self.area_range = min_object_covered, aspect_ratio_range, area_range
        self.min_eject_coverage, self.max_attempts = min_eject_coverage, max_attempts

    def __call__(self, src, label):
        h, w = src.shape[0], src.shape[1]
        for _ in range(self.max_attempts):
            area = random.uniform(*self.area_range) * h * w
            ratio = random.uniform(*self.aspect_ratio_range)
            cw, ch = int(round(np.sqrt(area * ratio))), int(round(np.sqrt(area / ratio)))
            if cw <= 0 or ch <= 0 or cw > w or ch > h:
                continue
            x0, y0 = random.randint(0, w - cw), random.randint(0, h - ch)
            box = np.array([x0 / w, y0 / h, (x0 + cw) / w, (y0 + ch) / h])
            new = self._update_labels(label, box)
            if new is not None:
                return fixed_crop(src, x0, y0, cw, ch), new
        return src, label

    def _update_labels(self, label, box):
        valid = label[:, 0] >= 0
        if not valid.any():
            return None
        obj = label[valid].copy()
        ix1, iy1 = np.maximum(obj[:, 1], box[0]), np.maximum(obj[:, 2], box[1])
        ix2, iy2 = np.minimum(obj[:, 3], box[2]), np.minimum(obj[:, 4], box[3])
        inter = np.clip(ix2 - ix1, 0, None) * np.clip(iy2 - iy1, 0, None)
        areas = (obj[:, 3] - obj[:, 1]) * (obj[:, 4] - obj[:, 2])
        cov = inter / np.maximum(areas, 1e-12)
        if cov.max() < self.min_object_covered:
            return None
        keep = cov >= self.min_eject_coverage
        if not keep.any():
            return None
        obj = obj[keep]
        bw, bh = box[2] - box[0], box[3] - box[1]
        obj[:, 1] = np.clip((obj[:, 1] - box[0]) / bw, 0, 1)
        obj[:, 3] = np.clip((obj[:, 3] - box[0]) / bw, 0, 1)
        obj[:, 2] = np.clip((obj[:, 2] - box[1]) / bh, 0, 1)
        obj[:, 4] = np.clip((obj[:, 4] - box[1]) / bh, 0, 1)
        out = np.full_like(label, -1.0)
        out[:obj.shape[0]] = obj
        return out


class DetRandomPadAug(DetAugmenter):
    def __init__(self, aspect_ratio_range=(0.75, 1.33), area_range=(1.0, 3.0), max_attempts=50, pad_val=(128, 128, 128)):
        super().__init__(aspect_ratio_range=aspect_ratio_range, area_range=area_range, max_attempts=max_attempts, pad_val=pad_val)
        self.aspect_ratio_range, self.area_range, self.max_attempts, self.pad_val = aspect_ratio_range, area_range, max_attempts, pad_val

    def __call__(self, src, label):
        h, w = src.shape[0], src.shape[1]
        for _ in range(self.max_attempts):
            area = random.uniform(*self.area_range) * h * w
            ratio = random.uniform(*self.aspect_ratio_range)
            pw, ph = int(round(np.sqrt(area * ratio))), int(round(np.sqrt(area / ratio)))
            if pw < w or ph < h:
                continue
            x0, y0 = random.randint(0, pw - w), random.randint(0, ph - h)
            canvas = np.empty((ph, pw, src.shape[2]), dtype=src.asnumpy().dtype)
            canvas[:] = np.asarray(self.pad_val, dtype=canvas.dtype)
            canvas[y0:y0 + h, x0:x0 + w] = src.asnumpy()
            new = label.copy()
            valid = new[:, 0] >= 0
            new[valid, 1] = (new[valid, 1] * w + x0) / pw
            new[valid, 3] = (new[valid, 3] * w + x0) / pw
            new[valid, 2] = (new[valid, 2] * h + y0) / ph
            new[valid, 4] = (new[valid, 4] * h + y0) / ph
            return src.__class__(canvas, ctx=src.context, dtype=canvas.dtype), new
        return src, label


def CreateDetAugmenter(data_shape, resize=0, rand_crop=0, rand_pad=0, rand_gray=0, rand_mirror=False, mean=None,
                       std=None, brightness=0, contrast=0, saturation=0, pca_noise=0, hue=0, inter_method=2,
                       min_object_covered=0.1, aspect_ratio_range=(0.75, 1.33), area_range=(0.05, 3.0),
                       min_eject_coverage=0.3, max_attempts=50, pad_val=(127, 127, 127)):
    auglist = []
    if resize > 0:
        auglist.append(DetBorrowAug(ResizeAug(resize, inter_method)))
    if rand_crop > 0:
        crop = DetRandomCropAug(min_object_covered, aspect_ratio_range, (area_range[0], min(1.0, area_range[1])),
                                min_eject_coverage, max_attempts)
        auglist.append(DetRandomSelectAug([crop], 1 - rand_crop))
    if rand_mirror > 0:
        auglist.append(DetHorizontalFlipAug(0.5))
    if rand_pad > 0:
        pad = DetRandomPadAug(aspect_ratio_range, (max(1.0, area_range[0]), area_range[1]), max_attempts, pad_val)
        auglist.append(DetRandomSelectAug([pad], 1 - rand_pad))
    auglist.append(DetBorrowAug(ForceResizeAug((data_shape[2], data_shape[1]), inter_method)))
    auglist.append(DetBorrowAug(CastAug()))
    if brightness or contrast or saturation:
        auglist.append(DetBorrowAug(ColorJitterAug(brightness, contrast, saturation)))
    if hue:
        auglist.append(DetBorrowAug(HueJitterAug(hue)))
    if pca_noise > 0:
        eigval = np.array([55.46, 4.794, 1.148])
        eigvec = np.array([[-0.5675, 0.7192, 0.4009], [-0.5808, -0.0045, -0.8140], [-0.5836, -0.6948, 0.4203]])
        auglist.append(DetBorrowAug(LightingAug(pca_noise, eigval, eigvec)))
    if rand_gray > 0:
        auglist.append(DetBorrowAug(RandomGrayAug(rand_gray)))
    if mean is True:
        mean = np.array([123.68, 116.28, 103.53])
    if std is True:
        std = np.array([58.395, 57.12, 57.375])
    if mean is not None or std is not None:
        auglist.append(DetBorrowAug(ColorNormalizeAug(mean, std)))
    return auglist


class ImageDetIter(ImageIter):
    """Detection iterator: labels are ``[header..., obj0..., obj1...]`` arrays reshaped to (N, width)."""

    def __init__(self, batch_size, data_shape, path_imgrec=None, path_imglist=None, path_root=None, path_imgidx=None,
                 shuffle=False, part_index=0, num_parts=1, aug_list=None, imglist=None, data_name='data',
                 label_name='label', last_batch_handle='pad', **kwargs):
        super().__init__(batch_size=batch_size, data_shape=data_shape, path_imgrec=path_imgrec, path_imglist=path_imglist,
                         path_root=path_root, path_imgidx=path_imgidx, shuffle=shuffle, part_index=part_index,
                         num_parts=num_parts, aug_list=[], imglist=imglist, data_name=data_name, label_name=label_name,
                         last_batch_handle=last_batch_handle)
        self.auglist = CreateDetAugmenter(data_shape, **kwargs) if aug_list is None else aug_list
        label_shape = self._estimate_label_shape()
        from ..io import DataDesc
        self.provide_label = [DataDesc(label_name, (self.batch_size, label_shape[0], label_shape[1]))]
        self.label_shape = label_shape

    def _parse_label(self, label):
        raw = np.asarray(label).ravel()
        if raw.size < 7:
            raise RuntimeError('Label shape is invalid: ' + str(raw.shape))
        header_width, obj_width = int(raw[0]), int(raw[1])
        out = raw[header_width:].reshape(-1, obj_width)
        valid = np.where(np.logical_and(out[:, 3] > out[:, 1], out[:, 4] > out[:, 2]))[0]
        if valid.size < 1:
            raise RuntimeError('Encounter sample with no valid label.')
        return out[valid, :]

    def _estimate_label_shape(self):
        max_count, width = 0, 5
        self.reset()
        try:
            while True:
                label, _ = self.next_sample()
                label = self._parse_label(label)
                max_count = max(max_count, label.shape[0])
                width = label.shape[1]
        except StopIteration:
            pass
        self.reset()
        return (max_count, width)

    def next(self):
        from ..io import DataBatch
        from .. import ndarray as nd
        batch_size = self.batch_size
        c, h, w = self.data_shape
        batch_data = np.zeros((batch_size, c, h, w), dtype='float32')
        batch_label = np.full((batch_size,) + tuple(self.label_shape), -1.0, dtype='float32')
        i = 0
        try:
            while i < batch_size:
                label, s = self.next_sample()
                data = self.imdecode(s)
                try:
                    label = self._parse_label(label)
                except RuntimeError:
                    continue
                for aug in self.auglist:
                    data, label = aug(data, label)
                batch_data[i] = data.asnumpy().transpose(2, 0, 1)
                n = min(label.shape[0], self.label_shape[0])
                batch_label[i, :n] = label[:n]
                i += 1
        except StopIteration:
            if not i:
                raise StopIteration
        return DataBatch([nd.array(batch_data)], [nd.array(batch_label)], pad=batch_size - i)

    __next__ = next


def CreateMultiRandCropAugmenter(min_object_covered=0.1, aspect_ratio_range=(0.75, 1.33), area_range=(0.05, 1.0),
                                 min_eject_coverage=0.3, max_attempts=50, skip_prob=0):
    """Several random-crop augmenters of which one is picked per sample (or none, with probability ``skip_prob``).  Every
    parameter may be a single value (shared) or a list with one value per augmenter."""
    params = [min_object_covered, aspect_ratio_range, area_range, min_eject_coverage, max_attempts]
    num = max([len(p) for p in params if isinstance(p, list)] + [1])
    aligned = []
    for p in params:
        if isinstance(p, list):
            assert len(p) == num, 'all list parameters must have the same length'
            aligned.append(p)
        else:
            aligned.append([p] * num)
    augs = [DetRandomCropAug(min_object_covered=moc, aspect_ratio_range=arr, area_range=ar, min_eject_coverage=mec, max_attempts=ma)
            for moc, arr, ar, mec, ma in zip(*aligned)]
    return DetRandomSelectAug(augs, skip_prob=skip_prob)


__all__ += ['CreateMultiRandCropAugmenter']

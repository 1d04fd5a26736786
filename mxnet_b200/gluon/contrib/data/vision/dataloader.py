"""One-call data loaders for image classification and detection (``gluon/contrib/data/vision/dataloader.py``): a
record file or an image list becomes a ``DataLoader`` with the usual augmentation pipeline attached."""
import logging

import numpy as np

from mxnet_b200.gluon import block as _block
from mxnet_b200.gluon.data import DataLoader
from mxnet_b200.gluon.data.vision import ImageListDataset, ImageRecordDataset, transforms
from mxnet_b200.gluon.nn import Sequential
from .transforms import bbox as bbox_tf

__all__ = ['create_image_augment', 'ImageDataLoader', 'create_bbox_augment', 'ImageBboxDataLoader', 'BboxLabelTransform']


def create_image_augment(data_shape, resize=0, rand_crop=False, rand_resize=False, rand_mirror=False, mean=None, std=None,
                         brightness=0, contrast=0, saturation=0, hue=0, pca_noise=0, rand_gray=0, inter_method=2,
                         dtype='float32'):
    """The classification pipeline as one block: optional resize of the short side, (random resized | random | centre)
    crop to ``data_shape`` (C, H, W), mirror, colour jitter, lighting noise, gray, then ToTensor and normalisation
    (``mean=True`` / ``std=True`` select the ImageNet statistics)."""
    if inter_method == 10:
        inter_method = np.random.randint(0, 5)
    aug = Sequential()
    if resize > 0:
        aug.add(transforms.Resize(resize, keep_ratio=True, interpolation=inter_method))
    crop = (data_shape[2], data_shape[1])
    if rand_resize:
        assert rand_crop, 'rand_resize needs rand_crop'
        aug.add(transforms.RandomResizedCrop(crop, scale=(0.08, 1.0), ratio=(3.0 / 4.0, 4.0 / 3.0), interpolation=inter_method))
    elif rand_crop:
        aug.add(transforms.RandomCrop(crop, interpolation=inter_method))
    else:
        aug.add(transforms.CenterCrop(crop, interpolation=inter_method))
    if rand_mirror:
        aug.add(transforms.RandomFlipLeftRight(0.5))
    aug.add(transforms.Cast())
    if brightness or contrast or saturation or hue:
        aug.add(transforms.RandomColorJitter(brightness, contrast, saturation, hue))
    if pca_noise > 0:
        aug.add(transforms.RandomLighting(pca_noise))
    if rand_gray > 0:
        aug.add(transforms.RandomGray(rand_gray))
    if mean is True:
        mean = [123.68, 116.28, 103.53]
    if std is True:
        std = [58.395, 57.12, 57.375]
    aug.add(transforms.ToTensor())
    if mean is not None or std is not None:
        mean = [0.0] * 3 if mean is None else [m / 255.0 for m in np.atleast_1d(mean)]
        std = [1.0] * 3 if std is None else [s / 255.0 for s in np.atleast_1d(std)]
        aug.add(transforms.Normalize(mean, std))
    aug.add(transforms.Cast(dtype))
    return aug


def _dataset(path_imgrec, path_imglist, path_root, imglist, class_name):
    if path_imgrec:
        logging.info('%s: loading recordio %s...', class_name, path_imgrec)
        return ImageRecordDataset(path_imgrec, flag=1)
    if path_imglist:
        logging.info('%s: loading image list %s...', class_name, path_imglist)
        return ImageListDataset(path_root, path_imglist, flag=1)
    if isinstance(imglist, list):
        logging.info('%s: loading image list...', class_name)
        return ImageListDataset(path_root, imglist, flag=1)
    raise ValueError('Either path_imgrec, path_imglist, or imglist must be provided')


def _shard(dataset, num_parts, part_index):
    if num_parts > 1:
        return dataset.shard(num_parts, part_index)
    return dataset


class ImageDataLoader(object):
    """Classification batches (data (N, C, H, W), label (N,)) from a record file, an image list file or an in-memory list;
    ``aug_list=None`` takes :func:`create_image_augment` with the keyword arguments given here."""

    def __init__(self, batch_size, data_shape, path_imgrec=None, path_imglist=None, path_root='.', part_index=0, num_parts=1,
                 aug_list=None, imglist=None, dtype='float32', shuffle=False, sampler=None, last_batch=None, batch_sampler=None,
                 batchify_fn=None, num_workers=0, pin_memory=False, pin_device_id=0, prefetch=None, thread_pool=False,
                 timeout=120, try_nopython=None, **kwargs):
        assert path_imgrec or path_imglist or isinstance(imglist, list)
        assert dtype in ('int32', 'float32', 'int64', 'float64'), dtype + ' label not supported'
        dataset = _shard(_dataset(path_imgrec, path_imglist, path_root, imglist, type(self).__name__), num_parts, part_index)
        if aug_list is None:
            augmenter = create_image_augment(data_shape, **kwargs)
        elif isinstance(aug_list, list):
            augmenter = Sequential()
            for a in aug_list:
                augmenter.add(a)
        elif isinstance(aug_list, _block.Block):
            augmenter = aug_list
        else:
            raise ValueError('aug_list must be a list of Blocks or Block')
        self._iter = DataLoader(dataset.transform_first(augmenter), batch_size=batch_size, shuffle=shuffle, sampler=sampler,
                                last_batch=last_batch, batch_sampler=batch_sampler, batchify_fn=batchify_fn, num_workers=num_workers,
                                pin_memory=pin_memory, pin_device_id=pin_device_id, prefetch=prefetch, thread_pool=thread_pool,
                                timeout=timeout)

    def __iter__(self):
        return iter(self._iter)

    def __len__(self):
        return len(self._iter)


class _PairSequential(_block.Block):
    """Apply (image, boxes) -> (image, boxes) blocks in order."""

    def __init__(self, blocks=()):
        super().__init__()
        self._blocks = list(blocks)

    def add(self, b):
        self._blocks.append(b)

    def forward(self, img, label):
        for b in self._blocks:
            img, label = b(img, label)
        return img, label


class _ImageOnly(_block.Block):
    def __init__(self, fn):
        super().__init__()
        self._fn = fn

    def forward(self, img, label):
        return self._fn(img), label


def create_bbox_augment(data_shape, rand_crop=0, rand_pad=0, rand_gray=0, rand_mirror=False, mean=None, std=None, brightness=0,
                        contrast=0, saturation=0, pca_noise=0, hue=0, inter_method=2, max_aspect_ratio=2, area_range=(0.3, 3.0),
                        max_attempts=50, pad_val=(127, 127, 127), dtype='float32'):
    """The detection pipeline on (image, boxes) pairs: constrained random crop (probability ``rand_crop``), random expand
    (``rand_pad``), mirror, resize to ``data_shape`` (C, H, W), then the colour / tensor transforms on the image."""
    if inter_method == 10:
        inter_method = np.random.randint(0, 5)
    aug = _PairSequential()
    if rand_crop > 0:
        aug.add(bbox_tf.ImageBboxRandomCropWithConstraints(p=rand_crop, min_scale=area_range[0], max_scale=1.0,
                                                           max_aspect_ratio=max_aspect_ratio, max_trial=max_attempts))
    if rand_mirror:
        aug.add(bbox_tf.ImageBboxRandomFlipLeftRight(0.5))
    if rand_pad > 0:
        aug.add(bbox_tf.ImageBboxRandomExpand(p=rand_pad, max_ratio=area_range[1], fill=pad_val))
    aug.add(bbox_tf.ImageBboxResize(data_shape[2], data_shape[1], interp=inter_method))
    aug.add(_ImageOnly(transforms.Cast()))
    if brightness or contrast or saturation or hue:
        aug.add(_ImageOnly(transforms.RandomColorJitter(brightness, contrast, saturation, hue)))
    if pca_noise > 0:
        aug.add(_ImageOnly(transforms.RandomLighting(pca_noise)))
    if rand_gray > 0:
        aug.add(_ImageOnly(transforms.RandomGray(rand_gray)))
    if mean is True:
        mean = [123.68, 116.28, 103.53]
    if std is True:
        std = [58.395, 57.12, 57.375]
    aug.add(_ImageOnly(transforms.ToTensor()))
    if mean is not None or std is not None:
        mean = [0.0] * 3 if mean is None else [m / 255.0 for m in np.atleast_1d(mean)]
        std = [1.0] * 3 if std is None else [s / 255.0 for s in np.atleast_1d(std)]
        aug.add(_ImageOnly(transforms.Normalize(mean, std)))
    aug.add(_ImageOnly(transforms.Cast(dtype)))
    return aug


class BboxLabelTransform(_block.Block):
    """The flat detection label of a record (header length, object width, header ..., then per object id, x0, y0, x1, y1,
    extras) as an (N, 5+) array with columns x0, y0, x1, y1, id, extras; normalised coordinates become pixels."""

    def __init__(self, coord_normalized=True):
        super().__init__()
        self._coord_normalized = coord_normalized

    def forward(self, img, label):
        label = np.asarray(label.asnumpy() if hasattr(label, 'asnumpy') else label, dtype='float32').flatten()
        header_len, width = int(label[0]), int(label[1])
        if width < 5:
            raise ValueError('Label info for each object should >= 5, given %d' % width)
        if len(label) < header_len + 5:
            raise ValueError('Expected label length >= %d, got %d' % (header_len + 5, len(label)))
        if (len(label) - header_len) % width:
            raise ValueError('Broken label of size %d, cannot reshape into (N, %d) if header length %d is excluded'
                             % (len(label), width, header_len))
        objs = label[header_len:].reshape(-1, width).copy()
        ids = objs[:, 0].copy()
        objs[:, :4] = objs[:, 1:5]
        objs[:, 4] = ids
        if self._coord_normalized:
            h, w = img.shape[0], img.shape[1]
            objs[:, [0, 2]] *= w
            objs[:, [1, 3]] *= h
        return img, objs


def _pad_boxes_batchify(samples):
    """Stack the images; pad every sample's boxes with rows of -1 to the longest of the batch."""
    from mxnet_b200 import nd
    imgs = nd.stack(*[s[0] if hasattr(s[0], 'asnumpy') else nd.array(s[0]) for s in samples])
    boxes = [np.asarray(s[1].asnumpy() if hasattr(s[1], 'asnumpy') else s[1], dtype='float32') for s in samples]
    n = max(b.shape[0] for b in boxes)
    width = boxes[0].shape[1]
    out = np.full((len(boxes), n, width), -1.0, dtype='float32')
    for i, b in enumerate(boxes):
        out[i, :b.shape[0]] = b
    return imgs, nd.array(out)


class ImageBboxDataLoader(object):
    """Detection batches: data (N, C, H, W) and labels (N, M, 5+) padded with -1 rows, from a record file or list whose
    labels follow the detection header layout."""

    def __init__(self, batch_size, data_shape, path_imgrec=None, path_imglist=None, path_root='.', part_index=0, num_parts=1,
                 aug_list=None, imglist=None, coord_normalized=True, dtype='float32', shuffle=False, sampler=None,
                 last_batch=None, batch_sampler=None, batchify_fn=None, num_workers=0, pin_memory=False, pin_device_id=0,
                 prefetch=None, thread_pool=False, timeout=120, try_nopython=None, **kwargs):
        assert path_imgrec or path_imglist or isinstance(imglist, list)
        assert dtype in ('int32', 'float32', 'int64', 'float64'), dtype + ' label not supported'
        dataset = _shard(_dataset(path_imgrec, path_imglist, path_root, imglist, type(self).__name__), num_parts, part_index)
        if aug_list is None:
            augmenter = create_bbox_augment(data_shape, **kwargs)
        elif isinstance(aug_list, list):
            augmenter = _PairSequential(aug_list)
        elif isinstance(aug_list, _block.Block):
            augmenter = aug_list
        else:
            raise ValueError('aug_list must be a list of Blocks or Block')
        to_boxes = BboxLabelTransform(coord_normalized)

        def pipeline(img, label):
            img, boxes = to_boxes(img, label)
            return augmenter(img, boxes)
        self._iter = DataLoader(dataset.transform(pipeline), batch_size=batch_size, shuffle=shuffle, sampler=sampler,
                                last_batch=last_batch, batch_sampler=batch_sampler, batchify_fn=batchify_fn or _pad_boxes_batchify,
                                num_workers=num_workers, pin_memory=pin_memory, pin_device_id=pin_device_id, prefetch=prefetch,
                                thread_pool=thread_pool, timeout=timeout)

    def __iter__(self):
        return iter(self._iter)

    def __len__(self):
        return len(self._iter)

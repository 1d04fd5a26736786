"""Image transforms (``python/mxnet/gluon/data/vision/transforms``) as Blocks over HWC arrays."""
import random

import numpy as np

from ....ops import registry as _reg
from ...block import Block, HybridBlock
from ...nn import Sequential, HybridSequential

__all__ = ['Compose', 'HybridCompose', 'Cast', 'ToTensor', 'Normalize', 'Resize', 'CenterCrop', 'RandomResizedCrop',
           'RandomCrop', 'CropResize', 'RandomFlipLeftRight', 'RandomFlipTopBottom', 'RandomBrightness',
           'RandomContrast', 'RandomSaturation', 'RandomHue', 'RandomColorJitter', 'RandomLighting', 'RandomApply',
           'HybridRandomApply', 'RandomGray', 'RandomRotation', 'Rotate']


def _op(name, arrays, **attrs):
    return _reg.invoke(name, arrays, attrs)


class Compose(Sequential):
    def __init__(self, transforms):
        super().__init__()
        for t in transforms:
            self.add(t)


class HybridCompose(HybridSequential):
    def __init__(self, transforms):
        super().__init__()
        for t in transforms:
            self.add(t)


class Cast(HybridBlock):
    def __init__(self, dtype='float32'):
        super().__init__()
        self._dtype = dtype

    def forward(self, x):
        return x.astype(self._dtype)


class ToTensor(HybridBlock):
    def forward(self, x):
        return _op('_image_to_tensor', [x])


class Normalize(HybridBlock):
    def __init__(self, mean=0.0, std=1.0):
        super().__init__()
        self._mean = mean if isinstance(mean, (tuple, list)) else (mean,)
        self._std = std if isinstance(std, (tuple, list)) else (std,)

    def forward(self, x):
        return _op('_image_normalize', [x], mean=tuple(self._mean), std=tuple(self._std))


class Resize(HybridBlock):
    def __init__(self, size, keep_ratio=False, interpolation=1):
        super().__init__()
        self._size, self._keep, self._interpolation = size, keep_ratio, interpolation

    def forward(self, x):
        size = self._size if isinstance(self._size, (tuple, list)) else (self._size, self._size)
        return _op('_image_resize', [x], size=tuple(size), keep_ratio=self._keep, interp=self._interpolation)


class CropResize(HybridBlock):
    def __init__(self, x, y, width, height, size=None, interpolation=None):
        super().__init__()
        self._x, self._y, self._width, self._height, self._size, self._interpolation = x, y, width, height, size, interpolation

    def forward(self, x):
        out = _op('_image_crop', [x], x=self._x, y=self._y, width=self._width, height=self._height)
        if self._size:
            size = self._size if isinstance(self._size, (tuple, list)) else (self._size, self._size)
            out = _op('_image_resize', [out], size=tuple(size), interp=self._interpolation or 1)
        return out


class CenterCrop(Block):
    def __init__(self, size, interpolation=1):
        super().__init__()
        self._size = size if isinstance(size, (tuple, list)) else (size, size)
        self._interpolation = interpolation

    def forward(self, x):
        h, w = x.shape[-3], x.shape[-2]
        tw, th = self._size
        if tw > w or th > h:
            x = _op('_image_resize', [x], size=(max(tw, w), max(th, h)), interp=self._interpolation)
            h, w = x.shape[-3], x.shape[-2]
        x0, y0 = (w - tw) // 2, (h - th) // 2
        return _op('_image_crop', [x], x=x0, y=y0, width=tw, height=th)


class RandomCrop(Block):
    def __init__(self, size, pad=None, pad_value=0, interpolation=1):
        super().__init__()
        self._size = size if isinstance(size, (tuple, list)) else (size, size)
        self._pad, self._pad_value = pad, pad_value

    def forward(self, x):
        if self._pad:
            p = self._pad if isinstance(self._pad, (tuple, list)) else (self._pad,) * 4
            a = np.pad(x.asnumpy(), ((p[1], p[3]), (p[0], p[2]), (0, 0)), constant_values=self._pad_value)
            x = x.__class__(a, ctx=x.context, dtype=a.dtype)
        h, w = x.shape[-3], x.shape[-2]
        tw, th = self._size
        x0, y0 = random.randint(0, max(w - tw, 0)), random.randint(0, max(h - th, 0))
        return _op('_image_crop', [x], x=x0, y=y0, width=min(tw, w), height=min(th, h))


class RandomResizedCrop(Block):
    def __init__(self, size, scale=(0.08, 1.0), ratio=(3.0 / 4.0, 4.0 / 3.0), interpolation=1):
        super().__init__()
        self._size = size if isinstance(size, (tuple, list)) else (size, size)
        self._scale, self._ratio, self._interpolation = scale, ratio, interpolation

    def forward(self, x):
        import math
        h, w = x.shape[-3], x.shape[-2]
        area = h * w
        for _ in range(10):
            target = random.uniform(*self._scale) * area
            logr = (math.log(self._ratio[0]), math.log(self._ratio[1]))
            ar = math.exp(random.uniform(*logr))
            cw, ch = int(round(math.sqrt(target * ar))), int(round(math.sqrt(target / ar)))
            if 0 < cw <= w and 0 < ch <= h:
                x0, y0 = random.randint(0, w - cw), random.randint(0, h - ch)
                out = _op('_image_crop', [x], x=x0, y=y0, width=cw, height=ch)
                return _op('_image_resize', [out], size=tuple(self._size), interp=self._interpolation)
        return _op('_image_resize', [CenterCrop(min(h, w))(x)], size=tuple(self._size), interp=self._interpolation)


class RandomFlipLeftRight(HybridBlock):
    def __init__(self, p=0.5):
        super().__init__()
        self.p = p

    def forward(self, x):
        return _op('_image_random_flip_left_right', [x], p=self.p)


class RandomFlipTopBottom(HybridBlock):
    def __init__(self, p=0.5):
        super().__init__()
        self.p = p

    def forward(self, x):
        return _op('_image_random_flip_top_bottom', [x], p=self.p)


def _jitter(opname, label):
    class _J(HybridBlock):
        def __init__(self, value):
            super().__init__()
            self._args = (max(0, 1 - value), 1 + value)

        def forward(self, x):
            return _op(opname, [x], min_factor=self._args[0], max_factor=self._args[1])
    _J.__name__ = label
    return _J


RandomBrightness = _jitter('_image_random_brightness', 'RandomBrightness')
RandomContrast = _jitter('_image_random_contrast', 'RandomContrast')
RandomSaturation = _jitter('_image_random_saturation', 'RandomSaturation')
RandomHue = _jitter('_image_random_hue', 'RandomHue')


class RandomColorJitter(HybridBlock):
    def __init__(self, brightness=0, contrast=0, saturation=0, hue=0):
        super().__init__()
        self._args = dict(brightness=brightness, contrast=contrast, saturation=saturation, hue=hue)

    def forward(self, x):
        return _op('_image_random_color_jitter', [x], **self._args)


class RandomLighting(HybridBlock):
    def __init__(self, alpha):
        super().__init__()
        self._alpha = alpha

    def forward(self, x):
        return _op('_image_random_lighting', [x], alpha_std=self._alpha)


class RandomApply(Sequential):
    def __init__(self, transforms, p=0.5):
        super().__init__()
        self.transforms, self.p = transforms, p

    def forward(self, x):
        if self.p < random.random():
            return x
        return self.transforms(x)


class HybridRandomApply(HybridSequential):
    def __init__(self, transforms, p=0.5):
        super().__init__()
        self.transforms, self.p = transforms, p

    def forward(self, x):
        if self.p < random.random():
            return x
        return self.transforms(x)


class RandomGray(HybridBlock):
    def __init__(self, p=0.5):
        super().__init__()
        self.p = p

    def forward(self, x):
        if random.random() >= self.p:
            return x
        import torch
        coef = torch.tensor([0.299, 0.587, 0.114], device=x._data.device)
        if x.shape[-1] == 3:
            g = (x._data.float() * coef).sum(-1, keepdim=True).expand_as(x._data)
        else:
            g = (x._data.float() * coef.view(3, 1, 1)).sum(-3, keepdim=True).expand_as(x._data)
        return x.__class__._from_tensor(g.to(x._data.dtype).contiguous(), x.context)


class Rotate(Block):
    def __init__(self, rotation_degrees, zoom_in=False, zoom_out=False):
        super().__init__()
        self._deg, self._zoom_in, self._zoom_out = rotation_degrees, zoom_in, zoom_out

    def forward(self, x):
        import math
        import torch
        import torch.nn.functional as F
        t = x._data.float()
        chw = t if t.dim() == 3 else t
        batch = chw[None] if chw.dim() == 3 else chw
        a = math.radians(self._deg)
        theta = torch.tensor([[math.cos(a), -math.sin(a), 0.0], [math.sin(a), math.cos(a), 0.0]], device=t.device)
        grid = F.affine_grid(theta[None].expand(batch.shape[0], 2, 3), batch.shape, align_corners=False)
        out = F.grid_sample(batch, grid, align_corners=False)
        out = out[0] if chw.dim() == 3 else out
        return x.__class__._from_tensor(out.to(x._data.dtype), x.context)


class RandomRotation(Block):
    def __init__(self, angle_limits, zoom_in=False, zoom_out=False, rotate_with_proba=1.0):
        super().__init__()
        self._lim, self._p = angle_limits, rotate_with_proba
        self._zoom_in, self._zoom_out = zoom_in, zoom_out

    def forward(self, x):
        if random.random() > self._p:
            return x
        return Rotate(random.uniform(*self._lim), self._zoom_in, self._zoom_out)(x)

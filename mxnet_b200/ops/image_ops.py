"""Image operators (``src/operator/image/*``: to_tensor, normalize, crop, resize, flips, colour jitter)."""
from __future__ import annotations

import random as _pyrandom

import torch
import torch.nn.functional as F

from .registry import register


@register('_image_to_tensor', '_npx__image_to_tensor', inputs=('data',))
def to_tensor(data):
    x = data.float() / 255.0
    return x.permute(2, 0, 1) if x.dim() == 3 else x.permute(0, 3, 1, 2)


@register('_image_normalize', '_npx__image_normalize', inputs=('data',), defaults={'mean': (0.0,), 'std': (1.0,)})
def normalize(data, mean=(0.0,), std=(1.0,)):
    c = data.shape[-3]
    m = torch.as_tensor(mean, dtype=data.dtype, device=data.device).reshape(-1, 1, 1)
    s = torch.as_tensor(std, dtype=data.dtype, device=data.device).reshape(-1, 1, 1)
    if m.shape[0] == 1:
        m = m.expand(c, 1, 1)
    if s.shape[0] == 1:
        s = s.expand(c, 1, 1)
    return (data - m) / s


@register('_image_crop', '_npx__image_crop', inputs=('data',), defaults={'x': 0, 'y': 0, 'width': 1, 'height': 1})
def crop(data, x=0, y=0, width=1, height=1):
    return data[..., y:y + height, x:x + width, :]


@register('_image_resize', '_npx__image_resize', inputs=('data',), defaults={'size': (), 'keep_ratio': False, 'interp': 1})
def resize(data, size=(), keep_ratio=False, interp=1):
    if isinstance(size, int):
        size = (size, size)
    w, h = (size[0], size[1]) if len(size) == 2 else (size[0], size[0])
    batched = data.dim() == 4
    x = data if batched else data[None]
    H, W = x.shape[1], x.shape[2]
    if keep_ratio:
        if H > W:
            h, w = int(size[0] * H / W), size[0]
        else:
            h, w = size[0], int(size[0] * W / H)
    xf = x.permute(0, 3, 1, 2).float()
    mode = {0: 'nearest', 1: 'bilinear', 2: 'bicubic', 3: 'area'}.get(interp, 'bilinear')
    kw = {} if mode in ('nearest', 'area') else {'align_corners': False}
    y = F.interpolate(xf, size=(h, w), mode=mode, **kw)
    if data.dtype == torch.uint8:
        y = y.round().clamp(0, 255)
    y = y.to(data.dtype).permute(0, 2, 3, 1)
    return y if batched else y[0]


@register('_image_flip_left_right', '_npx__image_flip_left_right', inputs=('data',))
def flip_left_right(data):
    return torch.flip(data, (-2,))


@register('_image_flip_top_bottom', '_npx__image_flip_top_bottom', inputs=('data',))
def flip_top_bottom(data):
    return torch.flip(data, (-3,))


@register('_image_random_flip_left_right', '_npx__image_random_flip_left_right', inputs=('data',), defaults={'p': 0.5})
def random_flip_left_right(data, p=0.5):
    return torch.flip(data, (-2,)) if _pyrandom.random() < p else data


@register('_image_random_flip_top_bottom', '_npx__image_random_flip_top_bottom', inputs=('data',), defaults={'p': 0.5})
def random_flip_top_bottom(data, p=0.5):
    return torch.flip(data, (-3,)) if _pyrandom.random() < p else data


def _gray(x):
    coef = torch.tensor([0.299, 0.587, 0.114], dtype=torch.float32, device=x.device)
    return (x.float() * coef).sum(-1, keepdim=True)


def _blend(a, b, alpha, dtype):
    y = a.float() * alpha + b * (1 - alpha)
    if dtype == torch.uint8:
        y = y.clamp(0, 255)
    return y.to(dtype)


@register('_image_adjust_lighting', '_npx__image_adjust_lighting', inputs=('data',), defaults={'alpha': (0.0, 0.0, 0.0)})
def adjust_lighting(data, alpha=(0.0, 0.0, 0.0)):
    eigval = torch.tensor([55.46, 4.794, 1.148])
    eigvec = torch.tensor([[-0.5675, 0.7192, 0.4009], [-0.5808, -0.0045, -0.8140], [-0.5836, -0.6948, 0.4203]])
    rgb = (eigvec * torch.tensor(alpha) * eigval).sum(1).to(data.device)
    return _blend(data.float() + rgb, 0, 1.0, data.dtype)


@register('_image_random_brightness', '_npx__image_random_brightness', inputs=('data',), defaults={'min_factor': 1.0, 'max_factor': 1.0})
def random_brightness(data, min_factor=1.0, max_factor=1.0):
    return _blend(data, 0, _pyrandom.uniform(min_factor, max_factor), data.dtype)


@register('_image_random_contrast', '_npx__image_random_contrast', inputs=('data',), defaults={'min_factor': 1.0, 'max_factor': 1.0})
def random_contrast(data, min_factor=1.0, max_factor=1.0):
    return _blend(data, _gray(data).mean(), _pyrandom.uniform(min_factor, max_factor), data.dtype)


@register('_image_random_saturation', '_npx__image_random_saturation', inputs=('data',), defaults={'min_factor': 1.0, 'max_factor': 1.0})
def random_saturation(data, min_factor=1.0, max_factor=1.0):
    return _blend(data, _gray(data), _pyrandom.uniform(min_factor, max_factor), data.dtype)


@register('_image_random_hue', '_npx__image_random_hue', inputs=('data',), defaults={'min_factor': 1.0, 'max_factor': 1.0})
def random_hue(data, min_factor=1.0, max_factor=1.0):
    import math
    a = _pyrandom.uniform(min_factor, max_factor) - 1.0
    u, w = math.cos(a * math.pi), math.sin(a * math.pi)
    t_yiq = torch.tensor([[0.299, 0.587, 0.114], [0.596, -0.274, -0.321], [0.211, -0.523, 0.311]])
    t_rgb = torch.tensor([[1.0, 0.956, 0.621], [1.0, -0.272, -0.647], [1.0, -1.107, 1.705]])
    rot = torch.tensor([[1.0, 0.0, 0.0], [0.0, u, -w], [0.0, w, u]])
    m = (t_rgb @ rot @ t_yiq).t().to(data.device)
    return _blend(data.float() @ m, 0, 1.0, data.dtype)


@register('_image_random_color_jitter', '_npx__image_random_color_jitter', inputs=('data',),
          defaults={'brightness': 0.0, 'contrast': 0.0, 'saturation': 0.0, 'hue': 0.0})
def random_color_jitter(data, brightness=0.0, contrast=0.0, saturation=0.0, hue=0.0):
    ops = []
    if brightness > 0:
        ops.append(lambda x: random_brightness(x, 1 - brightness, 1 + brightness))
    if contrast > 0:
        ops.append(lambda x: random_contrast(x, 1 - contrast, 1 + contrast))
    if saturation > 0:
        ops.append(lambda x: random_saturation(x, 1 - saturation, 1 + saturation))
    if hue > 0:
        ops.append(lambda x: random_hue(x, 1 - hue, 1 + hue))
    _pyrandom.shuffle(ops)
    for f in ops:
        data = f(data)
    return data


@register('_image_random_lighting', '_npx__image_random_lighting', inputs=('data',), defaults={'alpha_std': 0.05})
def random_lighting(data, alpha_std=0.05):
    return adjust_lighting(data, tuple(_pyrandom.gauss(0, alpha_std) for _ in range(3)))


@register('_cvimresize', inputs=('data',), defaults={'w': 1, 'h': 1, 'interp': 1})
def cvimresize(data, w=1, h=1, interp=1):
    return resize(data, (w, h), False, interp)


@register('_cvcopyMakeBorder', inputs=('data',), defaults={'top': 0, 'bot': 0, 'left': 0, 'right': 0, 'type': 0, 'value': 0.0})
def cv_copy_make_border(data, top=0, bot=0, left=0, right=0, type=0, value=0.0, values=None):
    x = data.permute(2, 0, 1)[None].float()
    y = F.pad(x, (left, right, top, bot), 'constant', value)
    return y[0].permute(1, 2, 0).to(data.dtype)


# ---- random crops and the file / buffer decoders as operators (image/crop.cc, io/image_io.cc) -----------------------
@register('_image_random_crop', '_npx__image_random_crop', inputs=('data',), nout=1,
          defaults={'xrange': (0.0, 1.0), 'yrange': (0.0, 1.0), 'width': 1, 'height': 1, 'interp': 1})
def random_crop(data, xrange=(0.0, 1.0), yrange=(0.0, 1.0), width=1, height=1, interp=1):   # pylint: disable=redefined-builtin
    """Crop of ``width`` x ``height`` whose left / top edge is drawn uniformly from the given fractions of the free
    range; images smaller than the crop are resized up to it.  Layout (H, W, C) or (N, H, W, C)."""
    import random as _pyrandom
    h, w = data.shape[-3], data.shape[-2]
    if h < height or w < width:
        return resize(data, size=(width, height), interp=interp)
    x0 = int(round((xrange[0] + (xrange[1] - xrange[0]) * _pyrandom.random()) * (w - width)))
    y0 = int(round((yrange[0] + (yrange[1] - yrange[0]) * _pyrandom.random()) * (h - height)))
    return crop(data, x=x0, y=y0, width=width, height=height)


@register('_image_random_resized_crop', '_npx__image_random_resized_crop', inputs=('data',),
          defaults={'width': 1, 'height': 1, 'area': (0.08, 1.0), 'ratio': (3.0 / 4.0, 4.0 / 3.0), 'interp': 1, 'max_trial': 10})
def random_resized_crop(data, width=1, height=1, area=(0.08, 1.0), ratio=(3.0 / 4.0, 4.0 / 3.0), interp=1, max_trial=10):
    """A crop of random area (fraction of the image) and aspect ratio, resized to ``width`` x ``height``; after
    ``max_trial`` failed draws the centre crop of the target aspect ratio is used."""
    import math
    import random as _pyrandom
    h, w = data.shape[-3], data.shape[-2]
    area = (area, 1.0) if isinstance(area, (int, float)) else tuple(area)
    for _ in range(int(max_trial)):
        target = _pyrandom.uniform(*area) * h * w
        log_ratio = (math.log(ratio[0]), math.log(ratio[1]))
        aspect = math.exp(_pyrandom.uniform(*log_ratio))
        cw, ch = int(round(math.sqrt(target * aspect))), int(round(math.sqrt(target / aspect)))
        if 0 < cw <= w and 0 < ch <= h:
            x0, y0 = _pyrandom.randint(0, w - cw), _pyrandom.randint(0, h - ch)
            return resize(crop(data, x=x0, y=y0, width=cw, height=ch), size=(width, height), interp=interp)
    scale = min(w / width, h / height)
    cw, ch = int(width * scale), int(height * scale)
    return resize(crop(data, x=(w - cw) // 2, y=(h - ch) // 2, width=cw, height=ch), size=(width, height), interp=interp)


@register('_cvimdecode', inputs=('buf',), defaults={'flag': 1, 'to_rgb': True})
def cvimdecode(buf, flag=1, to_rgb=True):
    """Encoded image bytes (a uint8 vector) -> (H, W, C) uint8 image."""
    from ..image.image import _decode_to_numpy
    return torch.from_numpy(_decode_to_numpy(buf.detach().cpu().numpy().tobytes(), flag, to_rgb).copy())


@register('_cvimread', inputs=(), defaults={'filename': '', 'flag': 1, 'to_rgb': True})
def cvimread(filename='', flag=1, to_rgb=True):
    from ..image.image import _decode_to_numpy
    with open(filename, 'rb') as f:
        return torch.from_numpy(_decode_to_numpy(f.read(), flag, to_rgb).copy())

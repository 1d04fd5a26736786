"""NHWC max pooling on the sm_100a kernels (``pool.cu``)."""
import torch

from . import lib, ptr, stream_ptr, count_launch, check
from ._util import dt, require


def out_size(n, k, s, p, ceil_mode):
    """Output extent of one axis ('valid' = floor, 'full' = ceil; the last window must start inside
    the padded input, pooling-inl.h:118-180)."""
    span = n + 2 * p - k
    o = (-(-span // s) if ceil_mode else span // s) + 1
    if ceil_mode and (o - 1) * s >= n + p:
        o -= 1
    return o


def supported(x, kernel, stride, pad):
    return (x.dim() == 4 and x.dtype in (torch.float16, torch.bfloat16) and x.is_contiguous() and x.shape[-1] % 8 == 0
            and x.numel() > 0 and kernel[0] * kernel[1] <= 127 and pad[0] < kernel[0] and pad[1] < kernel[1])


class _MaxPoolNHWC(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, kernel, stride, pad, ceil_mode):
        require(x, 'data')
        n, h, w, c = x.shape
        ho = out_size(h, kernel[0], stride[0], pad[0], ceil_mode)
        wo = out_size(w, kernel[1], stride[1], pad[1], ceil_mode)
        y = torch.empty((n, ho, wo, c), dtype=x.dtype, device=x.device)
        idx = torch.empty((n, ho, wo, c), dtype=torch.int8, device=x.device)
        check(lib().mxb_maxpool_forward(dt(x), ptr(x), ptr(y), ptr(idx), n, h, w, c, ho, wo, kernel[0], kernel[1],
                                        stride[0], stride[1], pad[0], pad[1], stream_ptr(x.device)), 'maxpool_forward')
        count_launch(1)
        ctx.save_for_backward(idx)
        ctx.geom = (n, h, w, c, ho, wo, kernel, stride, pad)
        return y

    @staticmethod
    def backward(ctx, dy):
        idx, = ctx.saved_tensors
        n, h, w, c, ho, wo, kernel, stride, pad = ctx.geom
        dy = require(dy.contiguous(), 'out_grad', device=idx.device, shape=(n, ho, wo, c))
        dx = torch.empty((n, h, w, c), dtype=dy.dtype, device=dy.device)
        check(lib().mxb_maxpool_backward(dt(dy), ptr(dy), ptr(idx), ptr(dx), n, h, w, c, ho, wo, kernel[0], kernel[1],
                                         stride[0], stride[1], pad[0], pad[1], stream_ptr(dy.device)), 'maxpool_backward')
        count_launch(1)
        return dx, None, None, None, None


def max_pool2d_nhwc(x, kernel, stride, pad, ceil_mode=False):
    return _MaxPoolNHWC.apply(x, tuple(kernel), tuple(stride), tuple(pad), bool(ceil_mode))

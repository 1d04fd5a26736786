"""NHWC convolution on the sm_100a kernels.

1x1 stride-1 convolutions are GEMMs over the flattened pixels ([N*H*W, Cin] x [Cout, Cin]^T) and run on
the tcgen05 kernel when ``MXNET_B200_CONV1X1=1``; other shapes go to the library convolution on a
channels-last view (no layout copies)."""
import os

import torch

from . import gemm_ops


def supported(data, weight, stride, dilate, pad, num_group):
    if os.environ.get('MXNET_B200_CONV1X1', '0') != '1':
        return False
    if data.dtype not in (torch.float16, torch.bfloat16) or num_group != 1:
        return False
    kh, kw = weight.shape[1], weight.shape[2]
    if (kh, kw) != (1, 1) or tuple(stride) != (1, 1) or tuple(pad) != (0, 0) or tuple(dilate) != (1, 1):
        return False
    return data.is_contiguous() and gemm_ops.supported(data.numel() // data.shape[-1], weight.shape[0], data.shape[-1])


def conv2d_nhwc(data, weight, bias, stride, pad):
    n, h, w, c = data.shape
    cout = weight.shape[0]
    y = gemm_ops.LinearFn.apply(data.reshape(-1, c), weight.reshape(cout, c), bias, None)
    return y.reshape(n, h, w, cout)

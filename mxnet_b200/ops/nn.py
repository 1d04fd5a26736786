"""Neural-network operators with the reference's parameter schemas and semantics.

Reference: ``src/operator/nn/*`` (Convolution, FullyConnected, BatchNorm, LayerNorm, Pooling,
Activation, Dropout, softmax family …) and the legacy layer ops of ``src/operator/*.cc``
(SoftmaxOutput, regression outputs, RNN, UpSampling …).  Parameter names/defaults follow the
``dmlc::Parameter`` structs cited per operator so symbol JSON files round-trip.

CUDA tensors in half precision are routed to the sm_100a kernels of ``ops/cuda`` for the fused
hot paths (BatchNorm(+ReLU+add) in NHWC, LayerNorm, softmax/cross-entropy, FullyConnected GEMM
with bias/activation epilogue, fused LSTM cell).  The CPU and long-tail implementations double
as the numerical oracle of those kernels.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from .registry import register, alias
from .. import _state, env
from ..base import MXNetError, to_torch_dtype
from . import gemm as _gemm


def _use_kernels(t):
    if not t.is_cuda or not env.get('MXNET_B200_KERNELS'):
        return False
    from . import cuda
    return cuda.available()


def _use_ew(t):
    """The pointwise / gather / pooling vector kernels (``MXNET_B200_ELEMENTWISE``)."""
    return env.get('MXNET_B200_ELEMENTWISE') and _use_kernels(t)


def _tup(v, n):
    if v is None or v == ():
        return None
    if isinstance(v, int):
        return (v,) * n
    return tuple(int(x) for x in v)


# ------------------------------------------------------------------------------------------
# FullyConnected  (src/operator/nn/fully_connected-inl.h:77-81)
# ------------------------------------------------------------------------------------------
@register('FullyConnected', '_npx_fully_connected', inputs=('data', 'weight', 'bias'),
          defaults={'num_hidden': 0, 'no_bias': False, 'flatten': True})
def fully_connected(data, weight, bias=None, num_hidden=None, no_bias=False, flatten=True):
    if no_bias:
        bias = None
    if flatten:
        x = data.reshape(data.shape[0], -1) if data.dim() != 2 else data
        return _gemm.linear(x, weight, bias)
    lead = data.shape[:-1]
    y = _gemm.linear(data.reshape(-1, data.shape[-1]), weight, bias)
    return y.reshape(tuple(lead) + (weight.shape[0],))


# ------------------------------------------------------------------------------------------
# Convolution / Deconvolution (src/operator/nn/convolution-inl.h:60-110)
# ------------------------------------------------------------------------------------------
_CHANNEL_LAST = ('NWC', 'NHWC', 'NDHWC')


def _to_channel_first(x, layout):
    """Channel-last logical layout → channel-first *view* (channels_last strides, no copy)."""
    if layout in _CHANNEL_LAST:
        nd = x.dim()
        return x.permute(0, nd - 1, *range(1, nd - 1))
    return x


def _to_layout(y, layout):
    if layout in _CHANNEL_LAST:
        nd = y.dim()
        return y.permute(0, *range(2, nd), 1)
    return y


@register('Convolution', '_npx_convolution', inputs=('data', 'weight', 'bias'),
          defaults={'kernel': (), 'stride': (), 'dilate': (), 'pad': (), 'num_filter': 0, 'num_group': 1,
                    'workspace': 1024, 'no_bias': False, 'cudnn_tune': None, 'cudnn_off': False, 'layout': None})
def convolution(data, weight, bias=None, kernel=(), stride=(), dilate=(), pad=(), num_filter=0, num_group=1,
                workspace=1024, no_bias=False, cudnn_tune=None, cudnn_off=False, layout=None):
    nsp = data.dim() - 2
    stride = _tup(stride, nsp) or (1,) * nsp
    dilate = _tup(dilate, nsp) or (1,) * nsp
    pad = _tup(pad, nsp) or (0,) * nsp
    if no_bias:
        bias = None
    if layout in _CHANNEL_LAST and nsp == 2 and _use_kernels(data):
        from .cuda import conv_ops
        if conv_ops.supported(data, weight, stride, dilate, pad, num_group):
            return conv_ops.conv2d_nhwc(data, weight, bias, stride, pad, dilate)
    x = _to_channel_first(data, layout)
    w = _to_channel_first(weight, layout)
    fn = (F.conv1d, F.conv2d, F.conv3d)[nsp - 1]
    y = fn(x, w, bias, stride, pad, dilate, num_group)
    return _to_layout(y, layout)


@register('_contrib_conv_skip', inputs=('data', 'weight'),
          defaults={'kernel': (), 'stride': (), 'dilate': (), 'pad': (), 'num_filter': 0, 'num_group': 1, 'layout': None})
def conv_skip(data, weight, kernel=(), stride=(), dilate=(), pad=(), num_filter=0, num_group=1, layout=None):
    """``(Convolution(data, weight, no_bias=True), data)``: the first convolution of an identity residual block together
    with the skip connection that starts at the same tensor.  Mathematically the second output is the input; as one
    operator its gradient node receives the gradients of both branches at once, and on the GPU kernels the data gradient
    adds the skip gradient in its epilogue (the reference sums the two branches with a separate ElementWiseSum,
    src/nnvm/gradient.cc)."""
    nsp = data.dim() - 2
    stride = _tup(stride, nsp) or (1,) * nsp
    dilate = _tup(dilate, nsp) or (1,) * nsp
    pad = _tup(pad, nsp) or (0,) * nsp
    if layout in _CHANNEL_LAST and nsp == 2 and tuple(stride) == (1, 1) and _use_kernels(data):
        from .cuda import conv_ops
        if conv_ops.supported(data, weight, stride, dilate, pad, num_group):
            return conv_ops.conv2d_skip_nhwc(data, weight, pad, dilate)
    y = convolution(data, weight, None, kernel, stride, dilate, pad, num_filter, num_group, no_bias=True, layout=layout)
    return y, data


@register('Deconvolution', '_npx_deconvolution', inputs=('data', 'weight', 'bias'),
          defaults={'kernel': (), 'stride': (), 'dilate': (), 'pad': (), 'adj': (), 'target_shape': (),
                    'num_filter': 0, 'num_group': 1, 'workspace': 512, 'no_bias': True, 'cudnn_tune': None,
                    'cudnn_off': False, 'layout': None})
def deconvolution(data, weight, bias=None, kernel=(), stride=(), dilate=(), pad=(), adj=(), target_shape=(),
                  num_filter=0, num_group=1, workspace=512, no_bias=True, cudnn_tune=None, cudnn_off=False,
                  layout=None):
    nsp = data.dim() - 2
    stride = _tup(stride, nsp) or (1,) * nsp
    dilate = _tup(dilate, nsp) or (1,) * nsp
    pad = _tup(pad, nsp) or (0,) * nsp
    adj = _tup(adj, nsp) or (0,) * nsp
    if no_bias:
        bias = None
    x = _to_channel_first(data, layout)
    w = _to_channel_first(weight, layout)
    if target_shape:
        tgt = _tup(target_shape, nsp)
        k = w.shape[2:]
        in_sp = x.shape[2:]
        pad, adj = list(pad), list(adj)
        for i in range(nsp):
            total = stride[i] * (in_sp[i] - 1) + dilate[i] * (k[i] - 1) + 1
            diff = total - tgt[i]
            pad[i] = (diff + 1) // 2 if diff > 0 else 0
            adj[i] = tgt[i] - (total - 2 * pad[i])
        pad, adj = tuple(pad), tuple(adj)
    fn = (F.conv_transpose1d, F.conv_transpose2d, F.conv_transpose3d)[nsp - 1]
    y = fn(x, w, bias, stride, pad, adj, num_group, dilate)
    return _to_layout(y, layout)


# ------------------------------------------------------------------------------------------
# BatchNorm (src/operator/nn/batch_norm-inl.h:100-127)
# ------------------------------------------------------------------------------------------
def _bn_nout(attrs):
    return 3 if attrs.get('output_mean_var') in (True, 'True', 1) else 1


def _fused_bn_training(x, gamma, beta, eps):
    """(y, batch mean, 1 / sqrt(batch variance + eps)) of a channel-first tensor with one of the library's fused kernels:
    the cuDNN normalisation for dense 4-D / 5-D fp32 and fp16 CUDA tensors (its backward pass is several times faster than
    the generic kernel's on NCHW data), the generic fused kernel otherwise."""
    # (the size limits are the tensor library's own conditions for choosing this path)
    if x.is_cuda and x.dim() in (4, 5) and x.dtype in (torch.float32, torch.float16) and eps >= 1e-5 and \
            torch.backends.cudnn.enabled and 0 < x.numel() < (1 << 31) and x.shape[0] <= 880801 and \
            (x.is_contiguous() or (x.dim() == 4 and x.is_contiguous(memory_format=torch.channels_last))):
        w, b = (gamma.float(), beta.float()) if gamma.dtype != torch.float32 else (gamma, beta)
        try:
            y, mean, invstd, _ = torch.cudnn_batch_norm(x, w, b, None, None, True, 0.0, eps)
            return y, mean, invstd
        except RuntimeError:
            pass                                # a shape the library's cuDNN path refuses: the generic kernel takes it
    return torch.native_batch_norm(x, gamma, beta, None, None, True, 0.0, eps)


@register('BatchNorm', '_npx_batch_norm', 'BatchNorm_v1', inputs=('data', 'gamma', 'beta', 'moving_mean', 'moving_var', 'residual'),
          nout=_bn_nout, aux=('moving_mean', 'moving_var'),
          defaults={'eps': 1e-3, 'momentum': 0.9, 'fix_gamma': True, 'use_global_stats': False,
                    'output_mean_var': False, 'axis': 1, 'cudnn_off': False})
def batch_norm(data, gamma, beta, moving_mean, moving_var, residual=None, eps=1e-3, momentum=0.9, fix_gamma=True,
               use_global_stats=False, output_mean_var=False, axis=1, cudnn_off=False,
               min_calib_range=None, max_calib_range=None, act_type=None):
    """Batch normalisation; ``act_type``/``residual`` select the fused BN(+add)+ReLU form used by
    the NHWC ResNet blocks (one pass over the activations instead of three)."""
    axis = axis % data.dim()
    training = _state.state.training and not use_global_stats
    if fix_gamma:
        gamma = torch.ones_like(gamma)
    if axis == data.dim() - 1 and data.dim() == 4 and _use_kernels(data) and \
            data.dtype in (torch.float16, torch.bfloat16) and data.is_contiguous():
        from .cuda import norm_ops
        if norm_ops.bn_supported(data) and moving_mean.dtype == torch.float32 and moving_var.dtype == torch.float32 \
                and moving_mean.is_contiguous() and moving_var.is_contiguous():
            out, mean, var = norm_ops.batch_norm_nhwc(data, gamma, beta, moving_mean, moving_var, eps, momentum,
                                                      training, act_type, residual, want_stats=bool(output_mean_var))
            return (out, mean, var) if output_mean_var else out
    if not output_mean_var and data.dim() >= 2 and data.is_floating_point() and data.dtype != torch.float64 and \
            gamma.dtype == beta.dtype and gamma.dtype in (data.dtype, torch.float32):
        # every other layout / precision: the tensor library's fused normalisation (one statistics pass and one apply pass,
        # fused backward) on a channel-first view.  The running statistics are updated here, from the saved batch moments,
        # with the population variance as the reference does (src/operator/nn/batch_norm.cc); the library's own update would
        # use the sample variance.
        x = data if axis == 1 else data.movedim(axis, 1)
        if training:
            y, mean, invstd = _fused_bn_training(x, gamma, beta, eps)
            with torch.no_grad():
                var = invstd.float().pow(-2).sub_(eps).clamp_(min=0.0)
                moving_mean.mul_(momentum).add_(mean.to(moving_mean.dtype), alpha=1 - momentum)
                moving_var.mul_(momentum).add_(var.to(moving_var.dtype), alpha=1 - momentum)
        else:
            stat_dtype = torch.float32 if data.dtype in (torch.float16, torch.bfloat16) else data.dtype
            y = torch.native_batch_norm(x, gamma, beta, moving_mean.to(stat_dtype), moving_var.to(stat_dtype), False, 0.0, eps)[0]
        if axis != 1:
            y = y.movedim(1, axis)
        if residual is not None:
            y = y + residual.to(y.dtype)
        if act_type == 'relu':
            y = torch.relu(y)
        return y
    red = tuple(i for i in range(data.dim()) if i != axis)
    shape = [1] * data.dim()
    shape[axis] = data.shape[axis]
    xf = data.float() if data.dtype in (torch.float16, torch.bfloat16) else data
    if training:
        mean = xf.mean(red)
        var = xf.var(red, unbiased=False)
        with torch.no_grad():
            moving_mean.mul_(momentum).add_(mean.detach().to(moving_mean.dtype), alpha=1 - momentum)
            moving_var.mul_(momentum).add_(var.detach().to(moving_var.dtype), alpha=1 - momentum)
    else:
        mean, var = moving_mean.to(xf.dtype), moving_var.to(xf.dtype)
    inv = torch.rsqrt(var + eps)
    y = (xf - mean.reshape(shape)) * (inv * gamma.to(xf.dtype)).reshape(shape) + beta.to(xf.dtype).reshape(shape)
    if residual is not None:
        y = y + residual.to(y.dtype)
    if act_type == 'relu':
        y = torch.relu(y)
    y = y.to(data.dtype)
    if output_mean_var:
        return y, mean, var
    return y


@register('SyncBatchNorm', '_contrib_SyncBatchNorm', inputs=('data', 'gamma', 'beta', 'moving_mean', 'moving_var'),
          nout=_bn_nout, aux=('moving_mean', 'moving_var'),
          defaults={'eps': 1e-3, 'momentum': 0.9, 'fix_gamma': True, 'use_global_stats': False,
                    'output_mean_var': False, 'ndev': 1, 'key': ''})
def sync_batch_norm(data, gamma, beta, moving_mean, moving_var, eps=1e-3, momentum=0.9, fix_gamma=True,
                    use_global_stats=False, output_mean_var=False, ndev=1, key='', axis=1):
    """Cross-device BatchNorm (``src/operator/contrib/sync_batch_norm-inl.h``): batch statistics are
    all-reduced over the data-parallel group (one process per GPU) before normalisation."""
    from ..parallel import dist
    training = _state.state.training and not use_global_stats
    if not training or not dist.is_initialized() or dist.world_size() == 1:
        return batch_norm(data, gamma, beta, moving_mean, moving_var, None, eps, momentum, fix_gamma,
                          use_global_stats, output_mean_var, axis)
    if fix_gamma:
        gamma = torch.ones_like(gamma)
    red = tuple(i for i in range(data.dim()) if i != axis)
    shape = [1] * data.dim()
    shape[axis] = data.shape[axis]
    xf = data.float()
    mean, var = dist.SyncMoments.apply(xf, red)
    with torch.no_grad():
        moving_mean.mul_(momentum).add_(mean.detach(), alpha=1 - momentum)
        moving_var.mul_(momentum).add_(var.detach(), alpha=1 - momentum)
    y = (xf - mean.reshape(shape)) * (torch.rsqrt(var + eps) * gamma.float()).reshape(shape) + beta.float().reshape(shape)
    y = y.to(data.dtype)
    return (y, mean, var) if output_mean_var else y


# ------------------------------------------------------------------------------------------
# LayerNorm / GroupNorm / InstanceNorm
# ------------------------------------------------------------------------------------------
@register('LayerNorm', '_npx_layer_norm', inputs=('data', 'gamma', 'beta'),
          nout=lambda a: 3 if a.get('output_mean_var') in (True, 'True', 1) else 1,
          defaults={'axis': -1, 'eps': 1e-5, 'output_mean_var': False})
def layer_norm(data, gamma, beta, axis=-1, eps=1e-5, output_mean_var=False):
    axis = axis % data.dim()
    if axis == data.dim() - 1 and not output_mean_var:
        if _use_kernels(data) and data.dtype in (torch.float16, torch.bfloat16, torch.float32) and data.is_contiguous():
            from .cuda import norm_ops
            if norm_ops.ln_supported(data):
                return norm_ops.layer_norm(data, gamma, beta, eps)
        return F.layer_norm(data, (data.shape[-1],), gamma, beta, eps)
    xf = data.float() if data.dtype in (torch.float16, torch.bfloat16) else data
    mean = xf.mean(axis, keepdim=True)
    var = xf.var(axis, unbiased=False, keepdim=True)
    std = torch.sqrt(var + eps)
    shape = [1] * data.dim()
    shape[axis] = data.shape[axis]
    y = ((xf - mean) / std * gamma.to(xf.dtype).reshape(shape) + beta.to(xf.dtype).reshape(shape)).to(data.dtype)
    if output_mean_var:
        return y, mean.squeeze(axis), std.squeeze(axis)
    return y


@register('GroupNorm', '_npx_group_norm', inputs=('data', 'gamma', 'beta'),
          nout=lambda a: 3 if a.get('output_mean_var') in (True, 'True', 1) else 1,
          defaults={'num_groups': 1, 'eps': 1e-5, 'output_mean_var': False})
def group_norm(data, gamma, beta, num_groups=1, eps=1e-5, output_mean_var=False):
    n, c = data.shape[0], data.shape[1]
    if not output_mean_var and data.is_floating_point() and gamma.numel() == c and beta.numel() == c:
        return F.group_norm(data, num_groups, gamma.to(data.dtype), beta.to(data.dtype), eps)     # fused forward and backward
    x = data.reshape(n, num_groups, -1)
    xf = x.float() if x.dtype in (torch.float16, torch.bfloat16) else x
    mean = xf.mean(-1, keepdim=True)
    var = xf.var(-1, unbiased=False, keepdim=True)
    std = torch.sqrt(var + eps)
    y = ((xf - mean) / std).reshape(data.shape)
    shape = [1, c] + [1] * (data.dim() - 2)
    y = (y * gamma.to(y.dtype).reshape(shape) + beta.to(y.dtype).reshape(shape)).to(data.dtype)
    if output_mean_var:
        return y, mean.reshape(n, num_groups), std.reshape(n, num_groups)
    return y


@register('InstanceNorm', '_npx_instance_norm', inputs=('data', 'gamma', 'beta'), defaults={'eps': 1e-3})
def instance_norm(data, gamma, beta, eps=1e-3):
    return F.instance_norm(data, weight=gamma, bias=beta, eps=eps)


@register('LRN', inputs=('data',), defaults={'alpha': 1e-4, 'beta': 0.75, 'knorm': 2.0, 'nsize': 5})
def lrn(data, alpha=1e-4, beta=0.75, knorm=2.0, nsize=5):
    return F.local_response_norm(data, nsize, alpha, beta, knorm)


# ------------------------------------------------------------------------------------------
# Pooling (src/operator/nn/pooling-inl.h:58-119)
# ------------------------------------------------------------------------------------------
@register('Pooling', '_npx_pooling', 'Pooling_v1', inputs=('data',),
          defaults={'kernel': (), 'pool_type': 'max', 'global_pool': False, 'cudnn_off': False,
                    'pooling_convention': 'valid', 'stride': (), 'pad': (), 'p_value': None,
                    'count_include_pad': None, 'layout': None})
def pooling(data, kernel=(), pool_type='max', global_pool=False, cudnn_off=False, pooling_convention='valid',
            stride=(), pad=(), p_value=None, count_include_pad=None, layout=None, output_size=None):
    nsp = data.dim() - 2
    if layout in _CHANNEL_LAST and nsp == 2 and pool_type == 'max' and not global_pool and _use_kernels(data) \
            and pooling_convention in ('valid', 'full'):
        from .cuda import pool_ops
        k2, s2, p2 = _tup(kernel, 2), _tup(stride, 2) or (1, 1), _tup(pad, 2) or (0, 0)
        if pool_ops.supported(data, k2, s2, p2):
            return pool_ops.max_pool2d_nhwc(data, k2, s2, p2, pooling_convention == 'full')
    if layout in _CHANNEL_LAST and nsp == 2 and pool_type == 'avg' and _use_ew(data) \
            and pooling_convention in ('valid', 'full'):
        from .cuda import elementwise_ops as ew
        if ew.avgpool_supported(data):
            if global_pool:
                return ew.global_avg_pool_nhwc(data)
            k2, s2, p2 = _tup(kernel, 2), _tup(stride, 2) or (1, 1), _tup(pad, 2) or (0, 0)
            if p2[0] < k2[0] and p2[1] < k2[1]:
                return ew.avg_pool2d_nhwc(data, k2, s2, p2, pooling_convention == 'full',
                                          True if count_include_pad is None else bool(count_include_pad))
    x = _to_channel_first(data, layout)
    if global_pool:
        red = tuple(range(2, x.dim()))
        if pool_type == 'max':
            y = torch.amax(x, red, keepdim=True)
        elif pool_type == 'avg':
            y = x.float().mean(red, keepdim=True).to(x.dtype) if x.dtype in (torch.float16, torch.bfloat16) \
                else x.mean(red, keepdim=True)
        elif pool_type == 'sum':
            y = x.sum(red, keepdim=True)
        else:
            p = p_value or 2
            y = x.abs().pow(p).sum(red, keepdim=True).pow(1.0 / p)
        return _to_layout(y, layout)
    kernel = _tup(kernel, nsp)
    stride = _tup(stride, nsp) or (1,) * nsp
    pad = _tup(pad, nsp) or (0,) * nsp
    ceil_mode = pooling_convention == 'full'
    if pooling_convention == 'same':
        pad = tuple(max(((math.ceil(x.shape[2 + i] / stride[i]) - 1) * stride[i] + kernel[i] - x.shape[2 + i] + 1) // 2, 0)
                    for i in range(nsp))
    include = True if count_include_pad is None else bool(count_include_pad)
    if pool_type == 'max':
        fn = (F.max_pool1d, F.max_pool2d, F.max_pool3d)[nsp - 1]
        y = fn(x, kernel, stride, pad, 1, ceil_mode)
    elif pool_type in ('avg', 'sum'):
        fn = (F.avg_pool1d, F.avg_pool2d, F.avg_pool3d)[nsp - 1]
        y = fn(x, kernel, stride, pad, ceil_mode, include)
        if pool_type == 'sum':
            y = y * float(torch.tensor(kernel).prod())
    elif pool_type == 'lp':
        p = p_value or 2
        fn = (F.avg_pool1d, F.avg_pool2d, F.avg_pool3d)[nsp - 1]
        y = (fn(x.abs().pow(p), kernel, stride, pad, ceil_mode, True) * float(torch.tensor(kernel).prod())).pow(1.0 / p)
    else:
        raise MXNetError('unknown pool_type %s' % pool_type)
    return _to_layout(y, layout)


@register('_contrib_AdaptiveAvgPooling2D', inputs=('data',), defaults={'output_size': ()})
def adaptive_avg_pool2d(data, output_size=()):
    if isinstance(output_size, int):
        output_size = (output_size, output_size)
    if not output_size:
        output_size = (1, 1)
    if len(output_size) == 1:
        output_size = (output_size[0], output_size[0])
    return F.adaptive_avg_pool2d(data, tuple(output_size))


@register('UpSampling', inputs=('*data',), defaults={'scale': 1, 'num_filter': 0, 'sample_type': 'nearest',
                                                     'multi_input_mode': 'concat', 'num_args': 1, 'workspace': 512})
def upsampling(*data, scale=1, num_filter=0, sample_type='nearest', multi_input_mode='concat', num_args=1,
               workspace=512):
    if sample_type == 'nearest':
        outs = []
        tgt = None
        for d in data:
            if tgt is None:
                o = F.interpolate(d, scale_factor=scale, mode='nearest')
                tgt = o.shape[2:]
            else:
                o = F.interpolate(d, size=tgt, mode='nearest')
            outs.append(o)
        if len(outs) == 1:
            return outs[0]
        return torch.cat(outs, 1) if multi_input_mode == 'concat' else sum(outs[1:], outs[0])
    x, w = data[0], data[1]
    k = 2 * scale - scale % 2
    p = int(math.ceil((scale - 1) / 2.0))
    return F.conv_transpose2d(x, w, None, scale, p, 0, x.shape[1])


@register('_contrib_BilinearResize2D', inputs=('data', 'like'),
          defaults={'height': 1, 'width': 1, 'scale_height': None, 'scale_width': None, 'mode': 'size',
                    'align_corners': True})
def bilinear_resize2d(data, like=None, height=1, width=1, scale_height=None, scale_width=None, mode='size',
                      align_corners=True):
    if mode == 'like' and like is not None:
        size = like.shape[2:]
    elif scale_height is not None:
        size = (int(data.shape[2] * scale_height), int(data.shape[3] * (scale_width or scale_height)))
    else:
        size = (height, width)
    return F.interpolate(data, size=tuple(size), mode='bilinear', align_corners=align_corners)


# ------------------------------------------------------------------------------------------
# Activations
# ------------------------------------------------------------------------------------------
_ACT = {
    'relu': torch.relu, 'sigmoid': torch.sigmoid, 'tanh': torch.tanh, 'softrelu': F.softplus,
    'softsign': F.softsign, 'log_sigmoid': F.logsigmoid, 'mish': F.mish,
}


@register('Activation', '_npx_activation', inputs=('data',), defaults={'act_type': 'relu'})
def activation(data, act_type='relu'):
    try:
        return _ACT[act_type](data)
    except KeyError:
        raise MXNetError('unknown act_type %s' % act_type)


@register('LeakyReLU', '_npx_leaky_relu', inputs=('data', 'gamma'),
          defaults={'act_type': 'leaky', 'slope': 0.25, 'lower_bound': 0.125, 'upper_bound': 0.334})
def leaky_relu(data, gamma=None, act_type='leaky', slope=0.25, lower_bound=0.125, upper_bound=0.334):
    if act_type == 'leaky':
        return F.leaky_relu(data, slope)
    if act_type == 'elu':
        return F.elu(data, slope)
    if act_type == 'selu':
        return F.selu(data)
    if act_type == 'gelu':
        if _use_ew(data):
            from .cuda import elementwise_ops as ew
            if ew.pointwise_supported(data, data.shape[-1] if data.dim() else 1):
                return ew.gelu(data)
        return F.gelu(data)
    if act_type == 'gelu_tanh':
        return F.gelu(data, approximate='tanh')
    if act_type == 'prelu':
        g = gamma
        if g.numel() > 1 and data.dim() > 1:
            shape = [1] * data.dim()
            shape[1] = -1
            g = g.reshape(shape)
        return torch.where(data > 0, data, data * g)
    if act_type == 'rrelu':
        if _state.state.training:
            a = torch.empty_like(data).uniform_(lower_bound, upper_bound)
        else:
            a = (lower_bound + upper_bound) / 2.0
        return torch.where(data > 0, data, data * a)
    raise MXNetError('unknown act_type %s' % act_type)


@register('SoftmaxActivation', inputs=('data',), defaults={'mode': 'instance'})
def softmax_activation(data, mode='instance'):
    if mode == 'channel':
        return torch.softmax(data, 1)
    return torch.softmax(data.reshape(data.shape[0], -1), 1).reshape(data.shape)


# ------------------------------------------------------------------------------------------
# Dropout (src/operator/nn/dropout-inl.h:72-84)
# ------------------------------------------------------------------------------------------
@register('Dropout', '_npx_dropout', inputs=('data',), defaults={'p': 0.5, 'mode': 'training', 'axes': (), 'cudnn_off': False})
def dropout(data, p=0.5, mode='training', axes=(), cudnn_off=False):
    active = (mode == 'always') or _state.state.training
    if not active or p == 0:
        return data
    if axes:
        shape = list(data.shape)
        for a in axes:
            shape[a] = 1
        mask = (torch.rand(shape, device=data.device) >= p).to(data.dtype) / (1 - p)
        return data * mask
    if _use_ew(data) and 0 < p < 1:
        from .cuda import elementwise_ops as ew
        if ew.pointwise_supported(data, data.shape[-1] if data.dim() else 1):
            return ew.dropout(data, p)
    return F.dropout(data, p, True)


# ------------------------------------------------------------------------------------------
# softmax family (src/operator/nn/softmax-inl.h:955-1003)
# ------------------------------------------------------------------------------------------
def _length_mask(data, length, axis):
    n = data.shape[axis]
    shape = [1] * data.dim()
    shape[axis] = n
    steps = torch.arange(n, device=data.device).reshape(shape)
    lshape = list(data.shape)
    lshape[axis] = 1
    return steps < length.reshape(lshape).to(steps.dtype)


def _softmax_impl(data, axis, temperature, length, use_length, dtype, log=False, neg=False):
    x = data
    if dtype is not None:
        x = x.to(to_torch_dtype(dtype))
    if neg:
        x = -x
    if temperature is not None and temperature != 1.0:
        x = x / temperature
    if use_length and length is not None:
        mask = _length_mask(x, length, axis % x.dim())
        x = x.masked_fill(~mask, float('-inf'))
        out = torch.log_softmax(x, axis) if log else torch.softmax(x, axis)
        return out.masked_fill(~mask, 0.0)
    if x.is_cuda and axis in (-1, x.dim() - 1) and _use_kernels(x) and x.is_contiguous() and \
            x.dtype in (torch.float16, torch.bfloat16, torch.float32):
        from .cuda import softmax_ops
        if softmax_ops.supported(x):
            return softmax_ops.softmax(x, log)
    return torch.log_softmax(x, axis) if log else torch.softmax(x, axis)


@register('softmax', '_npx_softmax', inputs=('data', 'length'),
          defaults={'axis': -1, 'temperature': None, 'dtype': None, 'use_length': False})
def softmax(data, length=None, axis=-1, temperature=None, dtype=None, use_length=False):
    return _softmax_impl(data, axis, temperature, length, use_length, dtype)


@register('log_softmax', '_npx_log_softmax', inputs=('data', 'length'),
          defaults={'axis': -1, 'temperature': None, 'dtype': None, 'use_length': False})
def log_softmax(data, length=None, axis=-1, temperature=None, dtype=None, use_length=False):
    return _softmax_impl(data, axis, temperature, length, use_length, dtype, log=True)


@register('softmin', inputs=('data',), defaults={'axis': -1, 'temperature': None, 'dtype': None, 'use_length': False})
def softmin(data, axis=-1, temperature=None, dtype=None, use_length=False):
    return _softmax_impl(data, axis, temperature, None, False, dtype, neg=True)


@register('masked_softmax', '_npx_masked_softmax', inputs=('data', 'mask'),
          defaults={'axis': -1, 'temperature': 1.0, 'normalize': True})
def masked_softmax(data, mask=None, axis=-1, temperature=1.0, normalize=True):
    x = data / temperature if temperature not in (None, 1.0) else data
    if mask is None:
        return torch.softmax(x, axis)
    m = mask if mask.dtype == torch.bool else mask != 0
    x = x.masked_fill(~m, -1e18 if x.dtype == torch.float32 else -1e4) if not normalize else x.masked_fill(~m, float('-inf'))
    out = torch.softmax(x, axis)
    return torch.where(m, out, torch.zeros_like(out))


@register('masked_log_softmax', '_npx_masked_log_softmax', inputs=('data', 'mask'),
          defaults={'axis': -1, 'temperature': 1.0, 'normalize': True})
def masked_log_softmax(data, mask=None, axis=-1, temperature=1.0, normalize=True):
    x = data / temperature if temperature not in (None, 1.0) else data
    if mask is None:
        return torch.log_softmax(x, axis)
    m = mask if mask.dtype == torch.bool else mask != 0
    out = torch.log_softmax(x.masked_fill(~m, float('-inf')), axis)
    return torch.where(m, out, torch.full_like(out, float('-inf')))


class _SoftmaxOutputFn(torch.autograd.Function):
    """Forward = softmax; backward = (p - onehot(label)) * grad_scale, independent of the head
    gradient (``src/operator/softmax_output-inl.h:133-253``)."""

    @staticmethod
    def forward(ctx, data, label, grad_scale, ignore_label, multi_output, use_ignore, preserve_shape,
                normalization, out_grad, smooth_alpha):
        if multi_output:
            prob = torch.softmax(data.float(), 1).to(data.dtype)
        elif preserve_shape:
            prob = torch.softmax(data.float(), -1).to(data.dtype)
        else:
            prob = torch.softmax(data.float().reshape(data.shape[0], -1), 1).reshape(data.shape).to(data.dtype)
        ctx.save_for_backward(prob, label)
        ctx.cfg = (grad_scale, ignore_label, multi_output, use_ignore, preserve_shape, normalization, out_grad,
                   smooth_alpha)
        return prob

    @staticmethod
    def backward(ctx, gout):
        prob, label = ctx.saved_tensors
        grad_scale, ignore_label, multi_output, use_ignore, preserve_shape, normalization, out_grad, alpha = ctx.cfg
        p = prob.float()
        if label.shape == prob.shape:          # probability labels
            g = p - label.float()
            valid_cnt = None
        else:
            cax = 1 if multi_output else (p.dim() - 1 if preserve_shape else 1)
            if not multi_output and not preserve_shape:
                p2 = p.reshape(p.shape[0], -1)
                lab = label.reshape(-1).long()
                oh = F.one_hot(lab.clamp(0, p2.shape[1] - 1), p2.shape[1]).float()
                if alpha > 0:
                    oh = oh * (1 - alpha) + (1 - oh) * (alpha / (p2.shape[1] - 1))
                g = p2 - oh
                if use_ignore:
                    keep = (lab != int(ignore_label)).float().unsqueeze(1)
                    g = g * keep
                    valid_cnt = keep.sum()
                else:
                    valid_cnt = torch.tensor(float(lab.numel()), device=p.device)
                g = g.reshape(p.shape)
            else:
                lab = label.long()
                k = p.shape[cax]
                oh = F.one_hot(lab.clamp(0, k - 1), k).float()
                if alpha > 0:
                    oh = oh * (1 - alpha) + (1 - oh) * (alpha / (k - 1))
                if cax != p.dim() - 1:
                    oh = oh.movedim(-1, cax)
                g = p - oh
                if use_ignore:
                    keep = (lab != int(ignore_label)).float().unsqueeze(cax)
                    g = g * keep
                    valid_cnt = keep.sum()
                else:
                    valid_cnt = torch.tensor(float(lab.numel()), device=p.device)
        scale = grad_scale
        if normalization == 'batch':
            scale = scale / p.shape[0]
        elif normalization == 'valid' and valid_cnt is not None:
            g = g / valid_cnt.clamp(min=1.0)
        elif normalization == 'null' and multi_output and False:
            pass
        g = g * scale
        if out_grad:
            g = g * gout.float()
        return (g.to(prob.dtype),) + (None,) * 9


@register('SoftmaxOutput', 'Softmax', inputs=('data', 'label'),
          defaults={'grad_scale': 1.0, 'ignore_label': -1.0, 'multi_output': False, 'use_ignore': False,
                    'preserve_shape': False, 'normalization': 'null', 'out_grad': False, 'smooth_alpha': 0.0})
def softmax_output(data, label=None, grad_scale=1.0, ignore_label=-1.0, multi_output=False, use_ignore=False,
                   preserve_shape=False, normalization='null', out_grad=False, smooth_alpha=0.0):
    if label is None:
        if multi_output:
            return torch.softmax(data, 1)
        return torch.softmax(data.reshape(data.shape[0], -1), 1).reshape(data.shape) if not preserve_shape \
            else torch.softmax(data, -1)
    return _SoftmaxOutputFn.apply(data, label, grad_scale, ignore_label, multi_output, use_ignore, preserve_shape,
                                  normalization, out_grad, smooth_alpha)


class _RegressionOutputFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, data, label, grad_scale, kind):
        out = torch.sigmoid(data) if kind == 'logistic' else data.clone()
        ctx.save_for_backward(out, label)
        ctx.cfg = (grad_scale, kind)
        return out

    @staticmethod
    def backward(ctx, gout):
        out, label = ctx.saved_tensors
        grad_scale, kind = ctx.cfg
        lab = label.reshape(out.shape).to(out.dtype)
        n = out.numel() // out.shape[0] if out.dim() > 0 else 1
        if kind == 'mae':
            g = torch.sign(out - lab)
        else:
            g = out - lab
        return g * (grad_scale / n), None, None, None


for _nm, _kind in (('LinearRegressionOutput', 'linear'), ('LogisticRegressionOutput', 'logistic'),
                   ('MAERegressionOutput', 'mae')):
    def _mk(kind):
        def op(data, label=None, grad_scale=1.0):
            if label is None:
                return torch.sigmoid(data) if kind == 'logistic' else data
            return _RegressionOutputFn.apply(data, label, grad_scale, kind)
        return op
    register(_nm, inputs=('data', 'label'), defaults={'grad_scale': 1.0})(_mk(_kind))


class _SVMOutputFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, data, label, margin, reg, use_linear):
        ctx.save_for_backward(data, label)
        ctx.cfg = (margin, reg, use_linear)
        return data.clone()

    @staticmethod
    def backward(ctx, gout):
        data, label = ctx.saved_tensors
        margin, reg, use_linear = ctx.cfg
        k = data.shape[1]
        y = F.one_hot(label.long(), k).to(data.dtype) * 2 - 1
        viol = (margin - y * data) > 0
        if use_linear:
            g = torch.where(viol, -y * reg, torch.zeros_like(data))
        else:
            g = torch.where(viol, -2 * reg * (margin - y * data) * y, torch.zeros_like(data))
        return g, None, None, None, None


@register('SVMOutput', inputs=('data', 'label'), defaults={'margin': 1.0, 'regularization_coefficient': 1.0, 'use_linear': False})
def svm_output(data, label=None, margin=1.0, regularization_coefficient=1.0, use_linear=False):
    if label is None:
        return data
    return _SVMOutputFn.apply(data, label, margin, regularization_coefficient, use_linear)


@register('softmax_cross_entropy', inputs=('data', 'label'))
def softmax_cross_entropy(data, label):
    return F.cross_entropy(data.float(), label.long(), reduction='sum').reshape(1).to(data.dtype)


@register('_npx_softmax_ce_loss', 'sparse_softmax_ce', inputs=('data', 'label'),
          defaults={'axis': -1, 'ignore_label': None, 'smooth': 0.0})
def sparse_softmax_ce(data, label, axis=-1, ignore_label=None, smooth=0.0):
    """Per-row ``-log softmax(data)[label]`` (the composition ``pick(log_softmax(x), y)`` used by
    ``gluon.loss.SoftmaxCrossEntropyLoss``), computed by one fused kernel on the GPU so the
    probabilities of large vocabularies are never written out in the forward pass."""
    if axis in (-1, data.dim() - 1) and _use_kernels(data) and data.is_contiguous() and \
            data.dtype in (torch.float16, torch.bfloat16, torch.float32) and smooth == 0.0:
        from .cuda import softmax_ops
        if softmax_ops.supported(data):
            return softmax_ops.softmax_ce(data, label, ignore_label)
    logp = torch.log_softmax(data.float(), axis)
    lab = label.long()
    k = data.shape[axis]
    picked = -torch.gather(logp, axis, lab.clamp(0, k - 1).unsqueeze(axis)).squeeze(axis)
    if smooth > 0:
        picked = (1 - smooth) * picked - smooth * logp.mean(axis)
    if ignore_label is not None:
        picked = torch.where(lab == int(ignore_label), torch.zeros_like(picked), picked)
    return picked.to(data.dtype if data.dtype == torch.float32 else torch.float32)


# ------------------------------------------------------------------------------------------
# CTC loss
# ------------------------------------------------------------------------------------------
@register('CTCLoss', 'ctc_loss', '_contrib_CTCLoss', '_contrib_ctc_loss', '_npx_ctc_loss',
          inputs=('data', 'label', 'data_lengths', 'label_lengths'),
          defaults={'use_data_lengths': False, 'use_label_lengths': False, 'blank_label': 'first'})
def ctc_loss(data, label, data_lengths=None, label_lengths=None, use_data_lengths=False, use_label_lengths=False,
             blank_label='first'):
    T, N, C = data.shape
    logp = torch.log_softmax(data.float(), -1)
    lab = label.long()
    if blank_label == 'first':
        blank = 0
        pad_val = 0 if use_label_lengths else 0
        if label_lengths is None or not use_label_lengths:
            ll = (lab > 0).sum(1) if True else None
        else:
            ll = label_lengths.long()
    else:
        blank = C - 1
        if label_lengths is None or not use_label_lengths:
            ll = (lab >= 0).sum(1)
        else:
            ll = label_lengths.long()
        lab = lab.clamp(min=0)
    dl = data_lengths.long() if (use_data_lengths and data_lengths is not None) else \
        torch.full((N,), T, dtype=torch.long, device=data.device)
    return F.ctc_loss(logp, lab, dl, ll, blank=blank, reduction='none', zero_infinity=False).to(data.dtype)


# ------------------------------------------------------------------------------------------
# fused RNN (src/operator/rnn-inl.h:57-160; CPU math src/operator/rnn_impl.h)
# ------------------------------------------------------------------------------------------
_GATES = {'rnn_relu': 1, 'rnn_tanh': 1, 'lstm': 4, 'gru': 3}


def rnn_param_size(mode, num_layers, input_size, state_size, bidirectional=False, projection_size=None):
    """Length of the flat parameter vector: per layer/direction all weights first, then all biases."""
    g, d = _GATES[mode], 2 if bidirectional else 1
    h = state_size
    p = projection_size or h
    size = 0
    for l in range(num_layers):
        ni = input_size if l == 0 else p * d
        size += d * (g * h * ni + g * h * p + 2 * g * h)
        if projection_size:
            size += d * (p * h)
    return size


def rnn_unpack(params, mode, num_layers, input_size, state_size, bidirectional=False, projection_size=None):
    """Split the flat vector into per-(layer, direction) tensors (w_ih, w_hh, [w_hr], b_ih, b_hh)."""
    g, d = _GATES[mode], 2 if bidirectional else 1
    h = state_size
    p = projection_size or h
    ws, off = [], 0
    for l in range(num_layers):
        ni = input_size if l == 0 else p * d
        for _ in range(d):
            w_ih = params[off:off + g * h * ni].reshape(g * h, ni); off += g * h * ni
            w_hh = params[off:off + g * h * p].reshape(g * h, p); off += g * h * p
            w_hr = None
            if projection_size:
                w_hr = params[off:off + p * h].reshape(p, h); off += p * h
            ws.append([w_ih, w_hh, w_hr])
    bs = []
    for l in range(num_layers):
        for _ in range(d):
            b_ih = params[off:off + g * h]; off += g * h
            b_hh = params[off:off + g * h]; off += g * h
            bs.append((b_ih, b_hh))
    return [(w[0], w[1], w[2], b[0], b[1]) for w, b in zip(ws, bs)]


def _lstm_reorder(w):
    """MXNet/cuDNN gate order is (i, f, g, o), the same as the tensor library's: identity."""
    return w


def _rnn_layer_dir(x, h0, c0, w_ih, w_hh, w_hr, b_ih, b_hh, mode, reverse, seq_len, clip):
    T = x.shape[0]
    xs = x.flip(0) if reverse and seq_len is None else x
    gi_all = F.linear(xs, w_ih, b_ih)
    h, c = h0, c0
    outs = []
    H = w_hh.shape[0] // _GATES[mode]
    steps = range(T)
    for t in steps:
        tt = t
        gi = gi_all[tt]
        gh = F.linear(h, w_hh, b_hh)
        if mode == 'lstm':
            gates = gi + gh
            i, f, g, o = gates.chunk(4, 1)
            c_new = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(g)
            if clip is not None:
                c_new = c_new.clamp(clip[0], clip[1])
            h_new = torch.sigmoid(o) * torch.tanh(c_new)
            if w_hr is not None:
                h_new = F.linear(h_new, w_hr)
        elif mode == 'gru':
            ir, iz, in_ = gi.chunk(3, 1)
            hr, hz, hn = gh.chunk(3, 1)
            r = torch.sigmoid(ir + hr)
            z = torch.sigmoid(iz + hz)
            n = torch.tanh(in_ + r * hn)
            h_new = (1 - z) * n + z * h
            c_new = c
        else:
            act = torch.relu if mode == 'rnn_relu' else torch.tanh
            h_new = act(gi + gh)
            c_new = c
        if seq_len is not None:
            tpos = (T - 1 - t) if reverse else t
            # variable length: positions beyond a sequence's length keep the previous state
            # (reverse direction handled by the caller reversing each sequence individually)
            valid = (t < seq_len).to(h_new.dtype).unsqueeze(1)
            h_new = valid * h_new + (1 - valid) * h
            if mode == 'lstm':
                c_new = valid * c_new + (1 - valid) * c
            outs.append(h_new * valid)
        else:
            outs.append(h_new)
        h, c = h_new, c_new
    out = torch.stack(outs, 0)
    if reverse and seq_len is None:
        out = out.flip(0)
    return out, h, c


def _reverse_padded(x, seq_len):
    T, N = x.shape[0], x.shape[1]
    t = torch.arange(T, device=x.device)[:, None]
    L = seq_len.long()[None, :]
    src = torch.where(t < L, L - 1 - t, t)
    return x[src, torch.arange(N, device=x.device)[None, :]]


def _rnn_nout(attrs):
    if attrs.get('state_outputs') in (True, 'True', 1):
        return 3 if attrs.get('mode') == 'lstm' else 2
    return 1


@register('RNN', '_npx_rnn', inputs=('data', 'parameters', 'state', 'state_cell', 'sequence_length'), nout=_rnn_nout,
          defaults={'state_size': 0, 'num_layers': 1, 'bidirectional': False, 'mode': 'lstm', 'p': 0.0,
                    'state_outputs': False, 'projection_size': None, 'lstm_state_clip_min': None,
                    'lstm_state_clip_max': None, 'lstm_state_clip_nan': False, 'use_sequence_length': False})
def rnn(data, parameters, state, state_cell=None, sequence_length=None, state_size=0, num_layers=1,
        bidirectional=False, mode='lstm', p=0.0, state_outputs=False, projection_size=None,
        lstm_state_clip_min=None, lstm_state_clip_max=None, lstm_state_clip_nan=False,
        use_sequence_length=False):
    """Fused multi-layer RNN over a (T, N, C) batch with the flat parameter layout of the reference."""
    if mode != 'lstm' and state_cell is not None and sequence_length is None and use_sequence_length:
        sequence_length, state_cell = state_cell, None
    T, N, I = data.shape
    d = 2 if bidirectional else 1
    seq_len = sequence_length if use_sequence_length else None
    clip = (lstm_state_clip_min, lstm_state_clip_max) if lstm_state_clip_min is not None else None
    training = _state.state.training
    layers = rnn_unpack(parameters, mode, num_layers, I, state_size, bidirectional, projection_size)
    plain = projection_size is None and seq_len is None and clip is None

    def library(data, parameters, state, state_cell=None):
        """Library recurrence (cuDNN through the tensor library): same gate order and per-(layer, direction) weights."""
        flat = []
        for w_ih, w_hh, _w_hr, b_ih, b_hh in rnn_unpack(parameters, mode, num_layers, I, state_size, bidirectional, None):
            flat += [w_ih.contiguous(), w_hh.contiguous(), b_ih.contiguous(), b_hh.contiguous()]
        args = (flat, True, num_layers, float(p), bool(training), bool(bidirectional), False)
        if mode == 'lstm':
            return torch._VF.lstm(data, (state.contiguous(), state_cell.contiguous()), *args)
        fn = {'gru': torch._VF.gru, 'rnn_tanh': torch._VF.rnn_tanh, 'rnn_relu': torch._VF.rnn_relu}[mode]
        return fn(data, state.contiguous(), *args)

    if plain and _use_kernels(data) and data.dtype in (torch.float16, torch.bfloat16, torch.float32):
        from .cuda import rnn_ops
        if rnn_ops.supported(data, state_size, num_layers, mode):
            if mode == 'lstm':
                def own(data, parameters, state, state_cell):
                    return rnn_ops.lstm(data, parameters, state, state_cell, state_size, num_layers, p, training, bidirectional)
                inputs = (data, parameters, state, state_cell)
            else:
                def own(data, parameters, state):
                    return rnn_ops.recurrent(mode, data, parameters, state, state_size, num_layers, p, training, bidirectional)
                inputs = (data, parameters, state)
            key = (mode, str(data.dtype), T, N, I, state_size, num_layers, bool(bidirectional), bool(training))
            res = (own if rnn_ops.use_own(key, own, library, inputs, training) else library)(*inputs)
            return tuple(res) if state_outputs else res[0]
    if data.is_cuda and plain and not env.get('MXNET_RNN_UNROLLED'):
        res = library(data, parameters, state, state_cell) if mode == 'lstm' else library(data, parameters, state)
        return tuple(res) if state_outputs else res[0]
    x = data
    hy, cy = [], []
    for l in range(num_layers):
        outs = []
        for di in range(d):
            w_ih, w_hh, w_hr, b_ih, b_hh = layers[l * d + di]
            h0 = state[l * d + di]
            c0 = state_cell[l * d + di] if mode == 'lstm' else None
            xin = x
            if di == 1 and seq_len is not None:
                xin = _reverse_padded(x, seq_len)
                o, h, c = _rnn_layer_dir(xin, h0, c0, w_ih, w_hh, w_hr, b_ih, b_hh, mode, False, seq_len, clip)
                o = _reverse_padded(o, seq_len)
            else:
                o, h, c = _rnn_layer_dir(xin, h0, c0, w_ih, w_hh, w_hr, b_ih, b_hh, mode, di == 1, seq_len, clip)
            outs.append(o)
            hy.append(h)
            if mode == 'lstm':
                cy.append(c)
        x = outs[0] if d == 1 else torch.cat(outs, 2)
        if p > 0 and training and l < num_layers - 1:
            x = F.dropout(x, p, True)
    if not state_outputs:
        return x
    if mode == 'lstm':
        return x, torch.stack(hy, 0), torch.stack(cy, 0)
    return x, torch.stack(hy, 0)


# ------------------------------------------------------------------------------------------
# im2col / col2im, spatial ops
# ------------------------------------------------------------------------------------------
@register('im2col', inputs=('data',), defaults={'kernel': (), 'stride': (), 'dilate': (), 'pad': ()})
def im2col(data, kernel=(), stride=(), dilate=(), pad=()):
    n = len(kernel)
    return F.unfold(data, tuple(kernel), _tup(dilate, n) or 1, _tup(pad, n) or 0, _tup(stride, n) or 1)


@register('col2im', inputs=('data',), defaults={'output_size': (), 'kernel': (), 'stride': (), 'dilate': (), 'pad': ()})
def col2im(data, output_size=(), kernel=(), stride=(), dilate=(), pad=()):
    n = len(kernel)
    return F.fold(data, tuple(output_size), tuple(kernel), _tup(dilate, n) or 1, _tup(pad, n) or 0, _tup(stride, n) or 1)


@register('GridGenerator', inputs=('data',), defaults={'transform_type': 'affine', 'target_shape': (0, 0)})
def grid_generator(data, transform_type='affine', target_shape=(0, 0)):
    if transform_type == 'affine':
        h, w = target_shape
        theta = data.reshape(-1, 2, 3)
        ys = torch.linspace(-1, 1, h, device=data.device, dtype=data.dtype)
        xs = torch.linspace(-1, 1, w, device=data.device, dtype=data.dtype)
        gy, gx = torch.meshgrid(ys, xs, indexing='ij')
        base = torch.stack([gx.reshape(-1), gy.reshape(-1), torch.ones(h * w, device=data.device, dtype=data.dtype)], 0)
        return torch.matmul(theta, base).reshape(-1, 2, h, w)
    n, _, h, w = data.shape
    ys = torch.arange(h, device=data.device, dtype=data.dtype)
    xs = torch.arange(w, device=data.device, dtype=data.dtype)
    gy, gx = torch.meshgrid(ys, xs, indexing='ij')
    fx = (data[:, 0] + gx) / ((w - 1) / 2.0) - 1
    fy = (data[:, 1] + gy) / ((h - 1) / 2.0) - 1
    return torch.stack([fx, fy], 1)


@register('BilinearSampler', inputs=('data', 'grid'), defaults={'cudnn_off': False})
def bilinear_sampler(data, grid, cudnn_off=False):
    return F.grid_sample(data, grid.permute(0, 2, 3, 1), mode='bilinear', padding_mode='zeros', align_corners=True)


@register('SpatialTransformer', inputs=('data', 'loc'),
          defaults={'target_shape': (0, 0), 'transform_type': 'affine', 'sampler_type': 'bilinear', 'cudnn_off': False})
def spatial_transformer(data, loc, target_shape=(0, 0), transform_type='affine', sampler_type='bilinear', cudnn_off=False):
    grid = grid_generator(loc, 'affine', target_shape)
    return bilinear_sampler(data, grid)


@register('ROIPooling', inputs=('data', 'rois'), defaults={'pooled_size': (1, 1), 'spatial_scale': 1.0})
def roi_pooling(data, rois, pooled_size=(1, 1), spatial_scale=1.0):
    ph, pw = pooled_size
    outs = []
    H, W = data.shape[2], data.shape[3]
    for r in rois:
        b = int(r[0].item())
        x1, y1, x2, y2 = [int(round(v.item() * spatial_scale)) for v in r[1:5]]
        rh, rw = max(y2 - y1 + 1, 1), max(x2 - x1 + 1, 1)
        out = data.new_zeros(data.shape[1], ph, pw)
        for i in range(ph):
            hs = min(max(int(math.floor(i * rh / ph)) + y1, 0), H)
            he = min(max(int(math.ceil((i + 1) * rh / ph)) + y1, 0), H)
            for j in range(pw):
                ws = min(max(int(math.floor(j * rw / pw)) + x1, 0), W)
                we = min(max(int(math.ceil((j + 1) * rw / pw)) + x1, 0), W)
                if he > hs and we > ws:
                    out[:, i, j] = data[b, :, hs:he, ws:we].amax((1, 2))
        outs.append(out)
    return torch.stack(outs, 0)


@register('Correlation', inputs=('data1', 'data2'),
          defaults={'kernel_size': 1, 'max_displacement': 1, 'stride1': 1, 'stride2': 1, 'pad_size': 0, 'is_multiply': True})
def correlation(data1, data2, kernel_size=1, max_displacement=1, stride1=1, stride2=1, pad_size=0, is_multiply=True):
    n, c, h, w = data1.shape
    p1 = F.pad(data1, (pad_size,) * 4)
    p2 = F.pad(data2, (pad_size,) * 4)
    kr = (kernel_size - 1) // 2
    border = max_displacement + kr
    ph, pw = h + 2 * pad_size, w + 2 * pad_size
    oh = int(math.ceil((ph - 2 * border) / stride1))
    ow = int(math.ceil((pw - 2 * border) / stride1))
    r = max_displacement // stride2
    outs = []
    for dy in range(-r, r + 1):
        for dx in range(-r, r + 1):
            acc = 0
            for ky in range(-kr, kr + 1):
                for kx in range(-kr, kr + 1):
                    y0, x0 = border + ky, border + kx
                    a = p1[:, :, y0:y0 + oh * stride1:stride1, x0:x0 + ow * stride1:stride1]
                    b = p2[:, :, y0 + dy * stride2:y0 + dy * stride2 + oh * stride1:stride1,
                           x0 + dx * stride2:x0 + dx * stride2 + ow * stride1:stride1]
                    acc = acc + ((a * b) if is_multiply else (a - b).abs()).sum(1)
            outs.append(acc / (kernel_size * kernel_size * c))
    return torch.stack(outs, 1)


@register('IdentityAttachKLSparseReg', inputs=('data',), defaults={'sparseness_target': 0.1, 'penalty': 0.001, 'momentum': 0.9})
def identity_attach_kl(data, sparseness_target=0.1, penalty=0.001, momentum=0.9):
    return data


@register('Crop', inputs=('*data',), defaults={'num_args': 1, 'offset': (0, 0), 'h_w': (0, 0), 'center_crop': False})
def crop(*data, num_args=1, offset=(0, 0), h_w=(0, 0), center_crop=False):
    x = data[0]
    th, tw = (data[1].shape[2:] if len(data) > 1 else h_w)
    if center_crop:
        oy, ox = (x.shape[2] - th) // 2, (x.shape[3] - tw) // 2
    else:
        oy, ox = offset
    return x[:, :, oy:oy + th, ox:ox + tw]

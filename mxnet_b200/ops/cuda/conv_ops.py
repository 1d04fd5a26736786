"""NHWC convolution (stride 1, and strided 1x1) on the tcgen05 implicit-GEMM kernels (``conv_tcgen05.cu``).

``MXNET_B200_CONV`` selects which directions run on the in-tree kernels: ``auto`` (default) times the
in-tree kernel against the library convolution the first time a (shape, direction) is seen outside of
graph capture and keeps the faster one (the counterpart of the reference's ``cudnn_tune``,
src/operator/nn/cudnn/cudnn_algoreg-inl.h); a comma-separated subset of ``fwd,dgrad,wgrad`` or ``1``
forces the in-tree kernels, ``0`` the library.  Unsupported shapes (strided filters larger than 1x1, grouped, channel counts
that are not multiples of 8) always go to the library convolution on a channels-last view.  The forward kernel also accumulates the per-channel sums that a following
BatchNorm needs; they travel as an attribute of the output tensor and are used when that tensor
reaches the BatchNorm kernels unmodified.
"""
import os

import torch

from . import lib, ptr, stream_ptr, count_launch, check
from ._util import dt, require, job_wide
from .gemm_ops import _error_flag

_DEFAULT = 'auto'
_ALL = frozenset(('fwd', 'dgrad', 'wgrad'))
_tuned = {}          # (direction, dtype, geometry) -> True when the in-tree kernel won
_tuned_us = {}       # same keys -> (in-tree, library) microseconds measured by the autotuner on this rank
# rate credited to the separate BatchNorm statistics pass that the forward epilogue replaces, bytes per microsecond
# (the copy bandwidth: a conservative credit, the measured pass is slower)
_BN_REDUCE_BYTES_PER_US = 6.5e6
_MARGIN = 1.0        # the in-tree kernel is chosen when it is not slower
_flush = {}


def directions():
    v = os.environ.get('MXNET_B200_CONV', _DEFAULT).strip().lower()
    if v in ('0', '', 'none', 'off'):
        return frozenset()
    if v == 'auto':
        return frozenset(('auto',))
    if v in ('1', 'all', 'on'):
        return _ALL
    return frozenset(p.strip() for p in v.split(','))


def _time_us(fn, reps=5):
    """Median device time of `fn` with the L2 cache flushed before every run (as inside a training step, where the
    operands of a layer were evicted by the layers in between)."""
    dev = torch.cuda.current_device()
    flush = _flush.get(dev)
    if flush is None:
        flush = _flush[dev] = torch.empty(192 << 20, dtype=torch.uint8, device='cuda')
    fn()
    times = []
    for _ in range(reps):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e3)
    times.sort()
    return times[len(times) // 2]


def use_own(direction, dirs, key, own_fn, lib_fn, lib_extra_us=0.0):
    """Whether `direction` of the convolution described by `key` runs on the in-tree kernel."""
    if 'auto' not in dirs:
        return direction.split('+')[0] in dirs          # 'dgrad+skip' follows the setting of 'dgrad'
    k = (direction,) + key
    hit = _tuned.get(k)
    if hit is None:
        if torch.cuda.is_current_stream_capturing():
            return False                   # cannot time inside a capture; the eager warm-up run normally comes first
        with torch.no_grad():
            t_own, t_lib = _time_us(own_fn), _time_us(lib_fn) + lib_extra_us
            _tuned_us[k] = (round(t_own, 1), round(t_lib, 1))
            hit = _tuned[k] = job_wide(t_own <= _MARGIN * t_lib)
    return hit


def tuned_choices():
    """{(direction, dtype, N, H, W, Cin, Cout, R, S, pad, dilate): in-tree kernel chosen} of the auto mode so far."""
    return dict(_tuned)


def tuned_times():
    """Same keys -> (in-tree, library) microseconds with a cold L2, as timed on this rank."""
    return dict(_tuned_us)


def out_hw(h, w, kernel, pad, dilate, stride=(1, 1)):
    eh, ew = h + 2 * pad[0] - dilate[0] * (kernel[0] - 1), w + 2 * pad[1] - dilate[1] * (kernel[1] - 1)
    return (eh - 1) // stride[0] + 1, (ew - 1) // stride[1] + 1


def _pointwise_strided(weight, pad, stride):
    """The strided 1x1 convolution without padding: forward, data and weight gradient on sampled views of the tensors."""
    return _strided(stride) and tuple(weight.shape[1:3]) == (1, 1) and tuple(pad) == (0, 0)


def _strided(stride):
    return tuple(stride) != (1, 1)


def shape_ok(data, weight, stride, dilate, pad, num_group):
    if data.dtype not in (torch.float16, torch.bfloat16) or weight.dtype != data.dtype or num_group != 1:
        return False
    if data.dim() != 4 or weight.dim() != 4:
        return False
    if _strided(stride) and (min(stride) < 1 or max(stride) > 2):
        return False                     # strided filters: traversal strides of the input boxes, up to 2
    cin, cout = data.shape[-1], weight.shape[0]
    if cin % 8 or cout % 8 or weight.shape[3] != cin or not data.is_contiguous() or not weight.is_contiguous():
        return False
    ho, wo = out_hw(data.shape[1], data.shape[2], weight.shape[1:3], pad, dilate, stride)
    return ho >= 1 and wo >= 1 and data.numel() > 0 and max(pad) < 256


def supported(data, weight, stride, dilate, pad, num_group):
    return bool(directions()) and shape_ok(data, weight, stride, dilate, pad, num_group)


def conv_forward(x, w, bias=None, res=None, pad=(0, 0), dilate=(1, 1), relu=False, want_stats=False, stride=(1, 1)):
    """y = act(conv(x, w) + bias + res) and, optionally, the [rows, 2, Cout] partial sums of y and y*y.  A stride other
    than 1 is taken for 1x1 filters without padding (and without residual)."""
    L = lib()
    n, h, wd, cin = x.shape
    cout, r, s, _ = w.shape
    require(x, 'data')
    require(w, 'weight', dtype=x.dtype, device=x.device, shape=(cout, r, s, cin))
    ho, wo = out_hw(h, wd, (r, s), pad, dilate, stride)
    y = torch.empty((n, ho, wo, cout), dtype=x.dtype, device=x.device)
    if _strided(stride) and not _pointwise_strided(w, pad, stride):
        # any filter size: the input boxes are fetched with traversal strides
        if res is not None:
            raise ValueError('the strided convolution takes no residual input')
        if bias is not None:
            bias = require(bias.to(x.dtype).contiguous(), 'bias', numel=cout, device=x.device)
        stats = torch.empty((L.mxb_conv_stat_rows(), 2, cout), dtype=torch.float32, device=x.device) if want_stats else None
        check(L.mxb_conv_strided_forward(dt(x), ptr(x), ptr(w), ptr(y), ptr(bias), ptr(stats), n, h, wd, cin, cout, r, s,
                                         pad[0], pad[1], dilate[0], dilate[1], stride[0], stride[1], 1 if relu else 0,
                                         ptr(_error_flag(x.device)), stream_ptr(x.device)), 'conv_strided_forward')
        count_launch(1)
        return y, stats
    if _strided(stride):
        if res is not None:
            raise ValueError('the strided convolution takes no residual input')
        if bias is not None:
            bias = require(bias.to(x.dtype).contiguous(), 'bias', numel=cout, device=x.device)
        stats = torch.empty((L.mxb_conv_stat_rows(), 2, cout), dtype=torch.float32, device=x.device) if want_stats else None
        check(L.mxb_conv1x1_strided_forward(dt(x), ptr(x), ptr(w), ptr(y), ptr(bias), ptr(stats), n, h, wd, cin, cout, stride[0],
                                            stride[1], 1 if relu else 0, ptr(_error_flag(x.device)), stream_ptr(x.device)),
              'conv1x1_strided_forward')
        count_launch(1)
        return y, stats
    if bias is not None:
        bias = require(bias.to(x.dtype).contiguous(), 'bias', numel=cout, device=x.device)
    if res is not None:
        require(res, 'residual', dtype=x.dtype, device=x.device, shape=y.shape)
    stats = torch.empty((L.mxb_conv_stat_rows(), 2, cout), dtype=torch.float32, device=x.device) if want_stats else None
    check(L.mxb_conv_forward(dt(x), ptr(x), ptr(w), ptr(y), ptr(bias), ptr(res), ptr(stats), n, h, wd, cin, cout, r, s,
                             pad[0], pad[1], dilate[0], dilate[1], 1 if relu else 0, ptr(_error_flag(x.device)),
                             stream_ptr(x.device)), 'conv_forward')
    count_launch(1)
    return y, stats


def conv_dgrad(dy, w, in_hw, pad=(0, 0), dilate=(1, 1), res=None, stride=(1, 1)):
    """Gradient with respect to the input of the convolution (optionally added to ``res``)."""
    L = lib()
    n, ho, wo, cout = dy.shape
    _, r, s, cin = w.shape
    h, wd = in_hw
    require(dy, 'out_grad', shape=(n,) + out_hw(h, wd, (r, s), pad, dilate, stride) + (cout,))
    require(w, 'weight', dtype=dy.dtype, device=dy.device, shape=(cout, r, s, cin))
    dx = torch.empty((n, h, wd, cin), dtype=dy.dtype, device=dy.device)
    if _strided(stride):
        if not _pointwise_strided(w, pad, stride):
            raise ValueError('the data gradient of a strided filter larger than 1x1 has no in-tree kernel')
        if res is not None:
            raise ValueError('no residual input for the strided data gradient')
        check(L.mxb_conv1x1_strided_dgrad(dt(dy), ptr(dy), ptr(w), ptr(dx), n, h, wd, cin, cout, stride[0], stride[1],
                                          ptr(_error_flag(dy.device)), stream_ptr(dy.device)), 'conv1x1_strided_dgrad')
        count_launch(1)
        return dx
    if res is not None:
        require(res, 'residual', dtype=dy.dtype, device=dy.device, shape=dx.shape)
    check(L.mxb_conv_dgrad(dt(dy), ptr(dy), ptr(w), ptr(dx), ptr(res), n, h, wd, cin, cout, r, s, pad[0], pad[1],
                           dilate[0], dilate[1], ptr(_error_flag(dy.device)), stream_ptr(dy.device)), 'conv_dgrad')
    count_launch(1)
    return dx


def conv_wgrad(x, dy, kernel, pad=(0, 0), dilate=(1, 1), stride=(1, 1)):
    """Gradient with respect to the [Cout, R, S, Cin] filter."""
    L = lib()
    n, h, wd, cin = x.shape
    cout = dy.shape[-1]
    r, s = kernel
    require(x, 'data')
    require(dy, 'out_grad', dtype=x.dtype, device=x.device, shape=(n,) + out_hw(h, wd, (r, s), pad, dilate, stride) + (cout,))
    dw32 = torch.empty((cout, r, s, cin), dtype=torch.float32, device=x.device)
    dw = torch.empty((cout, r, s, cin), dtype=x.dtype, device=x.device)
    if _strided(stride) and not ((r, s) == (1, 1) and tuple(pad) == (0, 0)):
        check(L.mxb_conv_strided_wgrad(dt(x), ptr(x), ptr(dy), ptr(dw), ptr(dw32), n, h, wd, cin, cout, r, s, pad[0], pad[1],
                                       dilate[0], dilate[1], stride[0], stride[1], ptr(_error_flag(x.device)),
                                       stream_ptr(x.device)), 'conv_strided_wgrad')
        count_launch(2)
        return dw
    if _strided(stride):
        check(L.mxb_conv1x1_strided_wgrad(dt(x), ptr(x), ptr(dy), ptr(dw), ptr(dw32), n, h, wd, cin, cout, stride[0], stride[1],
                                          ptr(_error_flag(x.device)), stream_ptr(x.device)), 'conv1x1_strided_wgrad')
        count_launch(2)
        return dw
    check(L.mxb_conv_wgrad(dt(x), ptr(x), ptr(dy), ptr(dw), ptr(dw32), n, h, wd, cin, cout, r, s, pad[0], pad[1],
                           dilate[0], dilate[1], ptr(_error_flag(x.device)), stream_ptr(x.device)), 'conv_wgrad')
    count_launch(2)
    return dw


def _library_backward(x, w, dy, pad, dilate, need_dx, need_dw, stride=(1, 1)):
    """Library data / weight gradient on channels-last views of the NHWC tensors."""
    xc, wc, dyc = x.permute(0, 3, 1, 2), w.permute(0, 3, 1, 2), dy.permute(0, 3, 1, 2)
    dx, dw, _ = torch.ops.aten.convolution_backward(dyc, xc, wc, None, list(stride), list(pad), list(dilate), False, [0, 0], 1,
                                                    [need_dx, need_dw, False])
    if dx is not None:
        dx = dx.permute(0, 2, 3, 1).contiguous()
    if dw is not None:
        dw = dw.permute(0, 2, 3, 1).contiguous()
    return dx, dw


def _library_forward(x, w, bias, pad, dilate, stride=(1, 1)):
    y = torch.nn.functional.conv2d(x.permute(0, 3, 1, 2), w.permute(0, 3, 1, 2), bias, stride, pad, dilate)
    return y.permute(0, 2, 3, 1).contiguous()


class _ConvNHWC(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, pad, dilate, dirs, want_stats, stride):
        key = (x.dtype,) + tuple(x.shape) + (w.shape[0], w.shape[1], w.shape[2]) + tuple(pad) + tuple(dilate) + tuple(stride)
        ho, wo = out_hw(x.shape[1], x.shape[2], w.shape[1:3], pad, dilate, stride)
        credit = x.shape[0] * ho * wo * w.shape[0] * x.element_size() / _BN_REDUCE_BYTES_PER_US if want_stats else 0.0
        if use_own('fwd', dirs, key, lambda: conv_forward(x, w, bias, None, pad, dilate, False, want_stats, stride),
                   lambda: _library_forward(x, w, bias, pad, dilate, stride), credit):
            y, stats = conv_forward(x, w, bias, None, pad, dilate, False, want_stats, stride)
        else:
            y, stats = _library_forward(x, w, bias, pad, dilate, stride), None
        ctx.save_for_backward(x, w)
        ctx.geom = (pad, dilate, dirs, bias is not None, key, stride)
        if stats is None:
            stats = x.new_empty(0, dtype=torch.float32)
        ctx.mark_non_differentiable(stats)
        return y, stats

    @staticmethod
    def backward(ctx, dy, _ds):
        x, w = ctx.saved_tensors
        pad, dilate, dirs, has_bias, key, stride = ctx.geom
        dy = dy.contiguous()
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dx = dw = None
        own_dgrad = not _strided(stride) or _pointwise_strided(w, pad, stride)      # strided R x S filters: library dgrad
        if need_dx and own_dgrad and use_own('dgrad', dirs, key, lambda: conv_dgrad(dy, w, x.shape[1:3], pad, dilate, None, stride),
                               lambda: _library_backward(x, w, dy, pad, dilate, True, False, stride)):
            dx = conv_dgrad(dy, w, x.shape[1:3], pad, dilate, None, stride)
        if need_dw and use_own('wgrad', dirs, key, lambda: conv_wgrad(x, dy, w.shape[1:3], pad, dilate, stride),
                               lambda: _library_backward(x, w, dy, pad, dilate, False, True, stride)):
            dw = conv_wgrad(x, dy, w.shape[1:3], pad, dilate, stride)
        lib_dx, lib_dw = need_dx and dx is None, need_dw and dw is None
        if lib_dx or lib_dw:
            ldx, ldw = _library_backward(x, w, dy, pad, dilate, lib_dx, lib_dw, stride)
            dx = ldx if lib_dx else dx
            dw = ldw if lib_dw else dw
        db = dy.sum((0, 1, 2)) if has_bias and ctx.needs_input_grad[2] else None
        return dx, dw, db, None, None, None, None, None


class _ConvSkipNHWC(torch.autograd.Function):
    """``(conv(x, w), x)``: a stride-1 convolution whose input also continues down a skip connection (the first
    convolution of an identity residual block).  Both gradients of ``x`` reach this node together, so the backward pass
    can add the skip gradient inside the data-gradient kernel's epilogue instead of a separate pass that reads both
    tensors and writes the sum (three passes over the largest activation of the block).  The choice between the fused
    in-tree kernel and library data gradient + add is timed per shape like every other direction."""

    @staticmethod
    def forward(ctx, x, w, pad, dilate, dirs, want_stats):
        key = (x.dtype,) + tuple(x.shape) + (w.shape[0], w.shape[1], w.shape[2]) + tuple(pad) + tuple(dilate) + (1, 1)
        ho, wo = out_hw(x.shape[1], x.shape[2], w.shape[1:3], pad, dilate)
        credit = x.shape[0] * ho * wo * w.shape[0] * x.element_size() / _BN_REDUCE_BYTES_PER_US if want_stats else 0.0
        if use_own('fwd', dirs, key, lambda: conv_forward(x, w, None, None, pad, dilate, False, want_stats),
                   lambda: _library_forward(x, w, None, pad, dilate), credit):
            y, stats = conv_forward(x, w, None, None, pad, dilate, False, want_stats)
        else:
            y, stats = _library_forward(x, w, None, pad, dilate), None
        ctx.save_for_backward(x, w)
        ctx.geom = (pad, dilate, dirs, key)
        if stats is None:
            stats = x.new_empty(0, dtype=torch.float32)
        ctx.mark_non_differentiable(stats)
        return y, stats, x.view_as(x)

    @staticmethod
    def backward(ctx, dy, _ds, dskip):
        x, w = ctx.saved_tensors
        pad, dilate, dirs, key = ctx.geom
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            if dskip is None:
                if use_own('dgrad', dirs, key, lambda: conv_dgrad(dy, w, x.shape[1:3], pad, dilate),
                           lambda: _library_backward(x, w, dy, pad, dilate, True, False)):
                    dx = conv_dgrad(dy, w, x.shape[1:3], pad, dilate)
                else:
                    dx = _library_backward(x, w, dy, pad, dilate, True, False)[0]
            else:
                dskip = dskip.contiguous()
                fused = lambda: conv_dgrad(dy, w, x.shape[1:3], pad, dilate, dskip)
                separate = lambda: _library_backward(x, w, dy, pad, dilate, True, False)[0].add_(dskip)
                dx = fused() if use_own('dgrad+skip', dirs, key, fused, separate) else separate()
        if ctx.needs_input_grad[1]:
            if use_own('wgrad', dirs, key, lambda: conv_wgrad(x, dy, w.shape[1:3], pad, dilate),
                       lambda: _library_backward(x, w, dy, pad, dilate, False, True)):
                dw = conv_wgrad(x, dy, w.shape[1:3], pad, dilate)
            else:
                dw = _library_backward(x, w, dy, pad, dilate, False, True)[1]
        return dx, dw, None, None, None, None


def conv2d_skip_nhwc(data, weight, pad, dilate=(1, 1), want_stats=True):
    """``(conv(data, weight), data)`` for a stride-1 convolution without bias; see :class:`_ConvSkipNHWC`."""
    dirs = directions()
    want_stats = want_stats and ('fwd' in dirs or 'auto' in dirs) and torch.is_grad_enabled()
    y, stats, skip = _ConvSkipNHWC.apply(data, weight, tuple(pad), tuple(dilate), dirs, want_stats)
    if stats.numel():
        y._mxb_bn_partials = (stats, y._version)
    return y, skip


def conv2d_nhwc(data, weight, bias, stride, pad, dilate=(1, 1), want_stats=True):
    dirs = directions()
    want_stats = want_stats and ('fwd' in dirs or 'auto' in dirs) and torch.is_grad_enabled()
    y, stats = _ConvNHWC.apply(data, weight, bias, tuple(pad), tuple(dilate), dirs, want_stats, tuple(stride))
    if stats.numel():
        # per-channel partial sums of this tensor for a BatchNorm that consumes it unmodified
        y._mxb_bn_partials = (stats, y._version)
    return y

"""Numerics of the tcgen05 implicit-GEMM convolution kernels against an fp32 convolution of the same inputs."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import mxnet_b200 as mx
from mxnet_b200 import autograd, nd

pytestmark = pytest.mark.gpu

SHAPES = [
    # N, H, W, Cin, Cout, R, pad, dilate
    (2, 8, 8, 64, 64, 3, 1, 1),
    (3, 7, 7, 72, 136, 3, 1, 1),
    (4, 14, 14, 256, 264, 3, 1, 1),
    (2, 56, 56, 64, 256, 1, 0, 1),
    (5, 9, 11, 16, 24, 3, 1, 1),
    (2, 10, 10, 64, 64, 3, 2, 2),
    (1, 6, 6, 8, 8, 5, 2, 1),
    (2, 12, 12, 128, 64, 3, 0, 1),
    (33, 4, 4, 512, 512, 1, 0, 1),
]


def _dev():
    return torch.device('cuda', 0)


def _close(a, b, rtol, atol):
    np.testing.assert_allclose(a.detach().float().cpu().numpy(), b.detach().float().cpu().numpy(), rtol=rtol, atol=atol)


def _inputs(N, H, W, Cin, Cout, R, dtype, seed=3):
    torch.manual_seed(seed)
    x = torch.randn(N, H, W, Cin, device=_dev()).to(dtype)
    w = (torch.randn(Cout, R, R, Cin, device=_dev()) / (R * Cin ** 0.5)).to(dtype)
    return x, w


def _ref_conv(x, w, pad, dil):
    y = F.conv2d(x.float().permute(0, 3, 1, 2), w.float().permute(0, 3, 1, 2), None, 1, pad, dil)
    return y.permute(0, 2, 3, 1).contiguous()


@pytest.mark.parametrize('N,H,W,Cin,Cout,R,pad,dil', SHAPES)
@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_conv_forward_with_epilogue_and_statistics(N, H, W, Cin, Cout, R, pad, dil, dtype):
    from mxnet_b200.ops.cuda import conv_ops, gemm_ops
    x, w = _inputs(N, H, W, Cin, Cout, R, dtype)
    ref = _ref_conv(x, w, pad, dil)
    tol = (1e-2, 1e-2) if dtype == torch.float16 else (3e-2, 3e-2)
    y, stats = conv_ops.conv_forward(x, w, None, None, (pad, pad), (dil, dil), False, True)
    gemm_ops.check_errors()
    _close(y, ref, *tol)
    s = stats.sum(0)
    M = ref.numel() // Cout
    _close(s[0] / M, ref.reshape(-1, Cout).mean(0), 1e-2, 2e-3)
    _close(s[1] / M, (ref * ref).reshape(-1, Cout).mean(0), 1e-2, 2e-3)
    bias = torch.randn(Cout, device=_dev()).to(dtype)
    res = torch.randn_like(ref).to(dtype)
    y2, _ = conv_ops.conv_forward(x, w, bias, res, (pad, pad), (dil, dil), True, False)
    gemm_ops.check_errors()
    _close(y2, torch.relu(ref + bias.float() + res.float()), *tol)


@pytest.mark.parametrize('N,H,W,Cin,Cout,R,pad,dil', SHAPES)
@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_conv_data_and_weight_gradients(N, H, W, Cin, Cout, R, pad, dil, dtype):
    from mxnet_b200.ops.cuda import conv_ops, gemm_ops
    x, w = _inputs(N, H, W, Cin, Cout, R, dtype, seed=4)
    xr, wr = x.float().requires_grad_(True), w.float().requires_grad_(True)
    ref = _ref_conv(xr, wr, pad, dil)
    dy = (torch.randn_like(ref) / 4).to(dtype)
    ref.backward(dy.float())
    dx = conv_ops.conv_dgrad(dy, w, (H, W), (pad, pad), (dil, dil))
    dw = conv_ops.conv_wgrad(x, dy, (R, R), (pad, pad), (dil, dil))
    gemm_ops.check_errors()
    tol = (1e-2, 1e-2) if dtype == torch.float16 else (3e-2, 3e-2)
    _close(dx, xr.grad, *tol)
    k = dy.numel() // Cout
    wtol = (1e-2, 2e-3 * k ** 0.5) if dtype == torch.float16 else (3e-2, 8e-3 * k ** 0.5)
    _close(dw, wr.grad, *wtol)
    res = torch.randn_like(x)
    dx2 = conv_ops.conv_dgrad(dy, w, (H, W), (pad, pad), (dil, dil), res=res)
    gemm_ops.check_errors()
    _close(dx2, xr.grad + res.float(), *tol)


@pytest.mark.parametrize('N,H,W,Cin,Cout,stride', [(4, 56, 56, 64, 128, 2), (3, 7, 9, 16, 24, 2), (2, 14, 14, 256, 512, 2),
                                                  (2, 10, 10, 8, 8, 3)])
@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_strided_1x1_convolution_all_directions(N, H, W, Cin, Cout, stride, dtype):
    """The down-sampling shortcut: a 1x1 filter with stride, read and written through strided tensor maps."""
    from mxnet_b200.ops.cuda import conv_ops, gemm_ops
    x, w = _inputs(N, H, W, Cin, Cout, 1, dtype, seed=6)
    xr, wr = x.float().requires_grad_(True), w.float().requires_grad_(True)
    ref = F.conv2d(xr.permute(0, 3, 1, 2), wr.permute(0, 3, 1, 2), None, stride).permute(0, 2, 3, 1).contiguous()
    dy = (torch.randn_like(ref) / 4).to(dtype)
    ref.backward(dy.float())
    st = (stride, stride)
    y, stats = conv_ops.conv_forward(x, w, None, None, (0, 0), (1, 1), False, True, st)
    dx = conv_ops.conv_dgrad(dy, w, (H, W), (0, 0), (1, 1), None, st)
    dw = conv_ops.conv_wgrad(x, dy, (1, 1), (0, 0), (1, 1), st)
    gemm_ops.check_errors()
    tol = (1e-2, 1e-2) if dtype == torch.float16 else (3e-2, 3e-2)
    assert y.shape == ref.shape
    _close(y, ref, *tol)
    _close(stats.sum(0)[0] / (ref.numel() // Cout), ref.reshape(-1, Cout).mean(0), 1e-2, 2e-3)
    _close(dx, xr.grad, *tol)
    k = dy.numel() // Cout
    _close(dw, wr.grad, tol[0], (2e-3 if dtype == torch.float16 else 8e-3) * k ** 0.5)


@pytest.mark.parametrize('N,H,W,Cin,Cout,R,pad', [(4, 56, 56, 128, 128, 3, 1), (2, 28, 28, 256, 256, 3, 1), (3, 15, 17, 16, 24, 3, 1),
                                                 (2, 14, 14, 512, 512, 3, 1), (2, 32, 32, 8, 64, 7, 3), (2, 9, 9, 16, 16, 3, 0)])
@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_strided_filter_forward_and_weight_gradient(N, H, W, Cin, Cout, R, pad, dtype):
    """Stride-2 convolutions with 3x3 and 7x7 filters (the down-sampling layers of a residual network): the input boxes are
    fetched with traversal strides.  Forward (with the statistics epilogue) and weight gradient against fp32."""
    from mxnet_b200.ops.cuda import conv_ops, gemm_ops
    x, w = _inputs(N, H, W, Cin, Cout, R, dtype, seed=16)
    xr, wr = x.float().requires_grad_(True), w.float().requires_grad_(True)
    ref = F.conv2d(xr.permute(0, 3, 1, 2), wr.permute(0, 3, 1, 2), None, 2, pad).permute(0, 2, 3, 1).contiguous()
    dy = (torch.randn_like(ref) / 4).to(dtype)
    ref.backward(dy.float())
    y, stats = conv_ops.conv_forward(x, w, None, None, (pad, pad), (1, 1), False, True, (2, 2))
    dw = conv_ops.conv_wgrad(x, dy, (R, R), (pad, pad), (1, 1), (2, 2))
    gemm_ops.check_errors()
    tol = (1e-2, 1e-2) if dtype == torch.float16 else (3e-2, 3e-2)
    assert y.shape == ref.shape
    _close(y, ref, *tol)
    _close(stats.sum(0)[0] / (ref.numel() // Cout), ref.reshape(-1, Cout).mean(0), 1e-2, 2e-3)
    k = dy.numel() // Cout
    _close(dw, wr.grad, tol[0], (2e-3 if dtype == torch.float16 else 8e-3) * k ** 0.5)


def test_strided_convolution_operator_trains_through_the_kernels():
    """``Convolution(kernel=3, stride=2)`` through the operator registry with the in-tree kernels forced: forward and
    weight gradient on the strided kernels, data gradient from the library, all against fp32."""
    import os
    old = os.environ.get('MXNET_B200_CONV')
    os.environ['MXNET_B200_CONV'] = '1'
    try:
        rng = np.random.RandomState(2)
        x_np = rng.randn(2, 12, 12, 32).astype('float32')
        w_np = (rng.randn(64, 3, 3, 32) / 17).astype('float32')
        ctx = mx.gpu(0)
        x, w = nd.array(x_np, ctx=ctx, dtype='float16'), nd.array(w_np, ctx=ctx, dtype='float16')
        x.attach_grad()
        w.attach_grad()
        with autograd.record():
            y = nd.Convolution(x, w, kernel=(3, 3), stride=(2, 2), pad=(1, 1), num_filter=64, no_bias=True, layout='NHWC')
            loss = (y * y).sum()
        loss.backward()
        xr = torch.tensor(x_np, device='cuda').half().float().requires_grad_(True)
        wr = torch.tensor(w_np, device='cuda').half().float().requires_grad_(True)
        ref = F.conv2d(xr.permute(0, 3, 1, 2), wr.permute(0, 3, 1, 2), None, 2, 1)
        (ref * ref).sum().backward()
        _close(y._data, ref.permute(0, 2, 3, 1), 1e-2, 1e-2)
        _close(x.grad._data, xr.grad, 2e-2, 5e-2)
        _close(w.grad._data, wr.grad, 2e-2, 2e-1)
    finally:
        if old is None:
            os.environ.pop('MXNET_B200_CONV', None)
        else:
            os.environ['MXNET_B200_CONV'] = old


def _conv_bn_step(x_np, w_np, env):
    import os
    old = os.environ.get('MXNET_B200_CONV')
    os.environ['MXNET_B200_CONV'] = env
    try:
        ctx = mx.gpu(0)
        x = nd.array(x_np, ctx=ctx, dtype='float16')
        w = nd.array(w_np, ctx=ctx, dtype='float16')
        C = w_np.shape[0]
        gamma, beta = nd.ones((C,), ctx=ctx), nd.zeros((C,), ctx=ctx)
        mm, mv = nd.zeros((C,), ctx=ctx), nd.ones((C,), ctx=ctx)
        for t in (x, w, gamma, beta):
            t.attach_grad()
        with autograd.record():
            y = nd.Convolution(x, w, kernel=(3, 3), pad=(1, 1), num_filter=C, no_bias=True, layout='NHWC')
            z = nd.BatchNorm(y, gamma, beta, mm, mv, fix_gamma=False, axis=3, eps=1e-5)
            loss = (z * z).sum()
        loss.backward()
        return [t.asnumpy().astype('float32') for t in (z, x.grad, w.grad, gamma.grad, mm, mv)]
    finally:
        if old is None:
            os.environ.pop('MXNET_B200_CONV', None)
        else:
            os.environ['MXNET_B200_CONV'] = old


def test_convolution_operator_feeds_batchnorm_statistics():
    """Convolution -> BatchNorm through the operator registry: the kernels' epilogue statistics give the same
    normalisation, running averages and gradients as the library convolution followed by a separate reduction."""
    from mxnet_b200.ops.cuda import gemm_ops, norm_ops
    rng = np.random.RandomState(0)
    x = rng.randn(4, 12, 12, 64).astype('float32')
    w = (rng.randn(128, 3, 3, 64) / 24).astype('float32')
    hits = norm_ops.hint_hits
    own = _conv_bn_step(x, w, 'fwd,dgrad,wgrad')
    gemm_ops.check_errors()
    assert norm_ops.hint_hits == hits + 1          # the BatchNorm took its statistics from the convolution epilogue
    lib = _conv_bn_step(x, w, '0')
    assert norm_ops.hint_hits == hits + 1
    for a, b, tol in zip(own, lib, (2e-2, 5e-2, 5e-1, 5e-1, 1e-3, 1e-3)):
        np.testing.assert_allclose(a, b, rtol=2e-2, atol=tol)

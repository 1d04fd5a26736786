"""Numerics of the pointwise / gather / pooling kernels against plain fp32 PyTorch references."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import mxnet_b200 as mx
from mxnet_b200 import autograd, nd

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float16, torch.bfloat16]


def _dev():
    return torch.device('cuda', 0)


def _tol(dtype):
    return {torch.float32: (1e-5, 1e-5), torch.float16: (2e-3, 2e-3), torch.bfloat16: (2e-2, 2e-2)}[dtype]


def _close(a, b, rtol, atol):
    np.testing.assert_allclose(a.detach().float().cpu().numpy(), b.detach().float().cpu().numpy(), rtol=rtol, atol=atol)


@pytest.mark.parametrize('shape', [(64, 3072), (3, 5, 768), (16,)])
@pytest.mark.parametrize('with_bias', [False, True])
@pytest.mark.parametrize('dtype', DTYPES)
def test_gelu_forward_backward(shape, with_bias, dtype):
    from mxnet_b200.ops.cuda import elementwise_ops as ew
    torch.manual_seed(0)
    x = torch.randn(*shape, device=_dev()).to(dtype).requires_grad_(True)
    bias = torch.randn(shape[-1], device=_dev()).to(dtype).requires_grad_(True) if with_bias else None
    y = ew.gelu(x, bias)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_(True)
    br = bias.detach().float().requires_grad_(True) if with_bias else None
    ref = F.gelu(xr + br if with_bias else xr)
    ref.backward(dy.float())
    _close(y, ref, *_tol(dtype))
    _close(x.grad, xr.grad, *_tol(dtype))
    if with_bias:
        rows = x.numel() // shape[-1]
        _close(bias.grad, br.grad, _tol(dtype)[0] * 4, _tol(dtype)[1] * rows ** 0.5 * 4)


@pytest.mark.parametrize('dtype', DTYPES)
def test_dropout_is_unbiased_consistent_and_fuses_bias_residual(dtype):
    from mxnet_b200.ops.cuda import elementwise_ops as ew
    torch.manual_seed(1)
    p = 0.25
    x = torch.ones(512, 1024, device=_dev(), dtype=dtype).requires_grad_(True)
    y = ew.dropout(x, p)
    kept = (y != 0).float().mean().item()
    assert abs(kept - (1 - p)) < 0.01
    _close(y[y != 0], torch.full_like(y[y != 0], 1 / (1 - p)), 1e-2, 1e-2)
    dy = torch.randn_like(y)
    y.backward(dy)
    # the backward pass recomputes the same mask
    _close(x.grad, dy.float() * (y != 0).float() / (1 - p), *_tol(dtype))
    y2 = ew.dropout(x.detach(), p)
    assert (y2 != y).any()                     # a new pattern on the next call
    # residual + dropout(x + bias)
    bias = torch.randn(1024, device=_dev()).to(dtype)
    res = torch.randn(512, 1024, device=_dev()).to(dtype)
    xb = torch.randn(512, 1024, device=_dev()).to(dtype)
    y3 = ew.dropout(xb, 0.0, bias, res)
    _close(y3, xb.float() + bias.float() + res.float(), *_tol(dtype))
    y4 = ew.dropout(xb, p, bias, res)
    d = (y4.float() - res.float())
    mask = d.abs() > 1e-3
    _close(d[mask], ((xb.float() + bias.float()) / (1 - p))[mask], 5e-2, 5e-2)


@pytest.mark.parametrize('count', [2, 3, 8, 11])
@pytest.mark.parametrize('dtype', DTYPES)
def test_add_n(count, dtype):
    from mxnet_b200.ops.cuda import elementwise_ops as ew
    torch.manual_seed(2)
    ts = [torch.randn(33, 128, device=_dev()).to(dtype) for _ in range(count)]
    ref = sum(t.float() for t in ts)
    out = ew.add_n(ts)
    rt, at = _tol(dtype)
    _close(out, ref, rt * 2, at * count)


@pytest.mark.parametrize('src,dst', [(torch.float32, torch.float16), (torch.float16, torch.float32),
                                     (torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32),
                                     (torch.float16, torch.bfloat16)])
@pytest.mark.parametrize('n', [8, 1000, 100003])
def test_cast(src, dst, n):
    from mxnet_b200.ops.cuda import elementwise_ops as ew
    torch.manual_seed(3)
    x = torch.randn(n, device=_dev()).to(src)
    y = ew.cast(x, dst)
    assert y.dtype == dst
    assert torch.equal(y, x.to(dst))


@pytest.mark.parametrize('idx_dtype', [torch.int32, torch.int64])
@pytest.mark.parametrize('dtype', DTYPES)
def test_embedding_forward_and_sorted_gradient(idx_dtype, dtype):
    from mxnet_b200.ops.cuda import elementwise_ops as ew
    torch.manual_seed(4)
    rows, D = 1000, 72 if dtype != torch.float32 else 68
    w = torch.randn(rows, D, device=_dev()).to(dtype).requires_grad_(True)
    idx = torch.randint(0, 50, (7, 129), device=_dev()).to(idx_dtype)        # many repeated rows
    idx[0, 0] = rows + 5                                                      # clipped like take(mode='clip')
    out = ew.embedding(idx, w)
    ref_idx = idx.long().clamp(0, rows - 1)
    assert torch.equal(out, w.detach()[ref_idx])
    dy = torch.randn_like(out)
    out.backward(dy)
    ref = torch.zeros(rows, D, device=_dev()).index_add_(0, ref_idx.reshape(-1), dy.float().reshape(-1, D))
    rt, at = _tol(dtype)
    _close(w.grad, ref, rt * 4, at * 8)
    g1 = w.grad.clone()
    w.grad = None
    ew.embedding(idx, w).backward(dy)
    assert torch.equal(g1, w.grad)                                            # bitwise reproducible


@pytest.mark.parametrize('shape,k,s,p,ceil,include', [((2, 13, 17, 16), 3, 2, 1, False, True), ((3, 8, 8, 64), 2, 2, 0, False, True),
                                                      ((2, 7, 7, 2048), 7, 1, 0, False, True), ((2, 9, 9, 8), 3, 2, 1, True, False),
                                                      ((1, 10, 12, 24), 3, 1, 1, False, False)])
@pytest.mark.parametrize('dtype', [torch.float16, torch.float32])
def test_avgpool_nhwc(shape, k, s, p, ceil, include, dtype):
    from mxnet_b200.ops.cuda import elementwise_ops as ew
    torch.manual_seed(5)
    x = torch.randn(*shape, device=_dev()).to(dtype).requires_grad_(True)
    y = ew.avg_pool2d_nhwc(x, (k, k), (s, s), (p, p), ceil, include)
    xr = x.detach().float().cpu().requires_grad_(True)          # fp32 reference evaluated on the host
    ref = F.avg_pool2d(xr.permute(0, 3, 1, 2), k, s, p, ceil, include).permute(0, 2, 3, 1)
    assert y.shape == ref.shape
    _close(y, ref, *_tol(dtype))
    dy = torch.randn_like(y)
    y.backward(dy)
    ref.backward(dy.float().cpu())
    _close(x.grad, xr.grad, _tol(dtype)[0] * 2, _tol(dtype)[1] * 4)


def test_global_avg_pool_and_operator_dispatch():
    x = nd.array(np.random.RandomState(0).randn(4, 7, 7, 64).astype('float32'), ctx=mx.gpu(0), dtype='float16')
    x.attach_grad()
    with autograd.record():
        y = nd.Pooling(x, global_pool=True, pool_type='avg', kernel=(1, 1), layout='NHWC')
        z = (y * y).sum()
    z.backward()
    ref = x.asnumpy().astype('float32').mean((1, 2), keepdims=True)
    np.testing.assert_allclose(y.asnumpy().astype('float32'), ref, rtol=2e-3, atol=2e-3)
    np.testing.assert_allclose(x.grad.asnumpy().astype('float32'), np.broadcast_to(2 * ref / 49, x.shape), rtol=1e-2, atol=1e-3)


@pytest.mark.parametrize('shape', [(100, 37), (5, 64, 128), (3, 2, 33, 65)])
@pytest.mark.parametrize('dtype', [torch.float16, torch.float32])
def test_transpose_last2(shape, dtype):
    from mxnet_b200.ops.cuda import elementwise_ops as ew
    x = torch.randn(*shape, device=_dev()).to(dtype)
    assert torch.equal(ew.transpose_last2(x), x.transpose(-1, -2).contiguous())


def test_operators_reach_the_kernels():
    """LeakyReLU(gelu), Dropout, Embedding, add_n and amp_cast route CUDA tensors to the kernel library."""
    from mxnet_b200.ops import cuda
    ctx = mx.gpu(0)
    before = cuda.launches()
    x = nd.array(np.random.RandomState(1).randn(8, 64).astype('float32'), ctx=ctx)
    w = nd.array(np.random.RandomState(2).randn(20, 64).astype('float32'), ctx=ctx)
    idx = nd.array(np.arange(8) % 20, ctx=ctx)
    g = nd.LeakyReLU(x, act_type='gelu')
    np.testing.assert_allclose(g.asnumpy(), F.gelu(torch.from_numpy(x.asnumpy())).numpy(), rtol=1e-5, atol=1e-5)
    e = nd.Embedding(idx, w, input_dim=20, output_dim=64)
    np.testing.assert_allclose(e.asnumpy(), w.asnumpy()[np.arange(8) % 20])
    s = nd.add_n(x, g, e)
    np.testing.assert_allclose(s.asnumpy(), x.asnumpy() + g.asnumpy() + e.asnumpy(), rtol=1e-5, atol=1e-5)
    h = nd.amp_cast(x, dtype='float16')
    assert h.dtype == np.float16
    with autograd.record(train_mode=True):
        d = nd.Dropout(x, p=0.5)
    assert 0.2 < float((d.asnumpy() == 0).mean()) < 0.8
    assert cuda.launches() - before >= 5


@pytest.mark.parametrize('mp', [False, True])
def test_multi_adamw_kernel_matches_tensor_op_rule(mp):
    """_multi_(mp_)adamw_update on CUDA (one kernel, rescale read on the device) against the same operator on CPU."""
    rng = np.random.RandomState(7)
    shapes = [(33,), (128, 65), (9000,), (3, 5, 7)]
    wdt = 'float16' if mp else 'float32'

    def run(ctx):
        data = []
        for s in shapes:
            w32 = rng_w[s]
            w = nd.array(w32, ctx=ctx, dtype=wdt)
            g = nd.array(rng_g[s], ctx=ctx, dtype=wdt)
            m = nd.array(rng_m[s], ctx=ctx)
            v = nd.array(rng_v[s], ctx=ctx)
            data += [w, g, m, v] + ([nd.array(w.asnumpy().astype('float32'), ctx=ctx)] if mp else [])
        rescale = nd.array([0.5], ctx=ctx)
        op = nd.contrib.multi_mp_adamw_update if mp else nd.contrib.multi_adamw_update
        for _ in range(3):
            op(*data, rescale, lrs=[0.01, 0.02, 0.03, 0.04], wds=[0.0, 0.1, 0.01, 0.0], etas=[1.0, 0.9, 1.0, 0.5],
               beta1=0.9, beta2=0.99, epsilon=1e-6, clip_gradient=0.8, num_weights=len(shapes), out=data[::5 if mp else 4])
        return [d.asnumpy().astype('float32') for d in data]

    rng_w = {s: rng.randn(*s).astype('float32') for s in shapes}
    rng_g = {s: rng.randn(*s).astype('float32') for s in shapes}
    rng_m = {s: rng.randn(*s).astype('float32') * 0.1 for s in shapes}
    rng_v = {s: np.abs(rng.randn(*s)).astype('float32') * 0.1 for s in shapes}
    gpu = run(mx.gpu(0))
    cpu = run(mx.cpu())
    for a, b in zip(gpu, cpu):
        np.testing.assert_allclose(a, b, rtol=2e-3 if mp else 1e-5, atol=2e-3 if mp else 1e-6)
    # a non-finite rescale (overflowed loss scale) skips the update on the device
    ctx = mx.gpu(0)
    w = nd.array(rng_w[(33,)], ctx=ctx)
    before = w.asnumpy().copy()
    nd.contrib.multi_adamw_update(w, nd.array(rng_g[(33,)], ctx=ctx), nd.zeros((33,), ctx=ctx), nd.zeros((33,), ctx=ctx),
                                  nd.array([float('inf')], ctx=ctx), lrs=[0.1], wds=[0.0], etas=[1.0], num_weights=1, out=[w])
    np.testing.assert_array_equal(w.asnumpy(), before)


@pytest.mark.parametrize('rows,C', [(8192, 3072), (1000, 768), (5, 8), (70000, 136)])
@pytest.mark.parametrize('dtype', DTYPES)
def test_column_sums(rows, C, dtype):
    from mxnet_b200.ops.cuda import elementwise_ops as ew
    torch.manual_seed(6)
    x = torch.randn(rows, C, device=_dev()).to(dtype)
    out = ew.colsum(x)
    ref = x.double().sum(0)
    np.testing.assert_allclose(out.cpu().numpy(), ref.cpu().numpy(), rtol=1e-4, atol=1e-3 * rows ** 0.5)
    assert torch.equal(out, ew.colsum(x))              # deterministic


# ---------------------------------------------------------------------------------------- detection kernels
@pytest.mark.parametrize('dtype', ['float32', 'float16'])
@pytest.mark.parametrize('position_sensitive,aligned,sample_ratio', [(False, False, 2), (False, True, -1), (True, False, 2)])
def test_roi_align_kernels_against_the_host_operator(dtype, position_sensitive, aligned, sample_ratio):
    import mxnet_b200 as mx
    from mxnet_b200 import autograd, nd
    rng = np.random.RandomState(5)
    data = rng.randn(2, 8, 9, 10).astype('float32')
    rois = np.array([[0, 1.0, 1.5, 6.0, 7.0], [1, -3.0, -2.0, 4.0, 5.0], [0, 5.0, 5.0, 12.0, 11.0], [-1, 0, 0, 4, 4],
                     [1, 2.25, 3.0, 2.5, 3.25]], dtype='float32')
    res = []
    for ctx in (mx.cpu(), mx.gpu(0)):
        x = nd.array(data, ctx=ctx, dtype=dtype if ctx.device_type == 'gpu' else 'float32')
        r = nd.array(rois, ctx=ctx, dtype=x.dtype)
        x.attach_grad()
        with autograd.record():
            y = nd.contrib.ROIAlign(x, r, pooled_size=(2, 2), spatial_scale=1.0, sample_ratio=sample_ratio,
                                    position_sensitive=position_sensitive, aligned=aligned)
            loss = (y * y).sum()
        loss.backward()
        res.append((y.asnumpy().astype('float32'), x.grad.asnumpy().astype('float32')))
    tol = dict(rtol=1e-4, atol=1e-4) if dtype == 'float32' else dict(rtol=2e-2, atol=2e-2)
    np.testing.assert_allclose(res[1][0], res[0][0], **tol)
    np.testing.assert_allclose(res[1][1], res[0][1], **tol)


@pytest.mark.parametrize('n,force', [(60, False), (300, True), (1000, False)])
def test_nms_kernels_against_the_host_operator(n, force):
    import mxnet_b200 as mx
    from mxnet_b200 import nd
    rng = np.random.RandomState(n)
    xy, wh = rng.uniform(0, 120, (2, n, 2)), rng.uniform(5, 40, (2, n, 2))
    rows = np.concatenate([rng.randint(0, 3, (2, n, 1)).astype('float64'), rng.uniform(0, 1, (2, n, 1)), xy, xy + wh], 2).astype('float32')
    outs = [nd.contrib.box_nms(nd.array(rows, ctx=ctx), overlap_thresh=0.45, valid_thresh=0.05, topk=400, coord_start=2, score_index=1,
                               id_index=0, force_suppress=force).asnumpy() for ctx in (mx.cpu(), mx.gpu(0))]
    np.testing.assert_allclose(outs[1], outs[0], rtol=1e-6)


def test_rtc_cuda_module_compiles_and_launches_a_user_kernel():
    """``mx.rtc.CudaModule``: source compiled at run time for the running GPU (reference: python/mxnet/rtc.py, the
    `axpy` example of its docstring), launched on arrays of the framework; a compile error is reported with the log."""
    import mxnet_b200 as mx
    from mxnet_b200 import nd
    assert mx.runtime.Features().is_enabled('CUDA_RTC')
    source = r"""
    extern "C" __global__ void axpy(const float* x, float* y, float alpha, int n) {
        int i = threadIdx.x + blockIdx.x * blockDim.x;
        if (i < n) y[i] += alpha * x[i];
    }
    extern "C" __global__ void scale_half(__half* x, float s, int n) {
        int i = threadIdx.x + blockIdx.x * blockDim.x;
        if (i < n) x[i] = __float2half(__half2float(x[i]) * s);
    }
    """
    module = mx.rtc.CudaModule('#include <cuda_fp16.h>\n' + source, exports=['axpy', 'scale_half'])
    axpy = module.get_kernel('axpy', 'const float *x, float *y, float alpha, int n')
    ctx = mx.gpu(0)
    n = 1000
    x = nd.array(np.arange(n, dtype='float32'), ctx=ctx)
    y = nd.ones((n,), ctx=ctx)
    axpy.launch([x, y, 3.0, n], ctx, ((n + 255) // 256, 1, 1), (256, 1, 1))
    np.testing.assert_allclose(y.asnumpy(), 1 + 3 * np.arange(n, dtype='float32'))
    half = module.get_kernel('scale_half', '__half *x, float s, int n')
    h = nd.array(np.arange(16, dtype='float16'), ctx=ctx, dtype='float16')
    half.launch([h, 0.5, 16], ctx, (1, 1, 1), (32, 1, 1))
    np.testing.assert_allclose(h.asnumpy().astype('float32'), np.arange(16) * 0.5)
    with pytest.raises(mx.MXNetError, match='NVRTC compilation failed'):
        mx.rtc.CudaModule('__global__ void broken( { }')
    with pytest.raises(ValueError):
        module.get_kernel('axpy', 'const float x[3]')


@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16, torch.float32])
def test_multi_tensor_add_inplace(dtype):
    """One launch adds many (destination, source) pairs: odd lengths, lengths around the 8192-element chunk, sources that
    are not 16-byte aligned, and more pairs than one launch takes."""
    from mxnet_b200.ops.cuda import optim_ops
    torch.manual_seed(4)
    sizes = [1, 7, 8, 9, 8191, 8192, 8193, 100003, 64 * 3 * 7 * 7] + [33 + i for i in range(60)]
    dsts = [torch.randn(n, device='cuda').to(dtype) for n in sizes]
    backing = [torch.randn(n + 1, device='cuda').to(dtype) for n in sizes]
    srcs = [b[1:] if i % 3 == 0 else b[:-1] for i, b in enumerate(backing)]          # every third source is misaligned
    expect = [(d.float() + s.float()).to(dtype) for d, s in zip(dsts, srcs)]
    optim_ops.multi_add_(dsts, srcs)
    torch.cuda.synchronize()
    for d, e, n in zip(dsts, expect, sizes):
        assert torch.equal(d, e), n


def _jpeg_bytes(img, quality=95):
    import io as _io
    from PIL import Image
    b = _io.BytesIO()
    Image.fromarray(img).save(b, format='JPEG', quality=quality, subsampling=0)
    return b.getvalue()


def _smooth_image(rng, h, w):
    """A smooth colour image (low frequencies only), so that JPEG decoders agree to within a few levels."""
    yy, xx = np.mgrid[0:h, 0:w].astype('float32')
    chans = [127 + 100 * np.sin(yy / rng.uniform(15, 40) + rng.uniform(0, 6)) * np.cos(xx / rng.uniform(15, 40) + rng.uniform(0, 6))
             for _ in range(3)]
    return np.clip(np.stack(chans, -1), 0, 255).astype('uint8')


def _bilinear_reference(img, x0, y0, cw, ch, H, W, mirror):
    """NumPy restatement of the augmentation kernel's sampling on a decoded image (float64)."""
    h, w = img.shape[:2]
    ox = np.arange(W)
    sx = (W - 1 - ox) if mirror else ox
    fx = np.clip(x0 + (sx + 0.5) * (cw / W) - 0.5, 0, w - 1)
    fy = np.clip(y0 + (np.arange(H) + 0.5) * (ch / H) - 0.5, 0, h - 1)
    xa, ya = np.floor(fx).astype(int), np.floor(fy).astype(int)
    xb, yb = np.minimum(xa + 1, w - 1), np.minimum(ya + 1, h - 1)
    wx, wy = (fx - xa)[None, :, None], (fy - ya)[:, None, None]
    im = img.astype('float64')
    top = im[ya][:, xa] * (1 - wx) + im[ya][:, xb] * wx
    bot = im[yb][:, xa] * (1 - wx) + im[yb][:, xb] * wx
    return top * (1 - wy) + bot * wy


@pytest.mark.parametrize('layout,dtype', [('NHWC', 'float16'), ('NCHW', 'float32')])
def test_gpu_image_pipeline_decodes_and_augments_like_the_host_reference(layout, dtype):
    """nvJPEG decode + the crop / resize / mirror / normalise kernel against PIL's decode followed by a NumPy restatement
    of the same sampling (reference pipeline: src/io/iter_image_recordio_2.cc + image_aug_default.cc + iter_normalize.h).
    JPEG decoders may differ by a few levels; the images are smooth, so the bound is 4 levels of 255."""
    import io as _io
    from PIL import Image
    import mxnet_b200 as mx
    from mxnet_b200.io import gpu_pipeline
    assert gpu_pipeline.available()
    rng = np.random.RandomState(3)
    sizes = [(96, 128), (150, 100), (64, 64), (201, 77)]
    imgs = [_smooth_image(rng, h, w) for h, w in sizes]
    jpegs = [_jpeg_bytes(im) for im in imgs]
    mean, std, scale = (123.68, 116.28, 103.53), (58.4, 57.1, 57.4), 1.0
    pipe = gpu_pipeline.GPUImagePipeline(mx.gpu(0), (48, 40), layout=layout, dtype=dtype, mean=mean, std=std, scale=scale)
    crops = [(3.0, 5.0, 80.0, 60.0), (0.0, 10.0, 100.0, 120.0), (0.0, 0.0, 64.0, 64.0), (10.5, 20.25, 50.0, 150.0)]
    mirrors = [0, 1, 0, 1]
    out = pipe(jpegs, crops=crops, mirrors=mirrors).asnumpy().astype('float64')
    if layout == 'NCHW':
        out = out.transpose(0, 2, 3, 1)
    assert out.shape == (4, 48, 40, 3)
    for i, jb in enumerate(jpegs):
        dec = np.asarray(Image.open(_io.BytesIO(jb)).convert('RGB'))
        ref = (_bilinear_reference(dec, *crops[i], 48, 40, mirrors[i]) - np.array(mean)) / np.array(std) * scale
        err = np.abs(out[i] - ref).max() * max(std)
        assert err < 4.0 + (0.5 if dtype == 'float16' else 0.0), (i, err)
    assert pipe.bytes_to_device == sum(len(j) for j in jpegs)
    with pytest.raises(mx.MXNetError, match='not a readable JPEG'):
        pipe([b'not a jpeg at all'])


def test_image_record_iter_on_the_gpu_matches_the_host_iterator(tmp_path):
    """``ImageRecordIter(device=mx.gpu(0))``: records are read by the native prefetcher, decoded and augmented on the GPU, and
    the batches (centre crop, mean / std) agree with the host iterator on the same file; labels are identical."""
    import mxnet_b200 as mx
    from mxnet_b200 import recordio
    rng = np.random.RandomState(5)
    path = str(tmp_path / 'imgs.rec')
    w = recordio.MXRecordIO(path, 'w')
    for i in range(10):
        img = _smooth_image(rng, 72 + 4 * (i % 3), 80 + 8 * (i % 2))
        w.write(recordio.pack(recordio.IRHeader(0, float(i % 4), i, 0), _jpeg_bytes(img)))
    w.close()
    kw = dict(path_imgrec=path, data_shape=(3, 56, 64), batch_size=4, mean_r=120.0, mean_g=110.0, mean_b=100.0, std_r=60.0, std_g=61.0,
              std_b=62.0, round_batch=True)
    host = mx.io.ImageRecordIter(**kw)
    gpu = mx.io.ImageRecordIter(device=mx.gpu(0), **kw)
    n = 0
    for hb, gb in zip(host, gpu):
        assert gb.data[0].context == mx.gpu(0) and gb.data[0].shape == (4, 3, 56, 64)
        np.testing.assert_array_equal(hb.label[0].asnumpy(), gb.label[0].asnumpy())
        diff = np.abs(hb.data[0].asnumpy() - gb.data[0].asnumpy()).max() * 62.0
        assert diff < 4.0, diff
        assert hb.pad == gb.pad
        n += 1
    assert n == 3

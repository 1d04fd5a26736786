"""Numerics of the hand-written sm_100a kernels against plain fp32 references of the same operators."""
import numpy as np
import pytest
import torch

import mxnet_b200 as mx
from mxnet_b200 import autograd, gluon, nd

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device('cuda', 0)


def _close(a, b, rtol, atol):
    a, b = a.detach().float().cpu().numpy(), b.detach().float().cpu().numpy()
    np.testing.assert_allclose(a, b, rtol=rtol, atol=atol)


# ---------------------------------------------------------------------------------------- BatchNorm
@pytest.mark.parametrize('C', [64, 256, 2048])
@pytest.mark.parametrize('relu,res', [(False, False), (True, False), (True, True), (False, True)])
@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_batchnorm_nhwc_forward_backward(C, relu, res, dtype):
    from mxnet_b200.ops.cuda import norm_ops
    torch.manual_seed(0)
    N, H, W = 4, 7, 9
    x = (torch.randn(N, H, W, C, device=_dev()) * 2 + 0.5).to(dtype).requires_grad_(True)
    r = torch.randn(N, H, W, C, device=_dev()).to(dtype).requires_grad_(True) if res else None
    pdt = dtype if C == 256 else torch.float32          # parameters stored in the activation dtype or in fp32
    gamma = (torch.rand(C, device=_dev()) + 0.5).to(pdt).requires_grad_(True)
    beta = torch.randn(C, device=_dev()).to(pdt).requires_grad_(True)
    rm, rv = torch.zeros(C, device=_dev()), torch.ones(C, device=_dev())
    y, mean, var = norm_ops.batch_norm_nhwc(x, gamma, beta, rm, rv, 1e-5, 0.9, True, 'relu' if relu else None, r)
    gy = torch.randn_like(y)
    y.backward(gy)
    # fp32 reference on the same (rounded) inputs
    xf = x.detach().float().requires_grad_(True)
    rf = r.detach().float().requires_grad_(True) if res else None
    g2, b2 = gamma.detach().float().requires_grad_(True), beta.detach().float().requires_grad_(True)
    m = xf.mean((0, 1, 2))
    v = xf.var((0, 1, 2), unbiased=False)
    ref = (xf - m) * torch.rsqrt(v + 1e-5) * g2 + b2
    if res:
        ref = ref + rf
    if relu:
        ref = torch.relu(ref)
    ref.backward(gy.float())
    tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.float16 else dict(rtol=6e-2, atol=6e-2)
    _close(y, ref, **tol)
    _close(mean, m, 1e-3, 1e-3)
    _close(var, v, 1e-2, 1e-2)
    _close(rm, 0.1 * m, 1e-3, 1e-3)
    _close(rv, 0.9 + 0.1 * v, 1e-2, 1e-2)
    _close(x.grad, xf.grad, **tol)
    assert gamma.grad.dtype == pdt and beta.grad.dtype == pdt
    _close(gamma.grad, g2.grad, 3e-2, 0.3)
    _close(beta.grad, b2.grad, 3e-2, 0.3)
    if res:
        _close(r.grad, rf.grad, **tol)


def test_batchnorm_inference_uses_running_stats():
    from mxnet_b200.ops.cuda import norm_ops
    C = 128
    x = torch.randn(2, 5, 5, C, device=_dev()).half()
    gamma, beta = torch.rand(C, device=_dev()) + 0.5, torch.randn(C, device=_dev())
    rm, rv = torch.randn(C, device=_dev()), torch.rand(C, device=_dev()) + 0.5
    rm0, rv0 = rm.clone(), rv.clone()
    y, _, _ = norm_ops.batch_norm_nhwc(x, gamma, beta, rm, rv, 1e-3, 0.9, False, None, None)
    ref = (x.float() - rm0) * torch.rsqrt(rv0 + 1e-3) * gamma + beta
    _close(y, ref, 1e-2, 1e-2)
    _close(rm, rm0, 0, 0)
    _close(rv, rv0, 0, 0)


# ---------------------------------------------------------------------------------------- LayerNorm
@pytest.mark.parametrize('shape', [(3, 128, 768), (17, 33), (5, 2048), (4099, 768), (1000, 1024), (513, 264), (70, 8)])
@pytest.mark.parametrize('dtype', [torch.float32, torch.float16, torch.bfloat16])
def test_layernorm(shape, dtype):
    from mxnet_b200.ops.cuda import norm_ops
    torch.manual_seed(1)
    C = shape[-1]
    x = torch.randn(*shape, device=_dev()).to(dtype).requires_grad_(True)
    g = (torch.rand(C, device=_dev()) + 0.5).requires_grad_(True)
    b = torch.randn(C, device=_dev()).requires_grad_(True)
    y = norm_ops.layer_norm(x, g, b, 1e-5)
    gy = torch.randn_like(y)
    y.backward(gy)
    xf = x.detach().float().requires_grad_(True)
    g2, b2 = g.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    ref = torch.nn.functional.layer_norm(xf, (C,), g2, b2, 1e-5)
    ref.backward(gy.float())
    tol = {torch.float32: (1e-4, 1e-4), torch.float16: (2e-2, 2e-2), torch.bfloat16: (6e-2, 6e-2)}[dtype]
    _close(y, ref, *tol)
    _close(x.grad, xf.grad, *tol)
    _close(g.grad, g2.grad, 3e-2, 0.2)
    _close(b.grad, b2.grad, 3e-2, 0.2)


# ---------------------------------------------------------------------------------------- softmax / CE
@pytest.mark.parametrize('rows,C', [(64, 1000), (7, 33), (3, 30522)])
@pytest.mark.parametrize('dtype', [torch.float32, torch.float16])
@pytest.mark.parametrize('log', [False, True])
def test_softmax(rows, C, dtype, log):
    from mxnet_b200.ops.cuda import softmax_ops
    torch.manual_seed(2)
    x = (torch.randn(rows, C, device=_dev()) * 3).to(dtype).requires_grad_(True)
    y = softmax_ops.softmax(x, log)
    gy = torch.randn_like(y)
    y.backward(gy)
    xf = x.detach().float().requires_grad_(True)
    ref = torch.log_softmax(xf, -1) if log else torch.softmax(xf, -1)
    ref.backward(gy.float())
    tol = (1e-4, 1e-5) if dtype == torch.float32 else (1e-2, 2e-3)
    _close(y, ref, *tol)
    _close(x.grad, xf.grad, tol[0] * 3, tol[1] * 10)


@pytest.mark.parametrize('rows,C', [(256, 1000), (40, 33278), (5, 17)])
@pytest.mark.parametrize('dtype', [torch.float32, torch.float16, torch.bfloat16])
def test_softmax_cross_entropy(rows, C, dtype):
    from mxnet_b200.ops.cuda import softmax_ops
    torch.manual_seed(3)
    x = (torch.randn(rows, C, device=_dev()) * 2).to(dtype).requires_grad_(True)
    lab = torch.randint(0, C, (rows,), device=_dev())
    loss = softmax_ops.softmax_ce(x, lab, None)
    w = torch.rand(rows, device=_dev())
    (loss * w).sum().backward()
    xf = x.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(xf, lab, reduction='none')
    (ref * w).sum().backward()
    tol = {torch.float32: (1e-4, 1e-4), torch.float16: (2e-3, 2e-3), torch.bfloat16: (2e-2, 2e-2)}[dtype]
    _close(loss, ref, *tol)
    _close(x.grad, xf.grad, tol[0] * 5, tol[1])


def test_softmax_cross_entropy_ignore_label():
    from mxnet_b200.ops.cuda import softmax_ops
    x = torch.randn(6, 11, device=_dev(), requires_grad=True)
    lab = torch.tensor([1, 3, 0, 3, 10, 3], device=_dev())
    loss = softmax_ops.softmax_ce(x, lab, 3)
    loss.sum().backward()
    assert float(loss[1]) == 0.0 and float(loss[3]) == 0.0
    assert float(x.grad[1].abs().sum()) == 0.0
    ref = torch.nn.functional.cross_entropy(x.detach(), lab, reduction='none')
    _close(loss[[0, 2, 4]], ref[[0, 2, 4]], 1e-4, 1e-5)


# ---------------------------------------------------------------------------------------- multi-tensor ops
def test_multi_mp_sgd_mom_matches_reference_rule():
    from mxnet_b200.ops.cuda import optim_ops
    torch.manual_seed(4)
    shapes = [(1000,), (64, 3, 3, 64), (7,), (20000,)] * 15      # > one table
    w32 = [torch.randn(*s, device=_dev()) for s in shapes]
    w = [t.half() for t in w32]
    g = [torch.randn(*s, device=_dev()).half() for s in shapes]
    m = [torch.randn(*s, device=_dev()) * 0.1 for s in shapes]
    lrs = [0.1 + 0.01 * (i % 3) for i in range(len(shapes))]
    wds = [1e-4 * (i % 2) for i in range(len(shapes))]
    ref_w, ref_m = [], []
    for i in range(len(shapes)):
        gr = (g[i].float() * 0.5).clamp(-1.0, 1.0) + wds[i] * w32[i]
        mm = 0.9 * m[i] - lrs[i] * gr
        ref_m.append(mm)
        ref_w.append(w32[i] + mm)
    optim_ops.multi_sgd(w, g, m, w32, lrs, wds, 0.9, 0.5, 1.0)
    for i in range(len(shapes)):
        _close(m[i], ref_m[i], 1e-5, 1e-6)
        _close(w32[i], ref_w[i], 1e-5, 1e-6)
        _close(w[i], w32[i].half(), 0, 0)        # the low-precision copy is the rounding of the kernel's own master


def test_multi_all_finite_and_sum_sq():
    from mxnet_b200.ops.cuda import optim_ops
    ts = [torch.randn(n, device=_dev()).to(dt) for n, dt in
          [(10, torch.float32), (100000, torch.float16), (33, torch.bfloat16)] * 20]
    assert float(optim_ops.multi_all_finite(ts).item()) == 1.0
    ss = optim_ops.multi_sum_sq(ts)
    ref = torch.stack([(t.float() ** 2).sum() for t in ts])
    _close(ss, ref, 1e-4, 1e-4)
    ts[37][5] = float('inf')
    assert float(optim_ops.multi_all_finite(ts).item()) == 0.0
    ts[37][5] = float('nan')
    assert float(optim_ops.multi_all_finite(ts).item()) == 0.0
    # bitwise reproducible
    a, b = optim_ops.multi_sum_sq(ts[:20]), optim_ops.multi_sum_sq(ts[:20])
    assert torch.equal(a, b)


# ---------------------------------------------------------------------------------------- tcgen05 GEMM
@pytest.mark.parametrize('M,N,K', [(128, 128, 64), (256, 256, 512), (300, 136, 72), (1, 1000, 2048), (4096, 64, 64),
                                   (130, 8, 8), (777, 264, 1032)])
@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_tcgen05_gemm_matches_fp32_reference(M, N, K, dtype):
    from mxnet_b200.ops.cuda import gemm_ops
    torch.manual_seed(5)
    a = torch.randn(M, K, device=_dev()).to(dtype)
    b = torch.randn(N, K, device=_dev()).to(dtype)
    bias = torch.randn(N, device=_dev()).to(dtype)
    d = gemm_ops.gemm_tn(a, b)
    ref = a.float() @ b.float().t()
    gemm_ops.check_errors()
    tol = (1e-2, 1e-2 * K ** 0.5) if dtype == torch.float16 else (2e-2, 4e-2 * K ** 0.5)
    _close(d, ref, *tol)
    d2 = gemm_ops.gemm_tn(a, b, bias, 'relu')
    _close(d2, torch.relu(ref + bias.float()), *tol)
    gemm_ops.check_errors()


@pytest.mark.parametrize('a_mn,b_mn', [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize('M,N,K', [(128, 128, 64), (384, 200, 136), (72, 1000, 264), (1000, 72, 520), (4096, 512, 64)])
@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_tcgen05_gemm_operand_layouts(a_mn, b_mn, M, N, K, dtype):
    """K-major and MN-major operands (stored [rows, K] or [K, rows]) in every combination."""
    from mxnet_b200.ops.cuda import gemm_ops
    torch.manual_seed(8)
    a = torch.randn(M, K, device=_dev()).to(dtype)
    b = torch.randn(N, K, device=_dev()).to(dtype)
    ref = a.float() @ b.float().t()
    a_in = a.t().contiguous() if a_mn else a
    b_in = b.t().contiguous() if b_mn else b
    d = gemm_ops.gemm(a_in, b_in, a_mn, b_mn)
    gemm_ops.check_errors()
    tol = (1e-2, 1e-2 * K ** 0.5) if dtype == torch.float16 else (2e-2, 4e-2 * K ** 0.5)
    _close(d, ref, *tol)


@pytest.mark.parametrize('a_mn,b_mn', [(False, False), (False, True), (True, True)])
@pytest.mark.parametrize('M,N,K', [(256, 256, 64), (8192, 768, 768), (304, 200, 136), (136, 72, 264), (1000, 1000, 520),
                                   (4096, 192, 1024), (640, 384, 4096)])
def test_tcgen05_gemm_cta_pair_kernel(a_mn, b_mn, M, N, K):
    """The CTA-pair kernel (256-row tiles, two SMs per tile) against an fp32 product and against the single-CTA kernel,
    on shapes with partial row tiles, partial column tiles and a partner CTA whose rows lie entirely outside."""
    from mxnet_b200.ops.cuda import gemm_ops
    torch.manual_seed(12)
    dtype = torch.float16
    a = (torch.randn(M, K, device=_dev()) / 4).to(dtype)
    b = (torch.randn(N, K, device=_dev()) / 4).to(dtype)
    bias = torch.randn(N, device=_dev()).to(dtype)
    ref = a.float() @ b.float().t() + bias.float()
    a_in = a.t().contiguous() if a_mn else a
    b_in = b.t().contiguous() if b_mn else b
    try:
        gemm_ops.set_variant(1)
        single = gemm_ops.gemm(a_in, b_in, a_mn, b_mn, bias)
        gemm_ops.set_variant(2)
        pair = gemm_ops.gemm(a_in, b_in, a_mn, b_mn, bias)
    finally:
        gemm_ops.set_variant(0)
    gemm_ops.check_errors()
    _close(pair, ref, 1e-2, 2e-3 * K ** 0.5)
    _close(pair, single, 2e-3, 1e-3 * K ** 0.5)       # same products in the same order per k-step; split-K may differ


@pytest.mark.parametrize('M,N,K', [(768, 768, 8192), (256, 136, 4096), (128, 64, 2048)])
@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_tcgen05_gemm_split_k_weight_gradient_shapes(M, N, K, dtype):
    """Few output tiles and a long contraction: the k-steps are cut evenly over the SMs (stream-K), twice in a row so that
    the second launch meets the piece counters the first one left behind."""
    from mxnet_b200.ops import cuda
    from mxnet_b200.ops.cuda import gemm_ops
    assert cuda.lib().mxb_gemm_wants_workspace(M, N, K) == 1
    torch.manual_seed(9)
    a = (torch.randn(K, M, device=_dev()) / 8).to(dtype)          # MN-major operands, as in dW = dY^T X
    b = (torch.randn(K, N, device=_dev()) / 8).to(dtype)
    bias = torch.randn(N, device=_dev()).to(dtype)
    ref = torch.relu(a.float().t() @ b.float() + bias.float())
    tol = (1e-2, 2e-2) if dtype == torch.float16 else (3e-2, 8e-2)
    for _ in range(2):
        d = gemm_ops.gemm(a, b, True, True, bias, 'relu')
        gemm_ops.check_errors()
        _close(d, ref, *tol)


@pytest.mark.parametrize('M,N,K', [(8192, 768, 3072), (24000, 256, 1024), (128 * 150, 256, 640), (200, 520, 4096),
                                   (19000, 192, 512)])
def test_tcgen05_gemm_stream_k_last_round(M, N, K):
    """Outputs whose tiles do not fill the last round of the persistent grid: whole rounds tile by tile, the rest cut by
    k-steps over all CTAs and combined by the CTA that finishes last; against an fp32 product, bias and ReLU included."""
    from mxnet_b200.ops import cuda
    from mxnet_b200.ops.cuda import gemm_ops
    torch.manual_seed(13)
    a = (torch.randn(M, K, device=_dev()) / 8).half()
    b = (torch.randn(N, K, device=_dev()) / 8).half()
    bias = torch.randn(N, device=_dev()).half()
    ref = torch.relu(a.float() @ b.float().t() + bias.float())
    for _ in range(2):
        d = gemm_ops.gemm_tn(a, b, bias, 'relu')
        gemm_ops.check_errors()
        _close(d, ref, 1e-2, 2e-2)


@pytest.mark.parametrize('ta,tb', [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize('B,M,N,K', [(3, 128, 128, 64), (5, 200, 72, 136), (12, 128, 64, 128), (2, 1024, 1024, 1024), (7, 8, 8, 8)])
@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_tcgen05_batched_gemm_and_batch_dot_gradients(ta, tb, B, M, N, K, dtype):
    """``batch_dot`` with every combination of its transpose flags on the batched tcgen05 kernel: forward and both
    gradients against fp32, with matrices whose tiles are partial (no tile may read its neighbour in the batch)."""
    from mxnet_b200 import env
    torch.manual_seed(14)
    a = (torch.randn(B, K, M, device=_dev()) if ta else torch.randn(B, M, K, device=_dev())).div(4).to(dtype)
    b = (torch.randn(B, N, K, device=_dev()) if tb else torch.randn(B, K, N, device=_dev())).div(4).to(dtype)
    af, bf = a.float().requires_grad_(True), b.float().requires_grad_(True)
    ref = torch.bmm(af.transpose(1, 2) if ta else af, bf.transpose(1, 2) if tb else bf)
    dc = (torch.randn_like(ref) / 4).to(dtype)
    ref.backward(dc.float())
    with env.scope('MXNET_B200_GEMM_AUTOTUNE', '0'):          # always the in-tree kernel
        x, y = nd.NDArray._from_tensor(a.clone(), mx.gpu(0)), nd.NDArray._from_tensor(b.clone(), mx.gpu(0))
        x.attach_grad()
        y.attach_grad()
        with autograd.record():
            c = nd.batch_dot(x, y, transpose_a=ta, transpose_b=tb)
        c.backward(nd.NDArray._from_tensor(dc, mx.gpu(0)))
    from mxnet_b200.ops.cuda import gemm_ops
    gemm_ops.check_errors()
    tol = (1e-2, 2e-3 * K ** 0.5) if dtype == torch.float16 else (3e-2, 1.5e-2 * K ** 0.5)
    _close(c._data, ref, *tol)
    _close(x.grad._data, af.grad, tol[0], tol[1] * (N / K) ** 0.5 + 1e-2)
    _close(y.grad._data, bf.grad, tol[0], tol[1] * (M / K) ** 0.5 + 1e-2)


def test_linear_autograd_through_tcgen05():
    from mxnet_b200.ops.cuda import gemm_ops
    torch.manual_seed(6)
    x = torch.randn(64, 256, device=_dev()).half().requires_grad_(True)
    w = (torch.randn(128, 256, device=_dev()) * 0.1).half().requires_grad_(True)
    b = torch.randn(128, device=_dev()).half().requires_grad_(True)
    y = gemm_ops.LinearFn.apply(x, w, b, None)
    gy = torch.randn_like(y)
    y.backward(gy)
    xf, wf, bf = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    ref = torch.nn.functional.linear(xf, wf, bf)
    ref.backward(gy.float())
    _close(y, ref, 1e-2, 5e-2)
    _close(x.grad, xf.grad, 2e-2, 5e-2)
    _close(w.grad, wf.grad, 2e-2, 1e-1)
    _close(b.grad, bf.grad, 2e-2, 1e-1)
    gemm_ops.check_errors()


# ---------------------------------------------------------------------------------------- fused optimizer step
def _tiny_net(ctx, dtype):
    from mxnet_b200.gluon import nn
    net = nn.HybridSequential()
    net.add(nn.Dense(64, activation='relu', in_units=32), nn.Dense(10, in_units=64))
    net.initialize(mx.init.Xavier(), ctx=ctx)
    if dtype != 'float32':
        net.cast(dtype)
    return net


@pytest.mark.parametrize('dtype', ['float16', 'float32'])
def test_fused_step_matches_multi_precision_sgd(dtype):
    ctx = mx.gpu(0)
    net = _tiny_net(ctx, dtype)
    params = list(net.collect_params().values())
    ref_w = [p.data(ctx)._data.detach().float().clone() for p in params]
    ref_m = [torch.zeros_like(w) for w in ref_w]
    trainer = gluon.Trainer(net.collect_params(), 'sgd', {'learning_rate': 0.05, 'momentum': 0.9, 'wd': 1e-3,
                                                          'multi_precision': dtype != 'float32'}, kvstore='device')
    loss_fn = gluon.loss.SoftmaxCrossEntropyLoss()
    x = nd.array(np.random.randn(16, 32).astype(dtype), ctx=ctx, dtype=dtype)
    y = nd.array(np.random.randint(0, 10, (16,)), ctx=ctx)
    for step in range(4):
        with autograd.record():
            loss = loss_fn(net(x), y)
        loss.backward()
        grads = [p.grad(ctx)._data.detach().float().clone() for p in params]
        trainer.step(16)
        assert trainer._fused is not None
        for w, m, g in zip(ref_w, ref_m, grads):
            gr = g / 16 + 1e-3 * w
            m.mul_(0.9).add_(gr, alpha=-0.05)
            w.add_(m)
        for p, w in zip(params, ref_w):
            tol = (1e-5, 1e-6) if dtype == 'float32' else (2e-3, 2e-3)
            _close(p.data(ctx)._data, w, *tol)
            # the step clears the gradient arena
            assert float(p.grad(ctx)._data.abs().sum()) == 0.0


@pytest.mark.parametrize('name,kwargs', [('adam', {'learning_rate': 0.01, 'wd': 0.01}),
                                         ('adamw', {'learning_rate': 0.01, 'wd': 0.1}),
                                         ('lamb', {'learning_rate': 0.01, 'wd': 0.01}),
                                         ('lamb', {'learning_rate': 0.01, 'wd': 0.01, 'lower_bound': 0.5, 'upper_bound': 2.0}),
                                         ('nag', {'learning_rate': 0.05, 'momentum': 0.9, 'wd': 1e-3})])
def test_fused_step_matches_generic_optimizer(name, kwargs):
    """The fused kernels against the per-parameter optimizer path of the same framework, fp32 weights."""
    from mxnet_b200 import env
    ctx = mx.gpu(0)
    results = []
    for fused in (True, False):
        with env.scope('MXNET_KVSTORE_FUSED', '1' if fused else '0'):
            mx.random.seed(3)
            np.random.seed(3)
            net = _tiny_net(ctx, 'float32')
            trainer = gluon.Trainer(net.collect_params(), name, dict(kwargs), kvstore='device')
            loss_fn = gluon.loss.SoftmaxCrossEntropyLoss()
            rng = np.random.RandomState(5)
            for step in range(5):
                x = nd.array(rng.randn(16, 32).astype('float32'), ctx=ctx)
                y = nd.array(rng.randint(0, 10, (16,)), ctx=ctx)
                with autograd.record():
                    loss = loss_fn(net(x), y)
                loss.backward()
                trainer.step(16)
            assert (trainer._fused is not None) == fused
            results.append([p.data(ctx)._data.detach().clone() for p in net.collect_params().values()])
    for a, b in zip(*results):
        _close(a, b, 2e-4, 2e-5)


def test_amp_unscale_then_step_divides_by_the_loss_scale_once():
    """``amp.unscale(trainer)`` (the documented flow for clipping gradients by hand) followed by ``trainer.step`` on the
    fused path: the step must not divide by the loss scale a second time.  Checked on the first step (scale still on the
    host) and on later ones (scale on the device) against fp32 training without AMP."""
    from mxnet_b200 import amp, env
    ctx = mx.gpu(0)
    rng = np.random.RandomState(21)
    xs = [rng.randn(16, 32).astype('float32') for _ in range(3)]
    ys = [rng.randint(0, 10, (16,)) for _ in range(3)]
    loss_fn = gluon.loss.SoftmaxCrossEntropyLoss()

    def train(use_amp):
        mx.random.seed(3)
        np.random.seed(3)
        net = _tiny_net(ctx, 'float32')
        trainer = gluon.Trainer(net.collect_params(), 'sgd', {'learning_rate': 0.1}, kvstore='device')
        if use_amp:
            amp.init_trainer(trainer)
        for x, y in zip(xs, ys):
            with autograd.record():
                loss = loss_fn(net(nd.array(x, ctx=ctx)), nd.array(y, ctx=ctx))
                if use_amp:
                    with amp.scale_loss(loss, trainer) as scaled:
                        autograd.backward(scaled)
                else:
                    loss.backward()
            if use_amp:
                amp.unscale(trainer)
                g = net.collect_params()
                assert max(float(p.grad(ctx).abs().max().asscalar()) for p in g.values()) < 100.0   # really unscaled
            trainer.step(16)
        assert trainer._fused is not None
        return [p.data(ctx).asnumpy() for p in net.collect_params().values()]
    ref = train(False)
    amp._reset()
    amp.init('float16', target_precision_ops=[], fp32_ops=[])      # loss scaling only: the arithmetic stays fp32
    try:
        got = train(True)
    finally:
        amp._reset()
    for a, b in zip(got, ref):
        np.testing.assert_allclose(a, b, rtol=2e-4, atol=2e-5)


def test_fused_step_skips_stale_parameters_and_follows_multiplier_changes():
    """``step(ignore_stale_grad=True)`` leaves a parameter without a fresh gradient untouched (no weight decay, no
    momentum drift), and a changed ``lr_mult`` takes effect: both against the generic per-parameter path."""
    from mxnet_b200 import env
    from mxnet_b200.gluon import nn
    ctx = mx.gpu(0)
    results = []
    for fused in (True, False):
        with env.scope('MXNET_KVSTORE_FUSED', '1' if fused else '0'):
            mx.random.seed(4)
            np.random.seed(4)
            used, unused = nn.Dense(8, in_units=16), nn.Dense(4, in_units=16)
            for blk in (used, unused):
                blk.initialize(mx.init.Xavier(), ctx=ctx)
            params = list(used.collect_params().values()) + list(unused.collect_params().values())
            trainer = gluon.Trainer(params, 'adam', {'learning_rate': 0.05, 'wd': 0.1}, kvstore='device')
            rng = np.random.RandomState(6)
            for step in range(4):
                x = nd.array(rng.randn(8, 16).astype('float32'), ctx=ctx)
                with autograd.record():
                    out = used(x) if step != 1 else (used(x).sum() + unused(x).sum())
                    loss = (out * out).sum() if step != 1 else out * out
                loss.backward()
                if step == 2:
                    used.weight.lr_mult = 0.25
                trainer.step(8, ignore_stale_grad=(step != 1))
            assert (trainer._fused is not None) == fused
            with autograd.record():
                loss = (used(x) * 2).sum()
            loss.backward()
            with pytest.raises(UserWarning):
                trainer.step(8)                      # a stale gradient is an error unless the caller says otherwise
            results.append([p.data(ctx).asnumpy() for p in params])
    for a, b in zip(*results):
        np.testing.assert_allclose(a, b, rtol=2e-4, atol=2e-5)


def test_fused_step_states_round_trip(tmp_path):
    ctx = mx.gpu(0)
    net = _tiny_net(ctx, 'float32')
    trainer = gluon.Trainer(net.collect_params(), 'lamb', {'learning_rate': 0.01}, kvstore='device')
    x, y = nd.array(np.random.randn(8, 32).astype('float32'), ctx=ctx), nd.array(np.random.randint(0, 10, (8,)), ctx=ctx)
    loss_fn = gluon.loss.SoftmaxCrossEntropyLoss()
    for _ in range(2):
        with autograd.record():
            loss = loss_fn(net(x), y)
        loss.backward()
        trainer.step(8)
    f = str(tmp_path / 'lamb.states')
    trainer.save_states(f)
    mean0 = trainer._fused.mom.clone()
    trainer._fused.mom.zero_()
    trainer._fused.var.zero_()
    trainer.load_states(f)
    assert torch.equal(trainer._fused.mom, mean0) and float(trainer._fused.var.abs().sum()) > 0


def test_fused_step_skips_on_overflow_and_halves_loss_scale():
    from mxnet_b200 import amp
    ctx = mx.gpu(0)
    amp._reset()
    amp.init('float16')
    try:
        net = _tiny_net(ctx, 'float16')
        trainer = gluon.Trainer(net.collect_params(), 'sgd', {'learning_rate': 0.1, 'momentum': 0.9,
                                                              'multi_precision': True}, kvstore='device')
        amp.init_trainer(trainer)
        assert trainer._fused is not None
        loss_fn = gluon.loss.SoftmaxCrossEntropyLoss()
        x = nd.array(np.random.randn(8, 32).astype('float16'), ctx=ctx, dtype='float16')
        y = nd.array(np.random.randint(0, 10, (8,)), ctx=ctx)
        before = [p.data(ctx)._data.clone() for p in net.collect_params().values()]
        with autograd.record():
            loss = loss_fn(net(x), y)
            with amp.scale_loss(loss, trainer) as scaled:
                autograd.backward(scaled)
        next(iter(net.collect_params().values())).grad(ctx)._data.view(-1)[0] = float('inf')
        trainer.step(8)
        torch.cuda.synchronize()
        state = trainer._fused.scale_state.cpu()
        assert float(state[0]) == 2. ** 15 and float(state[2]) == 1.0
        for p, b in zip(net.collect_params().values(), before):
            assert torch.equal(p.data(ctx)._data, b)
        # the scale keeps halving on overflowing steps; the first clean step updates the weights
        changed = False
        for _ in range(16):
            with autograd.record():
                loss = loss_fn(net(x), y)
                with amp.scale_loss(loss, trainer) as scaled:
                    autograd.backward(scaled)
            trainer.step(8)
            torch.cuda.synchronize()
            changed = any(not torch.equal(p.data(ctx)._data, b) for p, b in zip(net.collect_params().values(), before))
            if changed:
                break
        st = trainer._fused.scale_state.cpu()
        assert changed and float(st[1]) == 1.0 and float(st[0]) == 2. ** 16 / 2. ** float(st[2])
    finally:
        amp._reset()


def test_device_wait_times_out_with_status_not_a_hang():
    ctx = mx.gpu(0)
    net = _tiny_net(ctx, 'float32')
    trainer = gluon.Trainer(net.collect_params(), 'sgd', {'learning_rate': 0.1}, kvstore='device')
    trainer._init_kvstore()
    assert trainer._fused is not None
    code = trainer._fused.wait_probe(timeout_ms=20)
    assert code == 1            # kErrWaitReady: the wait gave up and reported, the context is still usable
    assert float(torch.ones(4, device='cuda').sum()) == 4.0


# ---------------------------------------------------------------------------------------- attention
def _attention_reference(qkv, mask, heads):
    N, T, C3 = qkv.shape
    C = C3 // 3
    x = qkv.float().reshape(N, T, 3, heads, C // heads)
    q, k, v = (x[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    s = q @ k.transpose(-1, -2) / (C // heads) ** 0.5
    if mask is not None:
        s = s.masked_fill((mask == 0)[:, None, None, :], float('-inf'))
    return (torch.softmax(s, -1) @ v).permute(0, 2, 1, 3).reshape(N, T, C)


@pytest.mark.parametrize('N,T,heads', [(2, 128, 2), (3, 100, 12), (1, 17, 1), (5, 128, 4),
                                       (2, 256, 2), (1, 200, 3), (2, 384, 1), (2, 512, 4), (1, 129, 1), (1, 1000, 2)])   # T > 128: streaming kernels
@pytest.mark.parametrize('use_mask', [False, True])
@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_fused_self_attention_matches_reference(N, T, heads, use_mask, dtype):
    from mxnet_b200.ops.cuda import attn_ops
    torch.manual_seed(12)
    C = heads * 64
    qkv = (torch.randn(N, T, 3 * C, device=_dev()) * 0.7).to(dtype).requires_grad_(True)
    mask = None
    if use_mask:
        lens = torch.randint(1, T + 1, (N,), device=_dev())
        mask = (torch.arange(T, device=_dev())[None, :] < lens[:, None]).float()
    assert attn_ops.supported(qkv, heads)
    out = attn_ops.fused_self_attention(qkv, mask, heads, 0.0)
    g = torch.randn_like(out)
    out.backward(g)
    attn_ops.check_errors()
    ref_in = qkv.detach().float().requires_grad_(True)
    ref = _attention_reference(ref_in, mask, heads)
    ref.backward(g.float())
    tol = (2e-2, 2e-2) if dtype == torch.float16 else (6e-2, 6e-2)
    _close(out, ref, *tol)
    _close(qkv.grad, ref_in.grad, tol[0] * 2, tol[1] * 2)


@pytest.mark.parametrize('T', [128, 320])
def test_fused_self_attention_dropout_is_unbiased_and_consistent(T):
    from mxnet_b200.ops.cuda import attn_ops
    torch.manual_seed(13)
    N, heads, C = 4, 4, 256
    qkv = torch.zeros(N, T, 3 * C, device=_dev(), dtype=torch.float16)
    qkv[:, :, 2 * C:] = 1.0                                   # V = 1, Q = K = 0: out = sum of kept weights / (1 - p)
    out = attn_ops.fused_self_attention(qkv, None, heads, 0.5)
    attn_ops.check_errors()
    o = out.float()
    assert abs(float(o.mean()) - 1.0) < 0.02 and 0.05 < float(o.std()) < 0.2
    # with the dropout word pinned, forward is linear in V and backward is its adjoint: <dV, W> == <g, f(W)>
    base = (torch.randn(N, T, 3 * C, device=_dev()) * 0.5).half()
    state = attn_ops._seed[_dev()]

    def run(v_block, need_grad=False):
        state.fill_(1234567)
        x = base.clone()
        x[:, :, 2 * C:] = v_block
        x.requires_grad_(need_grad)
        return x, attn_ops.fused_self_attention(x, None, heads, 0.3)
    v1 = (torch.randn(N, T, C, device=_dev()) * 0.5).half()
    w = (torch.randn(N, T, C, device=_dev()) * 0.5).half()
    x, y = run(v1, True)
    g = torch.randn_like(y)
    y.backward(g)
    dv = x.grad[:, :, 2 * C:].float()
    _, fw = run(w)
    lhs, rhs = float((dv * w.float()).sum()), float((g.float() * fw.float()).sum())
    assert abs(lhs - rhs) < 2e-2 * max(1.0, abs(rhs))
    _, y2 = run(v1)
    assert torch.equal(y, y2)                                  # same word, same pattern


# ---------------------------------------------------------------------------------------- gradient compression
@pytest.mark.parametrize('kind,threshold', [('2bit', 0.5), ('1bit', 0.0)])
@pytest.mark.parametrize('n', [1, 15, 16, 33, 100003])
def test_gradient_compression_kernels_match_tensor_ops(kind, threshold, n):
    from mxnet_b200 import env
    from mxnet_b200.kvstore.gradient_compression import GradientCompression
    if kind == '1bit':
        threshold = 0.3
    torch.manual_seed(10)
    gk, gt = GradientCompression(kind, threshold), GradientCompression(kind, threshold)
    for step in range(3):                       # the residual carries over between steps
        g = torch.randn(n, device=_dev())
        pk = gk.quantize('k', g)
        with env.scope('MXNET_B200_KERNELS', '0'):
            pt = gt.quantize('k', g)
        assert pk.dtype == torch.int32 and pk.numel() == gk.compressed_size(n)
        assert torch.equal(pk.to(torch.int64) & 0xFFFFFFFF, pt)
        assert torch.equal(gk._residual['k'], gt._residual['k'])
        dk = gk.dequantize(pk, n)
        with env.scope('MXNET_B200_KERNELS', '0'):
            dt_ = gt.dequantize(pt, n)
        assert torch.equal(dk, dt_)


# ---------------------------------------------------------------------------------------- LSTM
@pytest.mark.parametrize('T,B,I,H,layers', [(5, 3, 8, 32, 1), (7, 4, 24, 40, 2), (35, 80, 650, 650, 2), (3, 1, 16, 200, 1),
                                             (4, 33, 64, 888, 1)])
@pytest.mark.parametrize('dtype', [torch.float32, torch.float16])
@pytest.mark.parametrize('tc', ['cluster', 'plain', False])
def test_fused_lstm_matches_library_lstm(T, B, I, H, layers, dtype, tc, monkeypatch, request):
    """tc='cluster' / 'plain': the tcgen05 recurrence (tf32 products for fp32 models), its backward pass with the contraction
    cut over clusters of four CTAs or with the plain kernel; tc=False: the fp32-pipe recurrence kernels."""
    from mxnet_b200.ops.cuda import rnn_ops, lib
    from mxnet_b200.ops.nn import rnn_param_size
    monkeypatch.setenv('MXNET_B200_RNN_TC', '1' if tc else '0')
    lib().mxb_lstm_tc_set_backward_variant(1 if tc == 'plain' else 0)
    request.addfinalizer(lambda: lib().mxb_lstm_tc_set_backward_variant(0))
    assert rnn_ops.tc_supported(dtype, B, H) == bool(tc)
    torch.manual_seed(9)
    ref = torch.nn.LSTM(I, H, layers).float()            # exact fp32 reference on the host
    # flat parameter vector in the RNN operator's order: all weights (layer by layer: w_ih, w_hh), then all biases
    ws, bs = [], []
    for l in range(layers):
        ws += [getattr(ref, 'weight_ih_l%d' % l).detach().reshape(-1), getattr(ref, 'weight_hh_l%d' % l).detach().reshape(-1)]
        bs += [getattr(ref, 'bias_ih_l%d' % l).detach(), getattr(ref, 'bias_hh_l%d' % l).detach()]
    flat = torch.cat(ws + bs).to(_dev()).to(dtype).requires_grad_(True)
    assert flat.numel() == rnn_param_size('lstm', layers, I, H)
    x = torch.randn(T, B, I, device=_dev()).to(dtype).requires_grad_(True)
    h0 = (torch.randn(layers, B, H, device=_dev()) * 0.5).to(dtype).requires_grad_(True)
    c0 = (torch.randn(layers, B, H, device=_dev()) * 0.5).to(dtype).requires_grad_(True)
    assert rnn_ops.supported(x, H, layers)
    y, hT, cT = rnn_ops.lstm(x, flat, h0, c0, H, layers, 0.0, True)
    gy, gh, gc = torch.randn_like(y), torch.randn_like(hT), torch.randn_like(cT)
    torch.autograd.backward([y, hT, cT], [gy, gh, gc])
    # reference in fp32 on the same (rounded) values
    with torch.no_grad():
        off = 0
        for l in range(layers):
            for name, shape in (('weight_ih_l%d' % l, (4 * H, I if l == 0 else H)), ('weight_hh_l%d' % l, (4 * H, H))):
                n = shape[0] * shape[1]
                getattr(ref, name).copy_(flat[off:off + n].float().reshape(shape).cpu())
                off += n
        for l in range(layers):
            for name in ('bias_ih_l%d' % l, 'bias_hh_l%d' % l):
                getattr(ref, name).copy_(flat[off:off + 4 * H].float().cpu())
                off += 4 * H
    xr = x.detach().float().cpu().requires_grad_(True)
    hr, cr = h0.detach().float().cpu().requires_grad_(True), c0.detach().float().cpu().requires_grad_(True)
    yr, (hTr, cTr) = ref(xr, (hr, cr))
    torch.autograd.backward([yr, hTr, cTr], [gy.float().cpu(), gh.float().cpu(), gc.float().cpu()])
    tol = (1e-3, 1e-3) if dtype == torch.float32 else (3e-2, 3e-2)     # fast exp/tanh intrinsics in the kernel
    if tc and dtype == torch.float32:
        tol = (6e-3, 6e-3)                  # tf32 operands: 10 mantissa bits in the recurrent product
    _close(y, yr, *tol)
    _close(hT, hTr, *tol)
    _close(cT, cTr, *tol)
    _close(x.grad, xr.grad, tol[0] * 3, tol[1] * 3)
    _close(h0.grad, hr.grad, tol[0] * 3, tol[1] * 3)
    _close(c0.grad, cr.grad, tol[0] * 3, tol[1] * 3)
    gref = torch.cat([getattr(ref, 'weight_%s_l%d' % (k, l)).grad.reshape(-1) for l in range(layers) for k in ('ih', 'hh')] +
                     [getattr(ref, 'bias_%s_l%d' % (k, l)).grad for l in range(layers) for k in ('ih', 'hh')])
    scale = float(gref.abs().max())
    _close(flat.grad.cpu() / scale, gref / scale, tol[0] * 5, tol[1] * 2)


@pytest.mark.parametrize('T,B,I,H,layers', [(6, 4, 24, 40, 2), (5, 3, 16, 16, 1)])
def test_fused_lstm_bidirectional(T, B, I, H, layers):
    """Both directions through the recurrence kernel (the reverse one on the time-flipped sequence) against an exact
    fp32 bidirectional LSTM on the host with the same parameters."""
    from mxnet_b200.ops.cuda import rnn_ops
    from mxnet_b200.ops.nn import rnn_param_size
    torch.manual_seed(11)
    ref = torch.nn.LSTM(I, H, layers, bidirectional=True).float()
    sfx = ['l%d%s' % (l, r) for l in range(layers) for r in ('', '_reverse')]
    ws = [getattr(ref, 'weight_%s_%s' % (k, s)).detach().reshape(-1) for s in sfx for k in ('ih', 'hh')]
    bs = [getattr(ref, 'bias_%s_%s' % (k, s)).detach() for s in sfx for k in ('ih', 'hh')]
    flat = torch.cat(ws + bs).to(_dev()).requires_grad_(True)
    assert flat.numel() == rnn_param_size('lstm', layers, I, H, True)
    x = torch.randn(T, B, I, device=_dev()).requires_grad_(True)
    h0 = (torch.randn(layers * 2, B, H, device=_dev()) * 0.5).requires_grad_(True)
    c0 = (torch.randn(layers * 2, B, H, device=_dev()) * 0.5).requires_grad_(True)
    assert rnn_ops.supported(x, H, layers)
    y, hT, cT = rnn_ops.lstm(x, flat, h0, c0, H, layers, 0.0, True, True)
    assert y.shape == (T, B, 2 * H)
    gy, gh, gc = torch.randn_like(y), torch.randn_like(hT), torch.randn_like(cT)
    torch.autograd.backward([y, hT, cT], [gy, gh, gc])
    xr = x.detach().cpu().requires_grad_(True)
    hr, cr = h0.detach().cpu().requires_grad_(True), c0.detach().cpu().requires_grad_(True)
    yr, (hTr, cTr) = ref(xr, (hr, cr))
    torch.autograd.backward([yr, hTr, cTr], [gy.cpu(), gh.cpu(), gc.cpu()])
    for a, b in ((y, yr), (hT, hTr), (cT, cTr)):
        _close(a, b, 1e-3, 1e-3)
    for a, b in ((x.grad, xr.grad), (h0.grad, hr.grad), (c0.grad, cr.grad)):
        _close(a, b, 3e-3, 3e-3)
    gref = torch.cat([getattr(ref, 'weight_%s_%s' % (k, s)).grad.reshape(-1) for s in sfx for k in ('ih', 'hh')] +
                     [getattr(ref, 'bias_%s_%s' % (k, s)).grad for s in sfx for k in ('ih', 'hh')])
    scale = float(gref.abs().max())
    _close(flat.grad.cpu() / scale, gref / scale, 5e-3, 2e-3)


@pytest.mark.parametrize('mode', ['gru', 'rnn_tanh', 'rnn_relu'])
@pytest.mark.parametrize('T,B,I,H,layers,bidir', [(6, 4, 24, 40, 2, False), (5, 3, 16, 16, 1, True), (12, 33, 64, 300, 1, False)])
@pytest.mark.parametrize('dtype', [torch.float32, torch.float16])
@pytest.mark.parametrize('tc', [True, False])
def test_gru_and_vanilla_rnn_kernels(mode, T, B, I, H, layers, bidir, dtype, tc, monkeypatch):
    """The GRU / vanilla RNN recurrence kernels against an exact fp32 module on the host with the same parameters.  tc=True:
    the GRU recurrence of layers with 32 units or more runs on the tensor cores (gru_tc.inl); tc=False: fp32-pipe kernels."""
    from mxnet_b200.ops.cuda import rnn_ops
    from mxnet_b200.ops.nn import rnn_param_size
    if tc and mode != 'gru':
        pytest.skip('only the LSTM and the GRU have a tensor-core recurrence')
    monkeypatch.setenv('MXNET_B200_RNN_TC', '1' if tc else '0')
    assert rnn_ops.gru_tc_supported(dtype, B, H) == bool(tc and H >= 32)
    on_tc = tc and H >= 32
    torch.manual_seed(13)
    if mode == 'gru':
        ref = torch.nn.GRU(I, H, layers, bidirectional=bidir).float()
    else:
        ref = torch.nn.RNN(I, H, layers, nonlinearity=mode[4:], bidirectional=bidir).float()
    d = 2 if bidir else 1
    sfx = ['l%d%s' % (l, r) for l in range(layers) for r in (('', '_reverse') if bidir else ('',))]
    names = [('weight_%s_%s' % (k, s_)) for s_ in sfx for k in ('ih', 'hh')] + [('bias_%s_%s' % (k, s_)) for s_ in sfx for k in ('ih', 'hh')]
    flat = torch.cat([getattr(ref, n).detach().reshape(-1) for n in names]).to(_dev()).to(dtype).requires_grad_(True)
    assert flat.numel() == rnn_param_size(mode, layers, I, H, bidir)
    with torch.no_grad():                              # the reference sees the rounded parameters
        off = 0
        for n in names:
            w = getattr(ref, n)
            w.copy_(flat[off:off + w.numel()].float().reshape(w.shape).cpu())
            off += w.numel()
    x = torch.randn(T, B, I, device=_dev()).to(dtype).requires_grad_(True)
    h0 = (torch.randn(layers * d, B, H, device=_dev()) * 0.5).to(dtype).requires_grad_(True)
    assert rnn_ops.supported(x, H, layers)
    y, hT = rnn_ops.recurrent(mode, x, flat, h0, H, layers, 0.0, True, bidir)
    gy, gh = torch.randn_like(y), torch.randn_like(hT)
    torch.autograd.backward([y, hT], [gy, gh])
    xr, hr = x.detach().float().cpu().requires_grad_(True), h0.detach().float().cpu().requires_grad_(True)
    yr, hTr = ref(xr, hr)
    torch.autograd.backward([yr, hTr], [gy.float().cpu(), gh.float().cpu()])
    tol = (1e-3, 1e-3) if dtype == torch.float32 else (3e-2, 3e-2)
    if on_tc and dtype == torch.float32:
        tol = (6e-3, 6e-3)                  # tf32 operands: 10 mantissa bits in the recurrent product
    _close(y, yr, *tol)
    _close(hT, hTr, *tol)
    scale = max(1.0, float(xr.grad.abs().max()))
    _close(x.grad / scale, xr.grad / scale, tol[0] * 3, tol[1] * 3)
    _close(h0.grad / scale, hr.grad / scale, tol[0] * 3, tol[1] * 3)
    gref = torch.cat([getattr(ref, n).grad.reshape(-1) for n in names])
    scale = float(gref.abs().max())
    _close(flat.grad.cpu() / scale, gref / scale, tol[0] * 5, tol[1] * 2)


@pytest.mark.parametrize('mode,bidir', [('gru', False), ('lstm', True), ('rnn_tanh', True), ('rnn_relu', False)])
def test_rnn_operator_gpu_matches_cpu_unrolled(mode, bidir):
    """The RNN operator on the GPU (recurrence kernels, library recurrence, and the timed choice between them) against
    the per-step CPU implementation of the same operator."""
    from mxnet_b200.ops.nn import rnn_param_size
    T, B, I, H, layers = 6, 3, 5, 7, 2
    d = 2 if bidir else 1
    rng = np.random.RandomState(3)
    params = (rng.randn(rnn_param_size(mode, layers, I, H, bidir)) * 0.3).astype('float32')
    x = rng.randn(T, B, I).astype('float32')
    h0 = rng.randn(layers * d, B, H).astype('float32')
    c0 = rng.randn(layers * d, B, H).astype('float32')
    outs = []
    from mxnet_b200 import env
    from mxnet_b200.ops.cuda import rnn_ops
    for ctx, flag in ((mx.cpu(), 'auto'), (mx.gpu(0), '1'), (mx.gpu(0), '0'), (mx.gpu(0), 'auto')):
        with env.scope('MXNET_B200_RNN', flag):
            args = [nd.array(x, ctx=ctx), nd.array(params, ctx=ctx), nd.array(h0, ctx=ctx)]
            if mode == 'lstm':
                args.append(nd.array(c0, ctx=ctx))
            args[0].attach_grad()
            args[1].attach_grad()
            with autograd.record():
                res = nd.RNN(*args, state_size=H, num_layers=layers, mode=mode, bidirectional=bidir, state_outputs=True)
                loss = sum((r * r).sum() for r in res)
            loss.backward()
            outs.append([r.asnumpy() for r in res] + [args[0].grad.asnumpy(), args[1].grad.asnumpy()])
    key = (mode, 'torch.float32', T, B, I, H, layers, bidir, True)
    assert key in rnn_ops.tuned_choices()                           # the auto run timed both implementations
    for other in outs[1:]:
        for a, b in zip(outs[0], other):
            np.testing.assert_allclose(a, b, rtol=1e-2, atol=1e-2)      # the library recurrence may use TF32


# ---------------------------------------------------------------------------------------- pooling
@pytest.mark.parametrize('shape,k,s,p,ceil', [((2, 13, 17, 16), 3, 2, 1, False), ((3, 8, 8, 64), 2, 2, 0, False),
                                              ((1, 9, 11, 8), 3, 1, 1, False), ((2, 10, 10, 24), 3, 2, 0, True),
                                              ((4, 112, 112, 64), 3, 2, 1, False)])
@pytest.mark.parametrize('dtype', [torch.float16, torch.bfloat16])
def test_maxpool_nhwc(shape, k, s, p, ceil, dtype):
    from mxnet_b200.ops.cuda import pool_ops
    torch.manual_seed(7)
    x = torch.randn(*shape, device=_dev()).to(dtype).requires_grad_(True)
    y = pool_ops.max_pool2d_nhwc(x, (k, k), (s, s), (p, p), ceil)
    gy = torch.randn_like(y)
    y.backward(gy)
    xf = x.detach().float().permute(0, 3, 1, 2).requires_grad_(True)
    ref = torch.nn.functional.max_pool2d(xf, k, s, p, 1, ceil)
    ref.backward(gy.float().permute(0, 3, 1, 2))
    assert tuple(y.shape) == tuple(ref.permute(0, 2, 3, 1).shape)
    _close(y, ref.permute(0, 2, 3, 1), 0, 0)
    _close(x.grad, xf.grad.permute(0, 2, 3, 1), 1e-2, 1e-2)


# ---------------------------------------------------------------------------------------- model-level checks
def _flip_tolerant_close(got, ref, tol, max_bad_frac, what):
    """Element-wise closeness that tolerates a bounded share of outliers plus a bound on the relative L2 error.

    A half-precision value that lands on the other side of a ReLU edge than the fp32 oracle switches one mask bit, and
    that changes whole gradient elements downstream; such flips are rare, so they are bounded by count, while the norm
    bound still catches a wrong kernel."""
    err = np.abs(got - ref)
    bad = err > (tol + tol * np.abs(ref))
    frac = float(bad.mean())
    rel = float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-12))
    assert frac <= max_bad_frac, '%s: %.4f of the elements differ by more than %g (max err %g)' % (what, frac, tol, err.max())
    assert rel <= 5e-2, '%s: relative L2 error %g' % (what, rel)


@pytest.mark.parametrize('downsample,cin', [(True, 32), (False, 64)])
def test_resnet_block_kernels_match_fp32_oracle(downsample, cin):
    """Both half-precision paths of a bottleneck block (in-tree kernels, library kernels) against an fp32 evaluation of
    the same block with the same weights: the down-sampling block, and the identity block whose first convolution and
    skip connection are one operator (skip gradient added in the data-gradient epilogue)."""
    from mxnet_b200 import env
    from mxnet_b200.gluon.model_zoo.vision.resnet import BottleneckV1
    ctx = mx.gpu(0)
    blk = BottleneckV1(64, 1, downsample, in_channels=cin, layout='NHWC', fused=True, v1b=True)
    blk.initialize(mx.init.Xavier(), ctx=ctx)
    for p in blk.collect_params().values():
        if p.grad_req != 'null':
            p.cast('float16')
    x = nd.array(np.random.randn(4, 8, 8, cin).astype('float16'), ctx=ctx, dtype='float16')
    blk(x)                       # finishes the deferred initialisation of the BatchNorm parameters

    def run(flag, dtype):
        with env.scope('MXNET_B200_KERNELS', flag), env.scope('MXNET_B200_CONV', '1'):      # every direction in-tree
            xx = x.astype(dtype)
            xx.attach_grad()
            for p in blk.collect_params().values():
                if p.grad_req == 'null':
                    p.set_data(nd.zeros(p.shape, ctx=ctx) if 'mean' in p.name else nd.ones(p.shape, ctx=ctx))
            with autograd.record():
                y = blk(xx)
            y.backward(nd.ones(y.shape, ctx=ctx, dtype=dtype))
            return y.asnumpy().astype('float32'), xx.grad.asnumpy().astype('float32')

    half = {flag: run(flag, 'float16') for flag in ('1', '0')}
    for p in blk.collect_params().values():
        if p.grad_req != 'null':
            p.cast('float32')
    ref_y, ref_dx = run('0', 'float32')
    for flag, (y, dx) in half.items():
        _flip_tolerant_close(y, ref_y, 3e-2, 0.002, 'y (MXNET_B200_KERNELS=%s)' % flag)
        _flip_tolerant_close(dx, ref_dx, 6e-2, 0.03, 'dx (MXNET_B200_KERNELS=%s)' % flag)


def test_hybridize_cuda_graph_matches_eager():
    from mxnet_b200.gluon import nn
    ctx = mx.gpu(0)
    net = nn.HybridSequential()
    net.add(nn.Dense(64, activation='relu', in_units=32), nn.LayerNorm(in_channels=64), nn.Dense(8, in_units=64))
    net.initialize(mx.init.Xavier(), ctx=ctx)
    x = nd.array(np.random.randn(16, 32).astype('float32'), ctx=ctx)
    with autograd.record():
        ref = net(x)
    ref.backward()
    ref_out = ref.asnumpy()
    ref_grads = [p.grad(ctx).asnumpy().copy() for p in net.collect_params().values()]
    net.hybridize(static_alloc=True, static_shape=True)
    for it in range(4):              # eager first call, warm-up, capture, replay
        with autograd.record():
            out = net(x)
        out.backward()
        np.testing.assert_allclose(out.asnumpy(), ref_out, rtol=1e-5, atol=1e-6)
        for p, g in zip(net.collect_params().values(), ref_grads):
            np.testing.assert_allclose(p.grad(ctx).asnumpy(), g, rtol=1e-4, atol=1e-5)
    assert net._cached_op is not None and not net._cached_op._disabled and len(net._cached_op._graphs) == 1


@pytest.mark.parametrize('M,N,K', [(1, 16, 16), (128, 128, 128), (130, 200, 144), (64, 1000, 2048), (1024, 1024, 1024),
                                   (300, 77, 4096), (4096, 512, 16)])
@pytest.mark.parametrize('with_bias', [False, True])
def test_tcgen05_int8_gemm_is_exact(M, N, K, with_bias):
    """``tcgen05.mma.kind::i8``: int8 x int8 products with int32 accumulation are exact, so the result must equal the
    integer reference bit for bit (fp64 matmul of the same integers is exact for these sizes), bias included; full
    range values (-128 .. 127) are used."""
    from mxnet_b200.ops.cuda import gemm_ops
    g = torch.Generator(device='cuda').manual_seed(M * 7 + N * 3 + K)
    a = torch.randint(-128, 128, (M, K), device='cuda', generator=g, dtype=torch.int32).to(torch.int8)
    b = torch.randint(-128, 128, (N, K), device='cuda', generator=g, dtype=torch.int32).to(torch.int8)
    bias = torch.randint(-100000, 100000, (N,), device='cuda', generator=g, dtype=torch.int32) if with_bias else None
    assert gemm_ops.gemm_i8_supported(a, b)
    d = gemm_ops.gemm_i8(a, b, bias)
    torch.cuda.synchronize()
    assert int(gemm_ops._error_flag(a.device).item()) == 0
    ref = torch.matmul(a.double(), b.double().t())
    if with_bias:
        ref = ref + bias.double()
    assert torch.equal(d, ref.to(torch.int32))


def test_quantized_fully_connected_runs_on_the_int8_kernel():
    """``_contrib_quantized_fully_connected`` with int8 CUDA inputs (reference: quantized_fully_connected.cu): the int32
    output equals the integer oracle, the launch counter shows that the tensor-core kernel ran, and the output range is
    the product of the input scales."""
    import mxnet_b200 as mx
    from mxnet_b200 import nd
    from mxnet_b200.ops import cuda as kc
    rng = np.random.RandomState(3)
    x = rng.randint(-127, 128, (48, 256)).astype('int8')
    w = rng.randint(-127, 128, (72, 256)).astype('int8')
    bias = rng.randint(-127, 128, (72,)).astype('int8')
    ctx = mx.gpu(0)
    args = [nd.array(x, ctx=ctx, dtype='int8'), nd.array(w, ctx=ctx, dtype='int8'), nd.array(bias, ctx=ctx, dtype='int8')]
    ranges = [nd.array([v], ctx=ctx) for v in (-2.0, 2.0, -0.5, 0.5, -1.0, 1.0)]
    before = kc.launches()
    out, lo, hi = nd.contrib.quantized_fully_connected(*args, *ranges, num_hidden=72)
    assert kc.launches() == before + 1
    sd, sw, sb = 2.0 / 127, 0.5 / 127, 1.0 / 127
    qb = np.round(bias.astype('float64') * np.float32(sb) / (np.float32(sd) * np.float32(sw)))
    ref = x.astype('int64') @ w.astype('int64').T + qb.astype('int64')
    assert out.dtype == np.int32
    np.testing.assert_array_equal(out.asnumpy(), ref.astype('int32'))
    np.testing.assert_allclose(hi.asnumpy(), [sd * sw * 2147483647.0], rtol=1e-5)
    np.testing.assert_allclose(lo.asnumpy(), [-sd * sw * 2147483647.0], rtol=1e-5)


def test_quantized_network_runs_its_dense_layers_on_the_int8_kernel():
    """``contrib.quantization.quantize_net`` on a small MLP (reference: python/mxnet/contrib/quantization.py,
    quantize_graph_pass.cc): every FullyConnected becomes quantize -> int8 FullyConnected -> dequantize, the int8 products
    run on the tensor-core kernel (launch counter), and the outputs stay close to the float network's."""
    from mxnet_b200.contrib import quantization
    from mxnet_b200.gluon import nn
    from mxnet_b200.ops import cuda as kc
    from mxnet_b200.ops.cuda import gemm_ops
    ctx = mx.gpu(0)
    mx.random.seed(5)
    net = nn.HybridSequential()
    net.add(nn.Dense(512, activation='relu', in_units=256), nn.Dense(128, activation='relu', in_units=512), nn.Dense(64, in_units=128))
    net.initialize(mx.init.Xavier(), ctx=ctx)
    net.hybridize()
    x = nd.array(np.random.RandomState(1).randn(96, 256).astype('float32'), ctx=ctx)
    ref = net(x).asnumpy()
    qnet = quantization.quantize_net(net, data_shapes=[(96, 256)], ctx=ctx)
    before = kc.launches()
    out = qnet(x).asnumpy()
    assert kc.launches() - before >= 3                      # three int8 GEMM launches (plus whatever else is in-tree)
    assert int(gemm_ops._error_flag(torch.device('cuda', 0)).item()) == 0
    err = np.abs(out - ref).max() / np.abs(ref).max()
    assert err < 0.05, err


@pytest.mark.parametrize('cin,cout,k,stride,pad,hw,bias', [(64, 128, 3, 1, 1, 14, True), (32, 64, 1, 1, 0, 9, False), (16, 48, 3, 2, 1, 17, True),
                                                         (64, 32, 5, 1, 2, 8, True)])
def test_quantized_convolution_runs_on_the_int8_kernel_and_is_exact(cin, cout, k, stride, pad, hw, bias):
    """``_contrib_quantized_conv`` with int8 CUDA inputs: receptive fields gathered into rows, product on the
    tcgen05 int8 GEMM (launch counter), int32 results equal to an integer convolution computed in float64 on the host."""
    from mxnet_b200.ops import cuda as kc
    from mxnet_b200.ops.cuda import gemm_ops
    ctx = mx.gpu(0)
    rng = np.random.RandomState(cin + k)
    x = rng.randint(-127, 128, (3, cin, hw, hw)).astype('int8')
    w = rng.randint(-127, 128, (cout, cin, k, k)).astype('int8')
    b = rng.randint(-127, 128, (cout,)).astype('int8')
    args = [nd.array(x, ctx=ctx, dtype='int8'), nd.array(w, ctx=ctx, dtype='int8')]
    rng_args = [nd.array([-1.0], ctx=ctx), nd.array([1.0], ctx=ctx), nd.array([-0.5], ctx=ctx), nd.array([0.5], ctx=ctx)]
    if bias:
        args.append(nd.array(b, ctx=ctx, dtype='int8'))
        rng_args += [nd.array([-2.0], ctx=ctx), nd.array([2.0], ctx=ctx)]
    before = kc.launches()
    if bias:
        out, mn, mxr = nd.contrib.quantized_conv(args[0], args[1], args[2], *rng_args, kernel=(k, k), stride=(stride, stride),
                                                 pad=(pad, pad), num_filter=cout)
    else:
        out, mn, mxr = nd.contrib.quantized_conv(args[0], args[1], None, *rng_args, kernel=(k, k), stride=(stride, stride),
                                                 pad=(pad, pad), num_filter=cout, no_bias=True)
    assert kc.launches() - before >= 1
    assert int(gemm_ops._error_flag(torch.device('cuda', 0)).item()) == 0
    ref = torch.nn.functional.conv2d(torch.from_numpy(x).double(), torch.from_numpy(w).double(), None, stride, pad)
    if bias:
        sd, sw, sb = 1.0 / 127, 0.5 / 127, 2.0 / 127
        ref = ref + torch.round(torch.from_numpy(b).double() * sb / (np.float32(sd) * np.float32(sw))).reshape(1, -1, 1, 1)
    got = out.asnumpy()
    assert got.dtype == np.int32 and got.shape == tuple(ref.shape)
    diff = np.abs(got.astype(np.int64) - ref.numpy().astype(np.int64))
    assert diff.max() <= (1 if bias else 0)             # the bias is rounded from fp32 scale arithmetic: one unit at most
    np.testing.assert_allclose(mxr.asnumpy(), [1.0 / 127 * 0.5 / 127 * 2147483647.0], rtol=1e-5)


def test_quantized_convolutional_network_runs_on_the_int8_kernel():
    """``quantize_net`` on a small CNN: the convolutions whose gathered rows are a multiple of 16 long and the dense layer run
    their int8 products on the tensor-core kernel; outputs stay close to the float network's."""
    from mxnet_b200.contrib import quantization
    from mxnet_b200.gluon import nn
    from mxnet_b200.ops import cuda as kc
    ctx = mx.gpu(0)
    mx.random.seed(7)
    net = nn.HybridSequential()
    net.add(nn.Conv2D(32, 3, padding=1, in_channels=16, activation='relu'), nn.Conv2D(64, 3, strides=2, padding=1, in_channels=32,
                                                                                    activation='relu'),
            nn.Conv2D(32, 1, in_channels=64), nn.GlobalAvgPool2D(), nn.Flatten(), nn.Dense(16, in_units=32))
    net.initialize(mx.init.Xavier(), ctx=ctx)
    net.hybridize()
    x = nd.array(np.random.RandomState(2).randn(8, 16, 12, 12).astype('float32'), ctx=ctx)
    ref = net(x).asnumpy()
    qnet = quantization.quantize_net(net, data_shapes=[(8, 16, 12, 12)], ctx=ctx)
    before = kc.launches()
    out = qnet(x).asnumpy()
    assert kc.launches() - before >= 4                      # three convolutions and the dense layer
    err = np.abs(out - ref).max() / np.abs(ref).max()
    assert err < 0.08, err


# ---------------------------------------------------------------------------------------- layout management
def test_layout_pass_puts_an_nchw_network_on_the_channel_last_kernels():
    """A model written in NCHW (the reference's default layout) runs its convolutions on the tcgen05 NHWC kernels once
    layout management is on (src/common/alm.cc in the reference): same results, in-tree convolution launches."""
    import mxnet_b200 as mx
    from mxnet_b200 import env
    from mxnet_b200.ops import cuda
    from mxnet_b200.symbol import layout
    from mxnet_b200.gluon.model_zoo import vision
    ctx = mx.gpu(0)
    net = vision.resnet18_v1(classes=10)
    net.initialize(mx.init.Xavier(), ctx=ctx)
    net.cast('float16')
    x = mx.nd.array(np.random.RandomState(6).uniform(-1, 1, (8, 3, 64, 64)).astype('float16'), ctx=ctx, dtype='float16')
    net.hybridize()
    net(x)
    expect = net(x).asnumpy().astype('float32')
    layout.set_optimize_layout(True)
    try:
        with env.scope('MXNET_B200_CONV', '1'):                   # take the in-tree kernels wherever they support the shape
            before = cuda.launches()
            got = net(x)
            assert '_layout_transpose' in net._partitioned.tojson()
            assert cuda.launches() - before >= 15                 # 20 convolutions; the 7x7 stem may stay with the library
            np.testing.assert_allclose(got.asnumpy().astype('float32'), expect, rtol=5e-2, atol=5e-2)
            with mx.autograd.record():
                loss = net(x).astype('float32').sum()
            loss.backward()
            g = net.features[0].weight.grad().asnumpy().astype('float32')
            assert np.isfinite(g).all() and np.abs(g).sum() > 0
            # with static allocation the re-laid graph is what the CUDA graphs capture
            net.hybridize(static_alloc=True, static_shape=True)
            for _ in range(3):
                again = net(x)
            tags = [sig[-1] for sig in net._cached_op._graphs]
            assert 'optimize_layout' in tags
        # the training pass above moved the running statistics: compare with the block's own code on the same parameters
        layout.set_optimize_layout(False)
        net.hybridize(False)
        np.testing.assert_allclose(again.asnumpy().astype('float32'), net(x).asnumpy().astype('float32'), rtol=5e-2, atol=5e-2)
    finally:
        layout.set_optimize_layout(False)


def test_plain_hybridize_is_captured_once_a_signature_repeats():
    """hybridize() without static_alloc / static_shape: eager for the first three calls of a signature, CUDA-graph replay
    from then on, at most four signatures per block; MXNET_CUDA_GRAPHS_AUTO=0 keeps such blocks eager."""
    import mxnet_b200 as mx
    from mxnet_b200 import env
    from mxnet_b200.gluon import nn
    ctx = mx.gpu(0)
    net = nn.HybridSequential()
    net.add(nn.Dense(32, activation='relu'), nn.Dense(8))
    net.initialize(ctx=ctx)
    net.hybridize()
    x = mx.nd.array(np.random.RandomState(0).uniform(-1, 1, (4, 16)).astype('float32'), ctx=ctx)
    outs = []
    for i in range(6):
        outs.append(net(x).asnumpy())
        assert len(net._cached_op._graphs) == (1 if i >= 4 else 0), i      # call 0 builds the op; calls 1-3 warm the signature
    for o in outs[1:]:
        np.testing.assert_allclose(o, outs[0], rtol=1e-6, atol=1e-6)
    # training through the captured pair gives the gradients of the eager pass
    x.attach_grad()
    grads = []
    for i in range(6):
        with mx.autograd.record():
            loss = (net(x) ** 2).sum()
        loss.backward()
        grads.append(x.grad.asnumpy().copy())
    for g in grads[1:]:
        np.testing.assert_allclose(g, grads[0], rtol=1e-5, atol=1e-6)
    assert len(net._cached_op._graphs) == 2
    for n in range(5, 12):                                               # changing shapes: no more than four signatures are kept
        y = mx.nd.ones((n, 16), ctx=ctx)
        for _ in range(5):
            net(y)
    assert len(net._cached_op._graphs) == 4
    with env.scope('MXNET_CUDA_GRAPHS_AUTO', '0'):
        net2 = nn.HybridSequential()
        net2.add(nn.Dense(8))
        net2.initialize(ctx=ctx)
        net2.hybridize()
        for _ in range(6):
            net2(x)
        assert len(net2._cached_op._graphs) == 0

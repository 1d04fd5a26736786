"""BatchNorm (NHWC, fused ReLU/residual) and LayerNorm on the sm_100a kernels (``norm.cu``)."""
import torch

from . import lib, ptr, stream_ptr, count_launch, check
from ._util import DT, dt, f32, require


hint_hits = 0        # BatchNorm calls whose batch statistics came from the producing convolution's epilogue


def bn_supported(x):
    c = x.shape[-1]
    l = c // 8
    return c % 8 == 0 and 1 <= l <= 256 and (l & (l - 1)) == 0 and x.numel() > 0


class _BatchNormNHWC(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, rmean, rvar, residual, eps, momentum, training, relu, partials=None):
        L = lib()
        C = x.shape[-1]
        M = x.numel() // C
        require(x, 'data')
        if gamma.dtype != beta.dtype or gamma.dtype not in DT:
            gamma, beta = gamma.float(), beta.float()
        gamma, beta = gamma.contiguous(), beta.contiguous()
        for t, name in ((gamma, 'gamma'), (beta, 'beta')):
            require(t, name, numel=C, device=x.device)
        for t, name in ((rmean, 'moving_mean'), (rvar, 'moving_var')):
            require(t, name, numel=C, dtype=torch.float32, device=x.device)
        res = residual.contiguous() if residual is not None else None
        if res is not None:
            require(res, 'residual', dtype=x.dtype, device=x.device, shape=x.shape)
        stats = torch.empty(4 * C, dtype=torch.float32, device=x.device)    # mean | invstd | scale | shift
        save_mean, save_invstd, scale_shift = stats[:C], stats[C:2 * C], stats[2 * C:]
        y = torch.empty_like(x)
        if training and partials is not None:
            # the producer of x (a convolution epilogue) already accumulated sum x and sum x^2 per channel
            require(partials, 'partials', dtype=torch.float32, device=x.device)
            if partials.dim() != 3 or partials.shape[1] != 2 or partials.shape[2] != C:
                raise ValueError('partials must be [rows, 2, %d], got %s' % (C, tuple(partials.shape)))
            check(L.mxb_bn_forward_stats(dt(x), ptr(x), ptr(res), ptr(gamma), ptr(beta), dt(gamma), ptr(rmean), ptr(rvar),
                                         ptr(save_mean), ptr(save_invstd), ptr(scale_shift), ptr(partials),
                                         partials.shape[0], ptr(y), M, C, eps, momentum, 1 if relu else 0,
                                         stream_ptr(x.device)), 'bn_forward_stats')
            count_launch(2)
        else:
            grid = L.mxb_bn_grid(M, C)
            scratch = torch.empty(grid * 2 * C, dtype=torch.float32, device=x.device)
            check(L.mxb_bn_forward(dt(x), ptr(x), ptr(res), ptr(gamma), ptr(beta), dt(gamma), ptr(rmean), ptr(rvar),
                                   ptr(save_mean), ptr(save_invstd), ptr(scale_shift), ptr(scratch), ptr(y), M, C, eps,
                                   momentum, 1 if training else 0, 1 if relu else 0, stream_ptr(x.device)), 'bn_forward')
            count_launch(3 if training else 2)
        ctx.save_for_backward(x, y if (relu and residual is not None) or not training else None, gamma, stats)
        ctx.relu, ctx.has_res, ctx.training = relu, residual is not None, training
        ctx.set_materialize_grads(False)
        ctx.mark_non_differentiable(save_mean, save_invstd)
        return y, save_mean, save_invstd

    @staticmethod
    def backward(ctx, dy, _gm, _gv):
        x, y, gamma, stats = ctx.saved_tensors
        if dy is None:
            return (None,) * 11
        L = lib()
        C = x.shape[-1]
        M = x.numel() // C
        save_mean, save_invstd, scale_shift = stats[:C], stats[C:2 * C], stats[2 * C:]
        dy = require(dy.contiguous(), 'out_grad', dtype=x.dtype, device=x.device, shape=x.shape)
        if not ctx.training:
            # inference statistics are constants: dx = dy' * gamma * invstd
            d = dy
            if ctx.relu:
                d = d * (y > 0).to(d.dtype)
            scale = (gamma.float() * save_invstd).to(d.dtype)
            dx = d * scale
            xh = (x.float() - save_mean) * save_invstd
            dgamma = (d.float() * xh).reshape(-1, C).sum(0)
            dbeta = d.float().reshape(-1, C).sum(0)
            return dx, dgamma.to(gamma.dtype), dbeta.to(gamma.dtype), None, None, (d if ctx.has_res else None), None, None, None, None, None
        grid = L.mxb_bn_grid(M, C)
        scratch = torch.empty((grid * 2 + 3) * C, dtype=torch.float32, device=x.device)
        dx = torch.empty_like(x)
        dres = torch.empty_like(x) if ctx.has_res else None
        dgb = torch.empty(2 * C, dtype=gamma.dtype, device=x.device)
        dgamma, dbeta = dgb[:C], dgb[C:]
        check(L.mxb_bn_backward(dt(x), ptr(x), ptr(dy), ptr(y), ptr(gamma), dt(gamma), ptr(save_mean), ptr(save_invstd),
                                ptr(scale_shift), ptr(scratch), ptr(dx), ptr(dres), ptr(dgamma), ptr(dbeta), M, C,
                                1 if ctx.relu else 0, stream_ptr(x.device)), 'bn_backward')
        count_launch(3)
        return dx, dgamma, dbeta, None, None, dres, None, None, None, None, None


def batch_norm_nhwc(x, gamma, beta, rmean, rvar, eps, momentum, training, act_type, residual, want_stats=True):
    """Returns (y, mean, var) like the BatchNorm operator with ``output_mean_var``; ``want_stats=False``
    skips the conversion of the saved inverse standard deviation back to a variance."""
    hint = getattr(x, '_mxb_bn_partials', None)
    partials = hint[0] if (training and hint is not None and hint[1] == x._version) else None
    if partials is not None:
        global hint_hits
        hint_hits += 1
    y, mean, invstd = _BatchNormNHWC.apply(x, gamma, beta, rmean, rvar, residual, float(eps), float(momentum),
                                           bool(training), act_type == 'relu', partials)
    if not want_stats:
        return y, None, None
    var = 1.0 / (invstd * invstd) - eps
    return y, mean, var


def ln_supported(x):
    return x.shape[-1] <= 2048 and x.numel() > 0


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps):
        L = lib()
        C = x.shape[-1]
        rows = x.numel() // C
        y = torch.empty_like(x)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        g32, b32 = f32(gamma), f32(beta)
        require(x, 'data')
        require(g32, 'gamma', numel=C, device=x.device)
        require(b32, 'beta', numel=C, device=x.device)
        check(L.mxb_ln_forward(dt(x), ptr(x), ptr(g32), ptr(b32), ptr(y), ptr(mean), ptr(rstd), rows, C, eps,
                               stream_ptr(x.device)), 'ln_forward')
        count_launch(1)
        ctx.save_for_backward(x, g32, mean, rstd)
        ctx.gdtype, ctx.bdtype = gamma.dtype, beta.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        x, g32, mean, rstd = ctx.saved_tensors
        L = lib()
        C = x.shape[-1]
        rows = x.numel() // C
        dy = require(dy.contiguous(), 'out_grad', dtype=x.dtype, device=x.device, shape=x.shape)
        dx = torch.empty_like(x)
        dgamma = torch.empty(C, dtype=torch.float32, device=x.device)
        dbeta = torch.empty(C, dtype=torch.float32, device=x.device)
        scratch = torch.empty(L.mxb_ln_grid(rows) * 2 * C, dtype=torch.float32, device=x.device)
        check(L.mxb_ln_backward(dt(x), ptr(x), ptr(dy), ptr(g32), ptr(mean), ptr(rstd), ptr(dx), ptr(dgamma), ptr(dbeta),
                                ptr(scratch), rows, C, stream_ptr(x.device)), 'ln_backward')
        count_launch(2)
        return dx, dgamma.to(ctx.gdtype), dbeta.to(ctx.bdtype), None


def layer_norm(x, gamma, beta, eps):
    return _LayerNorm.apply(x, gamma, beta, float(eps))

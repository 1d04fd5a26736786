"""Optimizer update operators (single- and multi-tensor), AMP finite checks, multi_sum_sq / LARS.

Reference: ``src/operator/optimizer_op-inl.h`` (SGD ``:219-250,600,718``, NAG ``:1107-1131``, Adam
``:1361``, LAMB phases ``:1736-1870``, FTML/FTRL/RMSProp/Signum), ``src/operator/contrib/
{adamw,adabelief,multi_lamb,multi_lans,multi_lars,multi_sum_sq,preloaded_multi_sgd,reset_arrays}*``
and ``src/operator/all_finite*``.  Common preprocessing:
``g' = clip(rescale_grad * g, clip_gradient)`` (clip only when ``clip_gradient >= 0``).

State tensors (momentum, mean/var, fp32 master weights) are updated in place; the new weight is
returned (and written to ``out=`` by the caller, normally the weight itself).  On CUDA the
multi-tensor forms run as a single multi-tensor-apply kernel launch (``ops/cuda/optim.cu``) whose
tensor table travels as a kernel argument, so no per-call host-to-device table copy is needed.
"""
from __future__ import annotations

import math

import torch

from .registry import register, alias
from .. import env


def _prep(grad, rescale_grad, clip_gradient, dtype=None):
    g = grad.to(dtype) if dtype is not None and grad.dtype != dtype else grad
    if rescale_grad != 1.0:
        g = g * rescale_grad
    if clip_gradient is not None and clip_gradient >= 0:
        g = g.clamp(-clip_gradient, clip_gradient)
    return g


_COMMON = {'lr': 0.01, 'wd': 0.0, 'rescale_grad': 1.0, 'clip_gradient': -1.0}


@register('sgd_update', inputs=('weight', 'grad'), defaults=dict(_COMMON, lazy_update=True))
def sgd_update(weight, grad, lr=0.01, wd=0.0, rescale_grad=1.0, clip_gradient=-1.0, lazy_update=True):
    g = _prep(grad, rescale_grad, clip_gradient)
    return weight.mul_(1 - lr * wd).add_(g, alpha=-lr)


@register('sgd_mom_update', inputs=('weight', 'grad', 'mom'), mutate=('mom',),
          defaults=dict(_COMMON, momentum=0.0, lazy_update=True))
def sgd_mom_update(weight, grad, mom, lr=0.01, momentum=0.0, wd=0.0, rescale_grad=1.0, clip_gradient=-1.0,
                   lazy_update=True):
    g = _prep(grad, rescale_grad, clip_gradient)
    mom.mul_(momentum).add_(g + wd * weight, alpha=-lr)
    return weight.add_(mom)


@register('mp_sgd_update', inputs=('weight', 'grad', 'weight32'), mutate=('weight32',),
          defaults=dict(_COMMON, lazy_update=True))
def mp_sgd_update(weight, grad, weight32, lr=0.01, wd=0.0, rescale_grad=1.0, clip_gradient=-1.0, lazy_update=True):
    g = _prep(grad, rescale_grad, clip_gradient, torch.float32)
    weight32.mul_(1 - lr * wd).add_(g, alpha=-lr)
    return weight.copy_(weight32)


@register('mp_sgd_mom_update', inputs=('weight', 'grad', 'mom', 'weight32'), mutate=('mom', 'weight32'),
          defaults=dict(_COMMON, momentum=0.0, lazy_update=True))
def mp_sgd_mom_update(weight, grad, mom, weight32, lr=0.01, momentum=0.0, wd=0.0, rescale_grad=1.0,
                      clip_gradient=-1.0, lazy_update=True):
    g = _prep(grad, rescale_grad, clip_gradient, torch.float32)
    mom.mul_(momentum).add_(g + wd * weight32, alpha=-lr)
    weight32.add_(mom)
    return weight.copy_(weight32)


@register('nag_mom_update', inputs=('weight', 'grad', 'mom'), mutate=('mom',), defaults=dict(_COMMON, momentum=0.0))
def nag_mom_update(weight, grad, mom, lr=0.01, momentum=0.0, wd=0.0, rescale_grad=1.0, clip_gradient=-1.0):
    g = _prep(grad, rescale_grad, clip_gradient) + wd * weight
    mom.mul_(momentum).add_(g, alpha=-lr)
    return weight.add_(mom, alpha=momentum).add_(g, alpha=-lr)


@register('mp_nag_mom_update', inputs=('weight', 'grad', 'mom', 'weight32'), mutate=('mom', 'weight32'),
          defaults=dict(_COMMON, momentum=0.0))
def mp_nag_mom_update(weight, grad, mom, weight32, lr=0.01, momentum=0.0, wd=0.0, rescale_grad=1.0, clip_gradient=-1.0):
    g = _prep(grad, rescale_grad, clip_gradient, torch.float32) + wd * weight32
    mom.mul_(momentum).add_(g, alpha=-lr)
    weight32.add_(mom, alpha=momentum).add_(g, alpha=-lr)
    return weight.copy_(weight32)


def _seq(v, n):
    if isinstance(v, (tuple, list)):
        return list(v)
    return [v] * n


def _multi(kind, stride):
    """multi_* forms: inputs interleaved per tensor (weight, grad[, mom][, weight32]) (``:201-250``)."""
    def op(*data, lrs=(), wds=(), momentum=0.0, rescale_grad=1.0, clip_gradient=-1.0, num_weights=1):
        n = num_weights
        lrs, wds = _seq(lrs, n), _seq(wds, n)
        ws = [data[i * stride] for i in range(n)]
        gs = [data[i * stride + 1] for i in range(n)]
        if data[0].is_cuda and env.get('MXNET_B200_KERNELS'):
            from . import cuda
            if cuda.available():
                from .cuda import optim_ops
                moms = [data[i * stride + 2] for i in range(n)] if 'mom' in kind else None
                w32 = [data[i * stride + stride - 1] for i in range(n)] if kind.startswith('mp') else None
                optim_ops.multi_sgd(ws, gs, moms, w32, lrs, wds, momentum, rescale_grad, clip_gradient)
                return tuple(ws)
        outs = []
        for i in range(n):
            args = data[i * stride:(i + 1) * stride]
            if kind == 'sgd':
                outs.append(sgd_update(*args, lr=lrs[i], wd=wds[i], rescale_grad=rescale_grad, clip_gradient=clip_gradient))
            elif kind == 'sgd_mom':
                outs.append(sgd_mom_update(*args, lr=lrs[i], momentum=momentum, wd=wds[i], rescale_grad=rescale_grad,
                                           clip_gradient=clip_gradient))
            elif kind == 'mp_sgd':
                outs.append(mp_sgd_update(*args, lr=lrs[i], wd=wds[i], rescale_grad=rescale_grad, clip_gradient=clip_gradient))
            else:
                outs.append(mp_sgd_mom_update(*args, lr=lrs[i], momentum=momentum, wd=wds[i], rescale_grad=rescale_grad,
                                              clip_gradient=clip_gradient))
        return tuple(outs)
    return op


for _k, _s in (('sgd', 2), ('sgd_mom', 3), ('mp_sgd', 3), ('mp_sgd_mom', 4)):
    register('multi_%s_update' % _k, inputs=('*data',), nout=lambda a: a.get('num_weights', 1),
             defaults={'lrs': (), 'wds': (), 'momentum': 0.0, 'rescale_grad': 1.0, 'clip_gradient': -1.0,
                       'num_weights': 1})(_multi(_k, _s))


def _preloaded(kind, stride):
    """preloaded_multi_*: learning rates and weight decays arrive as two trailing tensors."""
    inner = _multi(kind, stride)

    def op(*data, momentum=0.0, rescale_grad=1.0, clip_gradient=-1.0, num_weights=1):
        lrs = data[-2].tolist()
        wds = data[-1].tolist()
        return inner(*data[:-2], lrs=lrs, wds=wds, momentum=momentum, rescale_grad=rescale_grad,
                     clip_gradient=clip_gradient, num_weights=num_weights)
    return op


for _k, _s in (('sgd', 2), ('sgd_mom', 3), ('mp_sgd', 3), ('mp_sgd_mom', 4)):
    register('preloaded_multi_%s_update' % _k, inputs=('*data',), nout=lambda a: a.get('num_weights', 1),
             defaults={'momentum': 0.0, 'rescale_grad': 1.0, 'clip_gradient': -1.0, 'num_weights': 1})(_preloaded(_k, _s))


@register('adam_update', inputs=('weight', 'grad', 'mean', 'var'), mutate=('mean', 'var'),
          defaults=dict(_COMMON, beta1=0.9, beta2=0.999, epsilon=1e-8, lazy_update=True))
def adam_update(weight, grad, mean, var, lr=0.01, beta1=0.9, beta2=0.999, epsilon=1e-8, wd=0.0, rescale_grad=1.0,
                clip_gradient=-1.0, lazy_update=True):
    if _adam_kernel_ok(weight, grad, mean, var):
        from .cuda import optim_ops
        optim_ops.multi_adam([weight], [grad], [mean], [var], None, [lr], [wd], None, beta1, beta2, epsilon,
                             clip_gradient, float(rescale_grad), False)
        return weight
    g = _prep(grad, rescale_grad, clip_gradient) + wd * weight
    mean.mul_(beta1).add_(g, alpha=1 - beta1)
    var.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    return weight.addcdiv_(mean, var.sqrt().add_(epsilon), value=-lr)


def _adam_kernel_ok(weight, grad, mean, var, weight32=None):
    """The multi-tensor Adam kernel takes contiguous CUDA tensors with fp32 states."""
    if not (weight.is_cuda and env.get('MXNET_B200_KERNELS')):
        return False
    from . import cuda
    if not cuda.available():
        return False
    ts = [weight, grad, mean, var] + ([weight32] if weight32 is not None else [])
    return (all(t.is_contiguous() and t.device == weight.device for t in ts) and grad.dtype == weight.dtype
            and weight.dtype in (torch.float32, torch.float16, torch.bfloat16) and mean.dtype == torch.float32
            and var.dtype == torch.float32 and (weight32 is None or weight32.dtype == torch.float32))


def _rescale_arg(rescale_grad, device):
    """rescale_grad for the kernel: the device tensor itself (no host read) or a float."""
    if isinstance(rescale_grad, torch.Tensor):
        if rescale_grad.is_cuda and rescale_grad.device == device and rescale_grad.numel() == 1:
            return rescale_grad.reshape(1).float() if rescale_grad.dtype != torch.float32 else rescale_grad.reshape(1)
        return float(rescale_grad.item())
    return float(rescale_grad)


def _adamw_core(w, g, mean, var, lr, eta, beta1, beta2, epsilon, wd):
    mean.mul_(beta1).add_(g, alpha=1 - beta1)
    var.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    w.sub_(eta * (lr * mean / (var.sqrt() + epsilon) + wd * w))


def _rescale_tensor(rescale_grad):
    return float(rescale_grad.item()) if isinstance(rescale_grad, torch.Tensor) else float(rescale_grad)


@register('_adamw_update', '_contrib_adamw_update', inputs=('weight', 'grad', 'mean', 'var', 'rescale_grad'),
          mutate=('mean', 'var'),
          defaults={'lr': 0.01, 'beta1': 0.9, 'beta2': 0.999, 'epsilon': 1e-8, 'wd': 0.0, 'eta': 1.0, 'clip_gradient': -1.0})
def adamw_update(weight, grad, mean, var, rescale_grad=1.0, lr=0.01, beta1=0.9, beta2=0.999, epsilon=1e-8, wd=0.0,
                 eta=1.0, clip_gradient=-1.0):
    if _adam_kernel_ok(weight, grad, mean, var):
        from .cuda import optim_ops
        optim_ops.multi_adam([weight], [grad], [mean], [var], None, [lr], [wd], [eta], beta1, beta2, epsilon,
                             clip_gradient, _rescale_arg(rescale_grad, weight.device), True)
        return weight
    rs = _rescale_tensor(rescale_grad)
    if not math.isfinite(rs) or rs == 0:
        return weight
    g = _prep(grad, rs, clip_gradient)
    _adamw_core(weight, g, mean, var, lr, eta, beta1, beta2, epsilon, wd)
    return weight


@register('_mp_adamw_update', '_contrib_mp_adamw_update', inputs=('weight', 'grad', 'mean', 'var', 'weight32', 'rescale_grad'),
          mutate=('mean', 'var', 'weight32'),
          defaults={'lr': 0.01, 'beta1': 0.9, 'beta2': 0.999, 'epsilon': 1e-8, 'wd': 0.0, 'eta': 1.0, 'clip_gradient': -1.0})
def mp_adamw_update(weight, grad, mean, var, weight32, rescale_grad=1.0, lr=0.01, beta1=0.9, beta2=0.999,
                    epsilon=1e-8, wd=0.0, eta=1.0, clip_gradient=-1.0):
    if _adam_kernel_ok(weight, grad, mean, var, weight32):
        from .cuda import optim_ops
        optim_ops.multi_adam([weight], [grad], [mean], [var], [weight32], [lr], [wd], [eta], beta1, beta2, epsilon,
                             clip_gradient, _rescale_arg(rescale_grad, weight.device), True)
        return weight
    rs = _rescale_tensor(rescale_grad)
    if not math.isfinite(rs) or rs == 0:
        return weight
    g = _prep(grad, rs, clip_gradient, torch.float32)
    _adamw_core(weight32, g, mean, var, lr, eta, beta1, beta2, epsilon, wd)
    return weight.copy_(weight32)


def _multi_adamw(mp):
    stride = 5 if mp else 4

    def op(*data, lrs=(), wds=(), etas=(), beta1=0.9, beta2=0.999, epsilon=1e-8, clip_gradient=-1.0, num_weights=1):
        n = num_weights
        rs = data[-1]
        lrs, wds, etas = _seq(lrs, n), _seq(wds, n), _seq(etas, n)
        cols = [[data[i * stride + k] for i in range(n)] for k in range(stride)]
        if all(_adam_kernel_ok(*[c[i] for c in cols]) for i in range(n)) and len({c.dtype for c in cols[0]}) == 1:
            # one launch per 48 tensors; the rescale tensor is read on the device
            from .cuda import optim_ops
            optim_ops.multi_adam(cols[0], cols[1], cols[2], cols[3], cols[4] if mp else None, lrs, wds, etas, beta1, beta2,
                                 epsilon, clip_gradient, _rescale_arg(rs, cols[0][0].device), True)
            return tuple(cols[0])
        outs = []
        for i in range(n):
            a = data[i * stride:(i + 1) * stride]
            fn = mp_adamw_update if mp else adamw_update
            outs.append(fn(*a, rescale_grad=rs, lr=lrs[i], beta1=beta1, beta2=beta2, epsilon=epsilon, wd=wds[i],
                           eta=etas[i], clip_gradient=clip_gradient))
        return tuple(outs)
    return op


register('_multi_adamw_update', '_contrib_multi_adamw_update', inputs=('*data',), nout=lambda a: a.get('num_weights', 1),
         defaults={'lrs': (), 'wds': (), 'etas': (), 'beta1': 0.9, 'beta2': 0.999, 'epsilon': 1e-8,
                   'clip_gradient': -1.0, 'num_weights': 1})(_multi_adamw(False))
register('_multi_mp_adamw_update', '_contrib_multi_mp_adamw_update', inputs=('*data',), nout=lambda a: a.get('num_weights', 1),
         defaults={'lrs': (), 'wds': (), 'etas': (), 'beta1': 0.9, 'beta2': 0.999, 'epsilon': 1e-8,
                   'clip_gradient': -1.0, 'num_weights': 1})(_multi_adamw(True))


@register('_adabelief_update', '_contrib_adabelief_update', inputs=('weight', 'grad', 'mean', 'var', 'rescale_grad'),
          mutate=('mean', 'var'),
          defaults={'lr': 0.01, 'beta1': 0.9, 'beta2': 0.999, 'epsilon': 1e-8, 'wd': 0.0, 'eta': 1.0, 'clip_gradient': -1.0})
def adabelief_update(weight, grad, mean, var, rescale_grad=1.0, lr=0.01, beta1=0.9, beta2=0.999, epsilon=1e-8, wd=0.0,
                     eta=1.0, clip_gradient=-1.0):
    # tensor operations on every device: the second moment follows (g - mean)^2, which the multi-tensor Adam kernel does
    # not compute
    rs = _rescale_tensor(rescale_grad)
    if not math.isfinite(rs) or rs == 0:
        return weight
    g = _prep(grad, rs, clip_gradient) + wd * weight
    mean.mul_(beta1).add_(g, alpha=1 - beta1)
    diff = g - mean
    var.mul_(beta2).addcmul_(diff, diff, value=1 - beta2).add_(epsilon)
    return weight.sub_(eta * lr * mean / (var.sqrt() + epsilon))


@register('_mp_adabelief_update', '_contrib_mp_adabelief_update',
          inputs=('weight', 'grad', 'mean', 'var', 'weight32', 'rescale_grad'), mutate=('mean', 'var', 'weight32'),
          defaults={'lr': 0.01, 'beta1': 0.9, 'beta2': 0.999, 'epsilon': 1e-8, 'wd': 0.0, 'eta': 1.0, 'clip_gradient': -1.0})
def mp_adabelief_update(weight, grad, mean, var, weight32, rescale_grad=1.0, **kw):
    adabelief_update(weight32, grad.float(), mean, var, rescale_grad, **kw)
    return weight.copy_(weight32)


# ---- LAMB (optimizer_op-inl.h:1736-1870) -------------------------------------------------
@register('lamb_update_phase1', inputs=('weight', 'grad', 'mean', 'var'), mutate=('mean', 'var'),
          defaults={'beta1': 0.9, 'beta2': 0.999, 'epsilon': 1e-6, 't': 1, 'bias_correction': True, 'wd': 0.0,
                    'rescale_grad': 1.0, 'clip_gradient': -1.0})
def lamb_update_phase1(weight, grad, mean, var, beta1=0.9, beta2=0.999, epsilon=1e-6, t=1, bias_correction=True,
                       wd=0.0, rescale_grad=1.0, clip_gradient=-1.0):
    g = _prep(grad, rescale_grad, clip_gradient, mean.dtype)
    mean.mul_(beta1).add_(g, alpha=1 - beta1)
    var.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    if bias_correction:
        mh = mean / (1 - beta1 ** t)
        vh = var / (1 - beta2 ** t)
    else:
        mh, vh = mean, var
    return mh / (vh.sqrt() + epsilon) + wd * weight.to(mean.dtype)


@register('lamb_update_phase2', inputs=('weight', 'g', 'r1', 'r2'),
          defaults={'lr': 0.01, 'lower_bound': -1.0, 'upper_bound': -1.0})
def lamb_update_phase2(weight, g, r1, r2, lr=0.01, lower_bound=-1.0, upper_bound=-1.0):
    r1v = r1.reshape(()).float()
    if lower_bound is not None and lower_bound >= 0:
        r1v = r1v.clamp(min=lower_bound)
    if upper_bound is not None and upper_bound >= 0:
        r1v = r1v.clamp(max=upper_bound)
    r2v = r2.reshape(()).float()
    ratio = torch.where((r1v == 0) | (r2v == 0), torch.ones_like(r1v), r1v / r2v)
    return weight.sub_((lr * ratio * g).to(weight.dtype))


@register('mp_lamb_update_phase1', inputs=('weight', 'grad', 'mean', 'var', 'weight32'), mutate=('mean', 'var'),
          defaults={'beta1': 0.9, 'beta2': 0.999, 'epsilon': 1e-6, 't': 1, 'bias_correction': True, 'wd': 0.0,
                    'rescale_grad': 1.0, 'clip_gradient': -1.0})
def mp_lamb_update_phase1(weight, grad, mean, var, weight32, **kw):
    return lamb_update_phase1(weight32, grad, mean, var, **kw)


@register('mp_lamb_update_phase2', inputs=('weight', 'g', 'r1', 'r2', 'weight32'), mutate=('weight32',),
          defaults={'lr': 0.01, 'lower_bound': -1.0, 'upper_bound': -1.0})
def mp_lamb_update_phase2(weight, g, r1, r2, weight32, lr=0.01, lower_bound=-1.0, upper_bound=-1.0):
    lamb_update_phase2(weight32, g, r1, r2, lr, lower_bound, upper_bound)
    return weight.copy_(weight32)


def _multi_lamb(mp, lans=False):
    stride = 5 if mp else 4

    def op(*data, learning_rates=(), wds=(), beta1=0.9, beta2=0.999, epsilon=1e-6, rescale_grad=1.0,
           lower_bound=-1.0, upper_bound=-1.0, clip_gradient=-1.0, bias_correction=True, step_count=(),
           num_tensors=1):
        n = num_tensors
        lrs, wds_, steps = _seq(learning_rates, n), _seq(wds, n), _seq(step_count, n)
        outs = []
        for i in range(n):
            a = data[i * stride:(i + 1) * stride]
            w, g, mean, var = a[0], a[1], a[2], a[3]
            master = a[4] if mp else w
            if lans:
                _lans_step(master, g, mean, var, lrs[i], wds_[i], beta1, beta2, epsilon, steps[i], rescale_grad,
                           lower_bound, upper_bound, clip_gradient)
            else:
                u = lamb_update_phase1(master, g, mean, var, beta1, beta2, epsilon, steps[i], bias_correction,
                                       wds_[i], rescale_grad, clip_gradient)
                r1 = master.float().norm()
                r2 = u.float().norm()
                lamb_update_phase2(master, u, r1, r2, lrs[i], lower_bound, upper_bound)
            if mp:
                w.copy_(master)
            outs.append(w)
        return tuple(outs)
    return op


def _lans_step(w, grad, mean, var, lr, wd, beta1, beta2, eps, t, rescale_grad, lower, upper, clip):
    """LANS (``src/operator/contrib/multi_lans.cu``): gradient normalised per tensor, two trust ratios."""
    g = _prep(grad, rescale_grad, clip, torch.float32)
    gn = g.norm()
    g = torch.where(gn > 0, g / gn, g)
    mean.mul_(beta1).add_(g, alpha=1 - beta1)
    var.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    mh = mean / (1 - beta1 ** t)
    vh = var / (1 - beta2 ** t)
    denom = vh.sqrt() + eps
    wf = w.float()
    um = mh / denom + wd * wf
    ug = g / denom + wd * wf
    r1 = wf.norm()
    if lower is not None and lower >= 0:
        r1 = r1.clamp(min=lower)
    if upper is not None and upper >= 0:
        r1 = r1.clamp(max=upper)
    rm, rg = um.norm(), ug.norm()
    ratio_m = torch.where((r1 == 0) | (rm == 0), torch.ones_like(r1), r1 / rm)
    ratio_g = torch.where((r1 == 0) | (rg == 0), torch.ones_like(r1), r1 / rg)
    w.sub_((lr * (beta1 * ratio_m * um + (1 - beta1) * ratio_g * ug)).to(w.dtype))


_LAMB_DEFAULTS = {'learning_rates': (), 'wds': (), 'beta1': 0.9, 'beta2': 0.999, 'epsilon': 1e-6, 'rescale_grad': 1.0,
                  'lower_bound': -1.0, 'upper_bound': -1.0, 'clip_gradient': -1.0, 'bias_correction': True,
                  'step_count': (), 'num_tensors': 1}
register('_multi_lamb_update', inputs=('*data',), nout=lambda a: a.get('num_tensors', 1), defaults=_LAMB_DEFAULTS)(_multi_lamb(False))
register('_multi_mp_lamb_update', inputs=('*data',), nout=lambda a: a.get('num_tensors', 1), defaults=_LAMB_DEFAULTS)(_multi_lamb(True))
register('_multi_lans_update', inputs=('*data',), nout=lambda a: a.get('num_tensors', 1), defaults=_LAMB_DEFAULTS)(_multi_lamb(False, True))
register('_multi_mp_lans_update', inputs=('*data',), nout=lambda a: a.get('num_tensors', 1), defaults=_LAMB_DEFAULTS)(_multi_lamb(True, True))


# ---- other single-tensor rules -------------------------------------------------------------
@register('ftml_update', inputs=('weight', 'grad', 'd', 'v', 'z'), mutate=('d', 'v', 'z'),
          defaults={'lr': 0.01, 'beta1': 0.6, 'beta2': 0.999, 'epsilon': 1e-8, 't': 1, 'wd': 0.0, 'rescale_grad': 1.0,
                    'clip_grad': -1.0})
def ftml_update(weight, grad, d, v, z, lr=0.01, beta1=0.6, beta2=0.999, epsilon=1e-8, t=1, wd=0.0, rescale_grad=1.0,
                clip_grad=-1.0):
    g = _prep(grad, rescale_grad, clip_grad) + wd * weight
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    d_t = (1 - beta1 ** t) / lr * ((v / (1 - beta2 ** t)).sqrt() + epsilon)
    sigma = d_t - beta1 * d
    z.mul_(beta1).add_((1 - beta1) * g - sigma * weight)
    d.copy_(d_t)
    return weight.copy_(-z / d_t)


@register('ftrl_update', inputs=('weight', 'grad', 'z', 'n'), mutate=('z', 'n'),
          defaults={'lr': 0.01, 'lamda1': 0.01, 'beta': 1.0, 'wd': 0.0, 'rescale_grad': 1.0, 'clip_gradient': -1.0})
def ftrl_update(weight, grad, z, n, lr=0.01, lamda1=0.01, beta=1.0, wd=0.0, rescale_grad=1.0, clip_gradient=-1.0):
    g = _prep(grad, rescale_grad, clip_gradient)
    z.add_(g - ((n + g * g).sqrt() - n.sqrt()) * weight / lr)
    n.add_(g * g)
    new_w = (torch.sign(z) * lamda1 - z) / ((beta + n.sqrt()) / lr + wd) * (z.abs() > lamda1).to(weight.dtype)
    return weight.copy_(new_w)


@register('rmsprop_update', inputs=('weight', 'grad', 'n'), mutate=('n',),
          defaults={'lr': 0.01, 'gamma1': 0.95, 'epsilon': 1e-8, 'wd': 0.0, 'rescale_grad': 1.0, 'clip_gradient': -1.0,
                    'clip_weights': -1.0})
def rmsprop_update(weight, grad, n, lr=0.01, gamma1=0.95, epsilon=1e-8, wd=0.0, rescale_grad=1.0, clip_gradient=-1.0,
                   clip_weights=-1.0):
    g = _prep(grad, rescale_grad, clip_gradient) + wd * weight
    n.mul_(gamma1).addcmul_(g, g, value=1 - gamma1)
    weight.sub_(lr * g / (n.sqrt() + epsilon))
    if clip_weights is not None and clip_weights >= 0:
        weight.clamp_(-clip_weights, clip_weights)
    return weight


@register('rmspropalex_update', inputs=('weight', 'grad', 'n', 'g', 'delta'), mutate=('n', 'g', 'delta'),
          defaults={'lr': 0.01, 'gamma1': 0.95, 'gamma2': 0.9, 'epsilon': 1e-8, 'wd': 0.0, 'rescale_grad': 1.0,
                    'clip_gradient': -1.0, 'clip_weights': -1.0})
def rmspropalex_update(weight, grad, n, g, delta, lr=0.01, gamma1=0.95, gamma2=0.9, epsilon=1e-8, wd=0.0,
                       rescale_grad=1.0, clip_gradient=-1.0, clip_weights=-1.0):
    gr = _prep(grad, rescale_grad, clip_gradient) + wd * weight
    n.mul_(gamma1).addcmul_(gr, gr, value=1 - gamma1)
    g.mul_(gamma1).add_(gr, alpha=1 - gamma1)
    delta.mul_(gamma2).sub_(lr * gr / (n - g * g + epsilon).sqrt())
    weight.add_(delta)
    if clip_weights is not None and clip_weights >= 0:
        weight.clamp_(-clip_weights, clip_weights)
    return weight


@register('signsgd_update', inputs=('weight', 'grad'), defaults=dict(_COMMON))
def signsgd_update(weight, grad, lr=0.01, wd=0.0, rescale_grad=1.0, clip_gradient=-1.0):
    return weight.mul_(1 - lr * wd).sub_(lr * torch.sign(grad))


@register('signum_update', inputs=('weight', 'grad', 'mom'), mutate=('mom',),
          defaults=dict(_COMMON, momentum=0.0, wd_lh=0.0))
def signum_update(weight, grad, mom, lr=0.01, momentum=0.0, wd=0.0, rescale_grad=1.0, clip_gradient=-1.0, wd_lh=0.0):
    g = _prep(grad, rescale_grad, clip_gradient) + wd * weight
    mom.mul_(momentum).sub_(g, alpha=1 - momentum)
    return weight.mul_(1 - lr * wd_lh).add_(torch.sign(mom), alpha=lr)


@register('_sparse_adagrad_update', 'adagrad_update', inputs=('weight', 'grad', 'history'), mutate=('history',),
          defaults={'lr': 0.01, 'epsilon': 1e-7, 'wd': 0.0, 'rescale_grad': 1.0, 'clip_gradient': -1.0})
def adagrad_update(weight, grad, history, lr=0.01, epsilon=1e-7, wd=0.0, rescale_grad=1.0, clip_gradient=-1.0):
    g = _prep(grad, rescale_grad, clip_gradient) + wd * weight
    history.addcmul_(g, g)
    return weight.sub_(lr * g / (history.sqrt() + epsilon))


@register('_contrib_group_adagrad_update', inputs=('weight', 'grad', 'history'), mutate=('history',),
          defaults={'lr': 0.01, 'epsilon': 1e-5, 'rescale_grad': 1.0, 'clip_gradient': -1.0})
def group_adagrad_update(weight, grad, history, lr=0.01, epsilon=1e-5, rescale_grad=1.0, clip_gradient=-1.0):
    g = _prep(grad, rescale_grad, clip_gradient)
    history.add_((g * g).mean(1, keepdim=True))
    return weight.sub_(lr * g / (history.sqrt() + epsilon))


# ---- AMP finite checks (src/operator/all_finite.cu) -----------------------------------------
@register('all_finite', inputs=('data',), defaults={'init_output': True})
def all_finite(data, init_output=True):
    return torch.isfinite(data).all().to(torch.float32).reshape(1)


@register('multi_all_finite', inputs=('*data',), defaults={'num_arrays': 1, 'init_output': True})
def multi_all_finite(*data, num_arrays=1, init_output=True):
    if data and data[0].is_cuda and env.get('MXNET_B200_KERNELS'):
        from . import cuda
        if cuda.available():
            from .cuda import optim_ops
            return optim_ops.multi_all_finite(list(data))
    ok = torch.ones(1, dtype=torch.float32, device=data[0].device)
    for d in data:
        ok = ok * torch.isfinite(d).all().to(torch.float32)
    return ok


@register('multi_sum_sq', inputs=('*data',), defaults={'num_arrays': 1})
def multi_sum_sq(*data, num_arrays=1):
    if data and data[0].is_cuda and env.get('MXNET_B200_KERNELS'):
        from . import cuda
        if cuda.available():
            from .cuda import optim_ops
            return optim_ops.multi_sum_sq(list(data))
    return torch.stack([(d.float() * d.float()).sum() for d in data])


@register('multi_lars', inputs=('lrs', 'weights_sum_sq', 'grads_sum_sq', 'wds'),
          defaults={'eta': 0.001, 'eps': 1e-8, 'rescale_grad': 1.0})
def multi_lars(lrs, weights_sum_sq, grads_sum_sq, wds, eta=0.001, eps=1e-8, rescale_grad=1.0):
    w = weights_sum_sq.sqrt()
    g = grads_sum_sq.sqrt() * rescale_grad
    ratio = eta * w / (g + wds * w + eps)
    return torch.where((w > 0) & (g > 0), lrs * ratio, lrs)


@register('reset_arrays', inputs=('*data',), nout=0, defaults={'num_arrays': 1})
def reset_arrays(*data, num_arrays=1):
    for d in data:
        d.zero_()
    return ()

"""Operator names of the reference's registry that have no home in the other operator modules: scalar variants of the
NumPy binary functions, the ``where`` / boolean-mask-assign scalar forms, bounding-box encode / decode, the intgemm
family, multi-tensor AdaBelief, binomial sampling, ``hard_sigmoid``, ``cast_storage`` and a few aliases
(``src/operator/numpy/np_elemwise_broadcast_op_extended*.cc``, ``np_where_op.cc``, ``np_boolean_mask_assign.cc``,
``contrib/bounding_box.cc``, ``contrib/intgemm/*.cc``, ``contrib/adabelief.cc``, ``random/sample_op.cc``,
``tensor/elemwise_unary_op_basic.cc``, ``tensor/cast_storage.cc``)."""
import math

import torch

from ..base import MXNetError, to_torch_dtype
from .registry import register, get, alias, has


def _scalar_tensor(data, scalar):
    dt = data.dtype if data.dtype.is_floating_point or isinstance(scalar, (bool, int)) else torch.float32
    return torch.as_tensor(scalar, dtype=dt, device=data.device)


def _reg_scalar_pair(name, fn):
    """``_npi_<name>_scalar`` (array op scalar) and ``_npi_r<name>_scalar`` (scalar op array)."""
    def fwd(data, scalar=0.0, is_int=None):
        return fn(data, _scalar_tensor(data, scalar))

    def rev(data, scalar=0.0, is_int=None):
        return fn(_scalar_tensor(data, scalar), data)
    if not has('_npi_%s_scalar' % name):
        register('_npi_%s_scalar' % name, inputs=('data',), defaults={'scalar': 0.0})(fwd)
    if not has('_npi_r%s_scalar' % name):
        register('_npi_r%s_scalar' % name, inputs=('data',), defaults={'scalar': 0.0})(rev)


def _ldexp(a, b):
    return a * torch.pow(torch.full_like(b, 2.0, dtype=torch.result_type(a, b) if b.dtype.is_floating_point else a.dtype), b)


for _name, _fn in (('arctan2', torch.atan2), ('copysign', torch.copysign), ('fmax', torch.fmax), ('fmin', torch.fmin),
                   ('fmod', torch.fmod), ('gcd', torch.gcd), ('lcm', torch.lcm), ('ldexp', _ldexp), ('logaddexp', torch.logaddexp),
                   ('bitwise_left_shift', torch.bitwise_left_shift), ('bitwise_right_shift', torch.bitwise_right_shift)):
    _reg_scalar_pair(_name, _fn)

if not has('_npi_bitwise_left_shift'):
    register('_npi_bitwise_left_shift', inputs=('lhs', 'rhs'))(lambda lhs, rhs: torch.bitwise_left_shift(lhs, rhs))
    register('_npi_bitwise_right_shift', inputs=('lhs', 'rhs'))(lambda lhs, rhs: torch.bitwise_right_shift(lhs, rhs))

for _new, _old in (('_sample_categorical', '_sample_multinomial'), ('sample_categorical', '_sample_multinomial'),
                   ('_npi_deg2rad', '_npi_radians'), ('_npi_rad2deg', '_npi_degrees'), ('_npx_relu', 'relu'), ('_npx_sigmoid', 'sigmoid'),
                   ('_npx_nonzero', '_npi_nonzero'), ('_copyto', '_copy')):
    if has(_old) and not has(_new):
        alias(get(_old).name, _new)


@register('_npi_diagflat', inputs=('data',), defaults={'k': 0})
def diagflat(data, k=0):
    return torch.diagflat(data, int(k))


@register('_npi_hsplit', inputs=('data',), nout=lambda a: _nsplit(a), defaults={'indices': (), 'axis': 1, 'squeeze_axis': False, 'sections': 0})
def hsplit(data, indices=(), axis=1, squeeze_axis=False, sections=0):
    ax = 0 if data.dim() == 1 else 1
    return _split(data, indices, sections, ax)


@register('_npi_dsplit', inputs=('data',), nout=lambda a: _nsplit(a), defaults={'indices': (), 'axis': 2, 'squeeze_axis': False, 'sections': 0})
def dsplit(data, indices=(), axis=2, squeeze_axis=False, sections=0):
    return _split(data, indices, sections, 2)


def _nsplit(attrs):
    sections = int(attrs.get('sections', 0) or 0)
    return sections if sections > 0 else len(tuple(attrs.get('indices', ()))) + 1


def _split(data, indices, sections, axis):
    if sections and int(sections) > 0:
        return tuple(torch.tensor_split(data, int(sections), dim=axis))
    return tuple(torch.tensor_split(data, [int(i) for i in indices], dim=axis))


@register('_npi_diag_indices_from', inputs=('data',))
def diag_indices_from(data):
    if data.dim() < 2 or len(set(data.shape)) != 1:
        raise MXNetError('All dimensions of input must be of equal length')
    idx = torch.arange(data.shape[0], device=data.device)
    return torch.stack([idx] * data.dim(), 0)


@register('_npi_share_memory', inputs=('a', 'b'))
def share_memory(a, b):
    same = a.untyped_storage().data_ptr() == b.untyped_storage().data_ptr() and a.numel() > 0 and b.numel() > 0
    return torch.tensor(bool(same), device=a.device)


# ---- where with scalar branches (np_where_op.cc) ---------------------------------------------------------
@register('_npi_where_lscalar', inputs=('condition', 'x'), defaults={'scalar': 0.0})
def where_lscalar(condition, x, scalar=0.0):
    return torch.where(condition.bool(), torch.as_tensor(scalar, dtype=x.dtype, device=x.device), x)


@register('_npi_where_rscalar', inputs=('condition', 'x'), defaults={'scalar': 0.0})
def where_rscalar(condition, x, scalar=0.0):
    return torch.where(condition.bool(), x, torch.as_tensor(scalar, dtype=x.dtype, device=x.device))


@register('_npi_where_scalar2', inputs=('condition',), defaults={'x': 0.0, 'y': 0.0})
def where_scalar2(condition, x=0.0, y=0.0):
    dt = torch.float32 if isinstance(x, float) or isinstance(y, float) else torch.int64
    return torch.where(condition.bool(), torch.as_tensor(x, dtype=dt, device=condition.device),
                       torch.as_tensor(y, dtype=dt, device=condition.device))


# ---- a[mask] = value (np_boolean_mask_assign.cc): returns the updated array ------------------------------------
@register('_npi_boolean_mask_assign_scalar', inputs=('data', 'mask'), defaults={'value': 0.0, 'start_axis': 0})
def boolean_mask_assign_scalar(data, mask, value=0.0, start_axis=0):
    out = data.clone()
    index = (slice(None),) * int(start_axis) + (mask.bool(),)
    out[index] = value
    return out


@register('_npi_boolean_mask_assign_tensor', inputs=('data', 'mask', 'value'), defaults={'start_axis': 0})
def boolean_mask_assign_tensor(data, mask, value, start_axis=0):
    out = data.clone()
    index = (slice(None),) * int(start_axis) + (mask.bool(),)
    out[index] = value.to(out.dtype)
    return out


@register('_npi_advanced_indexing', inputs=('data', 'indices'))
def advanced_indexing(data, indices):
    return data[indices.bool() if indices.dtype == torch.bool else indices.long()]


@register('_npi_advanced_indexing_multiple', inputs=('data', '*indices'))
def advanced_indexing_multiple(data, *indices):
    return data[tuple(i.long() for i in indices)]


# ---- random (sample_op.cc, np_normal_op.cc) ----------------------------------------------------------------------
@register('_npi_normal_n', inputs=('loc', 'scale'), defaults={'size': None, 'ctx': None, 'dtype': 'float32'})
def normal_n(loc=None, scale=None, size=None, ctx=None, dtype='float32', **kw):
    """Samples of shape ``size + broadcast(loc, scale).shape`` (the batch dimensions come first)."""
    loc_t = loc if isinstance(loc, torch.Tensor) else torch.as_tensor(kw.get('loc', 0.0) if loc is None else loc, dtype=torch.float32)
    scale_t = scale if isinstance(scale, torch.Tensor) else torch.as_tensor(kw.get('scale', 1.0) if scale is None else scale,
                                                                          dtype=torch.float32, device=loc_t.device)
    base = torch.broadcast_shapes(loc_t.shape, scale_t.shape)
    shape = tuple(size or ()) + tuple(base) if not isinstance(size, int) else (size,) + tuple(base)
    eps = torch.randn(shape, device=loc_t.device, dtype=torch.float32)
    return (loc_t + scale_t * eps).to(to_torch_dtype(dtype))


@register('_npi_uniform_n', inputs=('low', 'high'), defaults={'size': None, 'ctx': None, 'dtype': 'float32'})
def uniform_n(low=None, high=None, size=None, ctx=None, dtype='float32', **kw):
    low_t = low if isinstance(low, torch.Tensor) else torch.as_tensor(kw.get('low', 0.0) if low is None else low, dtype=torch.float32)
    high_t = high if isinstance(high, torch.Tensor) else torch.as_tensor(kw.get('high', 1.0) if high is None else high,
                                                                       dtype=torch.float32, device=low_t.device)
    base = torch.broadcast_shapes(low_t.shape, high_t.shape)
    shape = tuple(size or ()) + tuple(base) if not isinstance(size, int) else (size,) + tuple(base)
    u = torch.rand(shape, device=low_t.device, dtype=torch.float32)
    return (low_t + (high_t - low_t) * u).to(to_torch_dtype(dtype))


def _binomial(n, p, shape, device, dtype):
    n_t = torch.as_tensor(n, dtype=torch.float32, device=device).expand(shape)
    p_t = torch.as_tensor(p, dtype=torch.float32, device=device).expand(shape)
    return torch.binomial(n_t.contiguous(), p_t.contiguous()).to(dtype)


@register('_random_binomial', 'random_binomial', inputs=(), defaults={'n': 1, 'p': 1.0, 'shape': (), 'ctx': None, 'dtype': 'float32'})
def random_binomial(n=1, p=1.0, shape=(), ctx=None, dtype='float32'):
    from .tensor import _dev
    dev = _dev(ctx)
    shape = (shape,) if isinstance(shape, int) else tuple(shape or (1,))
    return _binomial(n, p, shape, dev, to_torch_dtype(dtype or 'float32'))


@register('_random_binomial_like', inputs=('data',), defaults={'n': 1, 'p': 1.0})
def random_binomial_like(data, n=1, p=1.0):
    return _binomial(n, p, tuple(data.shape), data.device, data.dtype if data.dtype.is_floating_point else torch.float32)


@register('_sample_binomial', 'sample_binomial', inputs=('n', 'p'), defaults={'shape': (), 'dtype': 'float32'})
def sample_binomial(n, p, shape=(), dtype='float32'):
    """One batch of ``shape`` samples per (n, p) pair: output shape = n.shape + shape."""
    shape = (shape,) if isinstance(shape, int) else tuple(shape or ())
    full = tuple(n.shape) + shape
    view = tuple(n.shape) + (1,) * len(shape)
    return torch.binomial(n.float().reshape(view).expand(full).contiguous(),
                          p.float().reshape(view).expand(full).contiguous()).to(to_torch_dtype(dtype or 'float32'))


# ---- small unary / storage operators -------------------------------------------------------------------------------
@register('hard_sigmoid', inputs=('data',), defaults={'alpha': 0.2, 'beta': 0.5})
def hard_sigmoid(data, alpha=0.2, beta=0.5):
    return torch.clamp(alpha * data + beta, 0.0, 1.0)


@register('cast_storage', inputs=('data',), defaults={'stype': 'default'})
def cast_storage(data, stype='default'):
    """Tensors inside the operator library are dense: the storage type is carried by the array wrappers
    (``NDArray.tostype``), so the value itself passes through."""
    if stype not in ('default', 'row_sparse', 'csr'):
        raise MXNetError('unknown storage type %s' % stype)
    return data


@register('_identity_with_attr_like_rhs', inputs=('lhs', 'rhs'))
def identity_with_attr_like_rhs(lhs, rhs):
    return lhs


@register('_sparse_retain', 'sparse_retain', inputs=('data', 'indices'))
def sparse_retain(data, indices):
    """Keep the rows listed in ``indices``, zero the others (dense result of the row-sparse operator)."""
    out = torch.zeros_like(data)
    idx = indices.long()
    out[idx] = data[idx]
    return out


# ---- bounding boxes (bounding_box.cc: box_encode / box_decode) -------------------------------------------------------
@register('_contrib_box_encode', 'box_encode', inputs=('samples', 'matches', 'anchors', 'refs', 'means', 'stds'), nout=2)
def box_encode(samples, matches, anchors, refs, means, stds):
    """Regression targets of matched anchors: samples (B, N) in {+1 positive, other}, matches (B, N) index into refs
    (B, M, 4), anchors (B, N, 4) corner boxes -> targets (B, N, 4), masks (B, N, 4)."""
    ref = torch.gather(refs, 1, matches.long().clamp(min=0).unsqueeze(-1).expand(-1, -1, 4))

    def centre(b):
        w, h = b[..., 2] - b[..., 0], b[..., 3] - b[..., 1]
        return b[..., 0] + 0.5 * w, b[..., 1] + 0.5 * h, w, h
    ax, ay, aw, ah = centre(anchors)
    rx, ry, rw, rh = centre(ref)
    t = torch.stack([(rx - ax) / aw, (ry - ay) / ah, torch.log(rw / aw), torch.log(rh / ah)], -1)
    t = (t - means.reshape(1, 1, 4)) / stds.reshape(1, 1, 4)
    mask = (samples > 0.5).unsqueeze(-1).expand_as(t).to(t.dtype)
    return torch.where(mask > 0, t, torch.zeros_like(t)), mask


@register('_contrib_box_decode', 'box_decode', inputs=('data', 'anchors'),
          defaults={'std0': 1.0, 'std1': 1.0, 'std2': 1.0, 'std3': 1.0, 'clip': -1.0, 'format': 'center'})
def box_decode(data, anchors, std0=1.0, std1=1.0, std2=1.0, std3=1.0, clip=-1.0, format='center'):   # pylint: disable=redefined-builtin
    """Corner boxes from regression outputs (B, N, 4) and anchors (1, N, 4) given as centre or corner boxes."""
    if format == 'corner':
        aw, ah = anchors[..., 2] - anchors[..., 0], anchors[..., 3] - anchors[..., 1]
        ax, ay = anchors[..., 0] + 0.5 * aw, anchors[..., 1] + 0.5 * ah
    else:
        ax, ay, aw, ah = anchors[..., 0], anchors[..., 1], anchors[..., 2], anchors[..., 3]
    ox, oy = data[..., 0] * std0 * aw + ax, data[..., 1] * std1 * ah + ay
    dw, dh = data[..., 2] * std2, data[..., 3] * std3
    if clip > 0:
        dw, dh = dw.clamp(max=clip), dh.clamp(max=clip)
    ow, oh = torch.exp(dw) * aw * 0.5, torch.exp(dh) * ah * 0.5
    return torch.stack([ox - ow, oy - oh, ox + ow, oy + oh], -1)


# ---- intgemm family (contrib/intgemm): int8 products with a float multiplier -----------------------------------------
@register('_contrib_intgemm_maxabsolute', 'intgemm_maxabsolute', inputs=('data',))
def intgemm_maxabsolute(data):
    return data.abs().max().reshape(1)


@register('_contrib_intgemm_prepare_data', 'intgemm_prepare_data', inputs=('data', 'maxabs'))
def intgemm_prepare_data(data, maxabs):
    """float -> int8 with the multiplier 127 / maxabs (round to nearest, saturate)."""
    return torch.clamp(torch.round(data * (127.0 / maxabs.reshape(()))), -127, 127).to(torch.int8)


@register('_contrib_intgemm_prepare_weight', 'intgemm_prepare_weight', inputs=('weight', 'maxabs'), defaults={'already_quantized': False})
def intgemm_prepare_weight(weight, maxabs=None, already_quantized=False):
    """The reference rearranges the weight for its CPU kernels; here the prepared form is the int8 matrix itself."""
    if already_quantized:
        return weight.to(torch.int8)
    return intgemm_prepare_data(weight, maxabs)


@register('_contrib_intgemm_take_weight', 'intgemm_take_weight', inputs=('weight', 'indices'))
def intgemm_take_weight(weight, indices):
    return weight[indices.long()]


@register('_contrib_intgemm_fully_connected', 'intgemm_fully_connected', inputs=('data', 'weight', 'scaling', 'bias'),
          defaults={'num_hidden': 0, 'no_bias': False, 'flatten': True, 'out_type': 'float32'})
def intgemm_fully_connected(data, weight, scaling=None, bias=None, num_hidden=0, no_bias=False, flatten=True, out_type='float32'):
    """int8 data (or float data, quantised on the fly with its own maximum) times prepared int8 weight, accumulated in
    int32; ``out_type='float32'`` multiplies by ``scaling`` and adds the bias, ``'int32'`` returns the raw sums."""
    x = data.reshape(data.shape[0], -1) if flatten and data.dim() > 2 else data
    mult = 1.0
    if x.dtype != torch.int8:
        m = x.abs().max().clamp(min=1e-30)
        mult = m / 127.0
        x = torch.clamp(torch.round(x / mult), -127, 127).to(torch.int8)
    if x.is_cuda and x.dim() == 2 and x.shape[0] > 16 and x.shape[1] % 8 == 0 and weight.shape[0] % 8 == 0:
        acc = torch._int_mm(x.contiguous(), weight.t().contiguous())
    else:
        acc = (x.to(torch.int32).cpu() @ weight.to(torch.int32).t().cpu()).to(x.device) if x.is_cuda else \
            x.to(torch.int32) @ weight.to(torch.int32).t()
    if out_type == 'int32':
        return acc
    out = acc.float() * (scaling.reshape(()) if scaling is not None else 1.0) * mult
    if bias is not None and not no_bias:
        out = out + bias
    return out


# ---- multi-tensor AdaBelief (contrib/adabelief.cc) ---------------------------------------------------------------------
def _multi_adabelief(mp):
    stride = 5 if mp else 4

    def op(*data, lrs=(), wds=(), etas=(), beta1=0.9, beta2=0.999, epsilon=1e-8, clip_gradient=-1.0, num_weights=1):
        from .optimizer_ops import adabelief_update, mp_adabelief_update, _seq
        n = int(num_weights)
        rs = data[-1]
        lrs, wds, etas = _seq(lrs, n), _seq(wds, n), _seq(etas, n)
        outs = []
        for i in range(n):
            a = data[i * stride:(i + 1) * stride]
            fn = mp_adabelief_update if mp else adabelief_update
            outs.append(fn(*a, rescale_grad=rs, lr=lrs[i], beta1=beta1, beta2=beta2, epsilon=epsilon, wd=wds[i], eta=etas[i],
                           clip_gradient=clip_gradient))
        return tuple(outs)
    return op


_ADABELIEF_DEFAULTS = {'lrs': (), 'wds': (), 'etas': (), 'beta1': 0.9, 'beta2': 0.999, 'epsilon': 1e-8, 'clip_gradient': -1.0,
                       'num_weights': 1}
register('_multi_adabelief_update', '_contrib_multi_adabelief_update', inputs=('*data',), nout=lambda a: a.get('num_weights', 1),
         defaults=_ADABELIEF_DEFAULTS)(_multi_adabelief(False))
register('_multi_mp_adabelief_update', '_contrib_multi_mp_adabelief_update', inputs=('*data',), nout=lambda a: a.get('num_weights', 1),
         defaults=_ADABELIEF_DEFAULTS)(_multi_adabelief(True))


# ---- more quantised operators (quantization/quantized_*.cc) -------------------------------------------------------------
def _qrange_of(t):
    return 127.0 if t.dtype == torch.int8 else 255.0


def _dq(q, lo, hi):
    return q.float() * (torch.maximum(lo.abs(), hi.abs()).reshape(()) / _qrange_of(q))


def _q_int8(x):
    m = x.abs().max().clamp(min=1e-30)
    return torch.clamp(torch.round(x * (127.0 / m)), -127, 127).to(torch.int8), (-m).reshape(1), m.reshape(1)


@register('_contrib_quantize_asym', 'quantize_asym', inputs=('data',), nout=3, defaults={'min_calib_range': None, 'max_calib_range': None})
def quantize_asym(data, min_calib_range=None, max_calib_range=None):
    """uint8 = round(scale * x + shift) with scale = 255 / (max - min), shift = -scale * min; returns (q, scale, shift)."""
    lo = torch.as_tensor(min_calib_range, dtype=torch.float32, device=data.device) if min_calib_range is not None else data.min().float()
    hi = torch.as_tensor(max_calib_range, dtype=torch.float32, device=data.device) if max_calib_range is not None else data.max().float()
    scale = 255.0 / (hi - lo).clamp(min=1e-30)
    shift = -scale * lo
    q = torch.clamp(torch.round(data.float() * scale + shift), 0, 255).to(torch.uint8)
    return q, scale.reshape(1), shift.reshape(1)


@register('_contrib_quantized_elemwise_mul', inputs=('lhs', 'rhs', 'lhs_min', 'lhs_max', 'rhs_min', 'rhs_max'), nout=3,
          defaults={'min_calib_range': None, 'max_calib_range': None, 'enable_float_output': False})
def quantized_elemwise_mul(lhs, rhs, lhs_min, lhs_max, rhs_min, rhs_max, min_calib_range=None, max_calib_range=None,
                           enable_float_output=False):
    out = _dq(lhs, lhs_min, lhs_max) * _dq(rhs, rhs_min, rhs_max)
    if enable_float_output:
        return out, out.min().reshape(1), out.max().reshape(1)
    return _q_int8(out)


@register('_contrib_quantized_npi_add', inputs=('lhs', 'rhs', 'lhs_min', 'lhs_max', 'rhs_min', 'rhs_max'), nout=3,
          defaults={'min_calib_range': None, 'max_calib_range': None})
def quantized_npi_add(lhs, rhs, lhs_min, lhs_max, rhs_min, rhs_max, min_calib_range=None, max_calib_range=None):
    return _q_int8(_dq(lhs, lhs_min, lhs_max) + _dq(rhs, rhs_min, rhs_max))


@register('_contrib_quantized_concat', inputs=('*data',), nout=3, defaults={'num_args': 1, 'dim': 1})
def quantized_concat(*data, num_args=1, dim=1):
    """Inputs: the n quantised arrays, then (min, max) of each; every part is rescaled to the widest range."""
    n = len(data) // 3
    parts, los, his = data[:n], data[n::2][:n], data[n + 1::2][:n]
    wide = torch.stack([torch.maximum(lo.abs(), hi.abs()).reshape(()) for lo, hi in zip(los, his)]).max()
    out = torch.cat([torch.clamp(torch.round(_dq(p, lo, hi) * (127.0 / wide)), -127, 127).to(torch.int8)
                     for p, lo, hi in zip(parts, los, his)], dim)
    return out, (-wide).reshape(1), wide.reshape(1)


@register('_contrib_quantized_embedding', inputs=('data', 'weight', 'min_weight', 'max_weight'), nout=3,
          defaults={'input_dim': 0, 'output_dim': 0, 'dtype': 'float32', 'sparse_grad': False})
def quantized_embedding(data, weight, min_weight, max_weight, **kw):
    return weight[data.long()], min_weight, max_weight


@register('_contrib_quantized_batch_norm', inputs=('data', 'gamma', 'beta', 'moving_mean', 'moving_var', 'min_data', 'max_data'), nout=3,
          defaults={'eps': 1e-3, 'momentum': 0.9, 'fix_gamma': True, 'use_global_stats': False, 'axis': 1,
                    'min_calib_range': None, 'max_calib_range': None})
def quantized_batch_norm(data, gamma, beta, moving_mean, moving_var, min_data, max_data, eps=1e-3, fix_gamma=True, axis=1,
                         min_calib_range=None, max_calib_range=None, **kw):
    x = _dq(data, min_data, max_data)
    shape = [1] * x.dim()
    shape[axis] = -1
    g = torch.ones_like(gamma) if fix_gamma else gamma
    y = (x - moving_mean.reshape(shape)) / torch.sqrt(moving_var.reshape(shape) + eps) * g.reshape(shape) + beta.reshape(shape)
    if min_calib_range is not None and max_calib_range is not None:
        m = max(abs(float(min_calib_range)), abs(float(max_calib_range)))
        q = torch.clamp(torch.round(y * (127.0 / m)), -127, 127).to(torch.int8)
        return q, torch.tensor([-m], device=y.device), torch.tensor([m], device=y.device)
    return _q_int8(y)


@register('_contrib_quantized_batch_norm_relu', inputs=('data', 'gamma', 'beta', 'moving_mean', 'moving_var', 'min_data', 'max_data'),
          nout=3, defaults=dict(get('_contrib_quantized_batch_norm').defaults))
def quantized_batch_norm_relu(*args, **kw):
    q, lo, hi = quantized_batch_norm(*args, **kw)
    return torch.clamp(q, min=0), torch.zeros_like(lo), hi


@register('_npx_quantized_reshape', inputs=('data', 'min_data', 'max_data'), nout=3, defaults={'newshape': (), 'reverse': False})
def quantized_reshape(data, min_data, max_data, newshape=(), reverse=False, **kw):
    return get('_npx_reshape').fn(data, newshape=newshape, reverse=reverse) if has('_npx_reshape') else data.reshape(newshape), \
        min_data, max_data


@register('_npx_quantized_transpose', inputs=('data', 'min_data', 'max_data'), nout=3, defaults={'axes': None})
def quantized_transpose(data, min_data, max_data, axes=None):
    return (data.permute(*axes) if axes else data.permute(*reversed(range(data.dim())))), min_data, max_data


@register('_contrib_quantized_rnn', 'quantized_rnn', inputs=('data', 'parameters', 'state', 'state_cell', 'data_scale', 'data_shift'),
          nout=lambda a: (1 + (2 if a.get('mode', 'lstm') == 'lstm' else 1)) if a.get('state_outputs') else 1,
          defaults=dict(get('RNN').defaults))
def quantized_rnn(data, parameters, state, state_cell=None, data_scale=None, data_shift=None, **attrs):
    """The RNN operator on asymmetrically quantised uint8 input (``q = round(scale * x + shift)``, the output of
    ``_contrib_quantize_asym``): the input is brought back to floating point and the recurrence runs in the precision of
    the parameters (``src/operator/quantization/quantized_rnn.cc``; lstm only in the reference)."""
    mode = attrs.get('mode', 'lstm')
    if mode != 'lstm':
        state_cell, data_scale, data_shift = None, state_cell, data_scale       # no cell state input for the other modes
    x = (data.to(parameters.dtype) - data_shift.reshape(()).to(parameters.dtype)) / data_scale.reshape(()).to(parameters.dtype)
    fn = get('RNN').fn
    return fn(x, parameters, state, state_cell, **attrs) if mode == 'lstm' else fn(x, parameters, state, **attrs)

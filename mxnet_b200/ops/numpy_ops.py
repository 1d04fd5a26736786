"""Remaining ``_npi_*`` operators: insertion/deletion, window functions, polynomials, set ops.

Reference: ``src/operator/numpy/**`` (47.8 kLoC).  Long-tail routines run through the tensor
library; a few with data-dependent output shapes go through NumPy on the host, as the reference
does with a device-to-host size copy for dynamic-shape outputs."""
from __future__ import annotations

import numpy as _np
import torch

from .registry import register
from .tensor import _dev
from ..base import to_torch_dtype


def _via_numpy(fn):
    def op(*arrays, **kw):
        dev = next((a.device for a in arrays if isinstance(a, torch.Tensor)), torch.device('cpu'))
        res = fn(*[a.detach().cpu().numpy() if isinstance(a, torch.Tensor) else a for a in arrays], **kw)
        if isinstance(res, tuple):
            return tuple(torch.from_numpy(_np.ascontiguousarray(r)).to(dev) for r in res)
        return torch.from_numpy(_np.ascontiguousarray(res)).to(dev)
    return op


register('_npi_insert', '_npi_insert_scalar', '_npi_insert_slice', '_npi_insert_tensor', inputs=('arr', 'values', 'obj_t'),
         defaults={'obj': None, 'axis': None})(
    lambda arr, values=None, obj_t=None, obj=None, axis=None, val=None, start=None, stop=None, step=None, int_ind=None:
    _via_numpy(_np.insert)(arr, obj_t.long() if obj_t is not None else (slice(start, stop, step) if obj is None and int_ind is None else (obj if obj is not None else int_ind)),
                           values if values is not None else val, axis=axis))
register('_npi_delete', inputs=('arr', 'obj_t'), defaults={'obj': None, 'axis': None})(
    lambda arr, obj_t=None, obj=None, axis=None, start=None, stop=None, step=None, int_ind=None:
    _via_numpy(_np.delete)(arr, obj_t.long() if obj_t is not None else (obj if obj is not None else
                                                                        (int_ind if int_ind is not None else slice(start, stop, step))), axis=axis))


def _window(fn):
    def op(M=1, ctx=None, dtype='float32'):
        return fn(M, periodic=False, dtype=to_torch_dtype(dtype or 'float32'), device=_dev(ctx))
    return op


register('_npi_hanning', inputs=(), defaults={'M': 1, 'ctx': None, 'dtype': 'float32'})(_window(torch.hann_window))
register('_npi_hamming', inputs=(), defaults={'M': 1, 'ctx': None, 'dtype': 'float32'})(_window(torch.hamming_window))
register('_npi_blackman', inputs=(), defaults={'M': 1, 'ctx': None, 'dtype': 'float32'})(_window(torch.blackman_window))


@register('_npi_polyval', inputs=('p', 'x'))
def polyval(p, x):
    out = torch.zeros_like(x)
    for c in p:
        out = out * x + c
    return out


@register('_npi_tril_indices', inputs=(), nout=2, defaults={'n': 1, 'k': 0, 'm': None})
def tril_indices(n=1, k=0, m=None):
    idx = torch.tril_indices(n, m or n, k)
    return idx[0], idx[1]


@register('_npi_fill_diagonal', inputs=('a',), defaults={'val': 0.0, 'wrap': False})
def fill_diagonal(a, val=0.0, wrap=False):
    out = a.clone()
    out.fill_diagonal_(val if not isinstance(val, (list, tuple)) else val[0], wrap)
    return out


@register('_npi_flatnonzero', inputs=('a',))
def flatnonzero(a):
    return torch.nonzero(a.reshape(-1)).reshape(-1)


@register('_npi_atleast_1d', inputs=('*arys',), nout=lambda a: a.get('num_args', 1))
def atleast_1d(*arys, num_args=None):
    r = torch.atleast_1d(*arys)
    return r if isinstance(r, tuple) else r


@register('_npi_atleast_2d', inputs=('*arys',), nout=lambda a: a.get('num_args', 1))
def atleast_2d(*arys, num_args=None):
    return torch.atleast_2d(*arys)


@register('_npi_atleast_3d', inputs=('*arys',), nout=lambda a: a.get('num_args', 1))
def atleast_3d(*arys, num_args=None):
    return torch.atleast_3d(*arys)


@register('_npi_logaddexp', inputs=('lhs', 'rhs'))
def logaddexp(lhs, rhs):
    return torch.logaddexp(lhs, rhs)


@register('_npi_fmax', inputs=('lhs', 'rhs'))
def fmax(lhs, rhs):
    return torch.fmax(lhs, rhs)


@register('_npi_fmin', inputs=('lhs', 'rhs'))
def fmin(lhs, rhs):
    return torch.fmin(lhs, rhs)


@register('_npi_fmod', inputs=('lhs', 'rhs'))
def fmod(lhs, rhs):
    return torch.fmod(lhs, rhs)


@register('_npi_heaviside', inputs=('lhs', 'rhs'))
def heaviside(lhs, rhs):
    return torch.heaviside(lhs, rhs)


@register('_npi_sinc', inputs=('data',))
def sinc(data):
    return torch.sinc(data)


@register('_npi_i0', inputs=('data',))
def i0(data):
    return torch.i0(data)


@register('_npi_isclose', inputs=('a', 'b'), defaults={'rtol': 1e-5, 'atol': 1e-8, 'equal_nan': False})
def isclose(a, b, rtol=1e-5, atol=1e-8, equal_nan=False):
    return torch.isclose(a, b, rtol, atol, equal_nan)


@register('_npi_median', inputs=('a',), defaults={'axis': None, 'keepdims': False})
def median(a, axis=None, keepdims=False):
    return torch.quantile(a.float(), 0.5, dim=axis, keepdim=keepdims).to(a.dtype if a.dtype.is_floating_point else torch.float32)


@register('_npi_cov', inputs=('m',), defaults={'rowvar': True, 'bias': False, 'ddof': None})
def cov(m, rowvar=True, bias=False, ddof=None):
    x = m if rowvar else m.t()
    return torch.cov(x, correction=(0 if bias else 1) if ddof is None else ddof)


@register('_npi_corrcoef', inputs=('x',))
def corrcoef(x):
    return torch.corrcoef(x)


register('_npi_intersect1d', inputs=('a', 'b'))(_via_numpy(_np.intersect1d))
register('_npi_union1d', inputs=('a', 'b'))(_via_numpy(_np.union1d))
register('_npi_setdiff1d', inputs=('a', 'b'))(_via_numpy(_np.setdiff1d))
register('_npi_in1d', inputs=('a', 'b'))(_via_numpy(_np.isin))
register('_npi_digitize', inputs=('x', 'bins'), defaults={'right': False})(_via_numpy(_np.digitize))
register('_npi_convolve', inputs=('a', 'v'), defaults={'mode': 'full'})(_via_numpy(_np.convolve))
register('_npi_correlate', inputs=('a', 'v'), defaults={'mode': 'valid'})(_via_numpy(_np.correlate))
register('_npi_unwrap', inputs=('p',))(_via_numpy(_np.unwrap))
register('_npi_trapz', inputs=('y',))(_via_numpy(_np.trapz if hasattr(_np, 'trapz') else _np.trapezoid))
register('_npi_gradient', inputs=('f',))(_via_numpy(_np.gradient))
register('_npi_partition', inputs=('a',), defaults={'kth': 0, 'axis': -1})(_via_numpy(_np.partition))
register('_npi_lexsort', inputs=('keys',))(_via_numpy(_np.lexsort))

"""``mx.np``: NumPy-compatible array class and functions.

Reference: ``python/mxnet/numpy/multiarray.py`` (13.4 kLoC) over the ``_npi_*`` operators.
``ndarray`` subclasses the shared array wrapper with NumPy semantics (boolean comparison results,
zero-dim arrays, dtype promotion); every function funnels through ``ops.registry.invoke`` so
autograd recording, AMP casting, profiling and deferred-compute tracing apply uniformly.
Functions without a native operator fall back to host NumPy like ``numpy/fallback.py`` does.
"""
from __future__ import annotations

import builtins as _bi

import numpy as _np
import torch

from .. import _state
from ..base import to_torch_dtype, numeric_types
from ..device import current_device, Device
from ..ndarray.ndarray import NDArray, _to_tensor
from ..ops import registry as _reg

__all__ = ['ndarray', 'array', 'asarray']

pi, e, inf, nan, euler_gamma = _np.pi, _np.e, _np.inf, _np.nan, _np.euler_gamma
PINF, NINF, NAN = _np.inf, -_np.inf, _np.nan
newaxis = None
float16, float32, float64 = _np.float16, _np.float32, _np.float64
int8, int16, int32, int64, uint8 = _np.int8, _np.int16, _np.int32, _np.int64, _np.uint8
uint16, uint32, uint64 = _np.uint16, _np.uint32, _np.uint64
bool_ = _np.bool_
bool = _np.bool_   # pylint: disable=redefined-builtin
dtype = _np.dtype
finfo, iinfo = _np.finfo, _np.iinfo
integer, floating, number, generic = _np.integer, _np.floating, _np.number, _np.generic


class ndarray(NDArray):   # pylint: disable=invalid-name
    """NumPy-semantics array (``mx.np.ndarray``)."""
    __slots__ = ()
    _kind = 'np'

    def __repr__(self):
        a = self.asnumpy()
        s = _np.array2string(a, separator=', ', prefix='array(')
        dt = ''
        if a.dtype not in (_np.float32, _np.int64, _np.bool_):
            dt = ', dtype=%s' % a.dtype
        dev = '' if self._ctx.device_type == 'cpu' else ', device=%s' % self._ctx
        return 'array(%s%s%s)' % (s, dt, dev)

    def __str__(self):
        return str(self.asnumpy())

    @property
    def dtype(self):
        from ..base import to_numpy_dtype
        return to_numpy_dtype(self._data.dtype)

    def astype(self, dtype, order='K', casting='unsafe', subok=True, copy=True):  # pylint: disable=arguments-differ
        td = to_torch_dtype(dtype)
        if not copy and td == self._data.dtype:
            return self
        return _reg.invoke('_npi_cast', [self], {'dtype': td})

    def item(self, *args):
        return self.asnumpy().item(*args)

    def ravel(self, order='C'):
        return self.reshape(-1)

    def flatten(self, order='C'):  # pylint: disable=arguments-differ
        return self.reshape(-1).copy()

    def nonzero(self):
        return nonzero(self)

    def to_device(self, device):
        return self.as_in_context(device)

    as_in_ctx = NDArray.as_in_context

    def __array_function__(self, func, types, args, kwargs):
        mx_fn = globals().get(func.__name__)
        if mx_fn is None or not callable(mx_fn):
            conv = lambda x: x.asnumpy() if isinstance(x, NDArray) else x
            return func(*[conv(a) for a in args], **{k: conv(v) for k, v in kwargs.items()})
        return mx_fn(*args, **kwargs)

    def __array_ufunc__(self, ufunc, method, *inputs, **kwargs):
        mx_fn = globals().get(ufunc.__name__)
        if method == '__call__' and mx_fn is not None:
            return mx_fn(*inputs, **kwargs)
        return NotImplemented


_reg._set_array_class('np', ndarray)


def _ctx_of(ctx, device):
    return ctx or device or current_device()


def _np_default_float():
    return torch.float64 if _state.state.np_default_dtype else torch.float32


def array(object, dtype=None, ctx=None, device=None, copy=True):  # pylint: disable=redefined-builtin
    ctx = _ctx_of(ctx, device)
    if isinstance(object, NDArray):
        t = object._data.to(device=ctx.torch_device, dtype=to_torch_dtype(dtype) or object._data.dtype)
        if copy and t is object._data:
            t = t.clone()
        return ndarray._from_tensor(t, ctx)
    if dtype is None:
        a = _np.asarray(object)
        if a.dtype.kind == 'O':
            a = _np.asarray([x.asnumpy() if isinstance(x, NDArray) else x for x in object])
        # python/mxnet/numpy/multiarray.py:2747-2760: without an explicit dtype everything that is not already an
        # mx.np.ndarray becomes float32, unless the NumPy default-dtype mode is on (then NumPy's own rules apply)
        from ..util import is_np_default_dtype
        td = to_torch_dtype(a.dtype) if is_np_default_dtype() else torch.float32
        return ndarray._from_tensor(torch.from_numpy(_np.ascontiguousarray(a)).to(device=ctx.torch_device, dtype=td), ctx)
    if isinstance(object, (list, tuple)) and any(isinstance(x, NDArray) for x in object):
        object = [x.asnumpy() if isinstance(x, NDArray) else x for x in object]
    return ndarray._from_tensor(_to_tensor(object, ctx, dtype, default_float32=False), ctx)


def asarray(a, dtype=None, ctx=None, device=None):
    if isinstance(a, ndarray) and (dtype is None or to_torch_dtype(dtype) == a._data.dtype):
        return a
    return array(a, dtype, ctx, device, copy=False)


def _shape(shape):
    if isinstance(shape, (int, _np.integer)):
        return (int(shape),)
    return tuple(int(s) for s in shape)


def _like(opname, a, attrs, out, ctx):
    r = _reg.invoke(opname, [a], attrs, out=out, kind='np')
    return r.as_in_context(ctx) if ctx is not None and out is None else r


def _init(opname, **attrs):
    return _reg.invoke(opname, [], attrs, kind='np')


def zeros(shape, dtype=None, order='C', ctx=None, device=None):
    return _init('_npi_zeros', shape=_shape(shape), ctx=_ctx_of(ctx, device), dtype=to_torch_dtype(dtype) or _np_default_float())


def ones(shape, dtype=None, order='C', ctx=None, device=None):
    return _init('_npi_ones', shape=_shape(shape), ctx=_ctx_of(ctx, device), dtype=to_torch_dtype(dtype) or _np_default_float())


def empty(shape, dtype=None, order='C', ctx=None, device=None):
    return zeros(shape, dtype, order, ctx, device)


def full(shape, fill_value, dtype=None, order='C', ctx=None, device=None, out=None):
    if isinstance(fill_value, NDArray):
        r = broadcast_to(fill_value.astype(dtype) if dtype else fill_value, _shape(shape)).copy()
    else:
        if dtype is None:
            dtype = _np_default_float() if isinstance(fill_value, float) else (torch.bool if isinstance(fill_value, _bi.bool) else torch.int64)
        r = _init('_npi_full', shape=_shape(shape), ctx=_ctx_of(ctx, device), dtype=to_torch_dtype(dtype), value=fill_value)
    if out is not None:
        out._data.copy_(r._data)
        return out
    return r


def zeros_like(a, dtype=None, order='C', ctx=None, out=None, device=None): return _like('_npi_zeros_like', a, {'dtype': dtype}, out, ctx or device)
def ones_like(a, dtype=None, order='C', ctx=None, out=None, device=None): return _like('_npi_ones_like', a, {'dtype': dtype}, out, ctx or device)
def empty_like(prototype, dtype=None, order='C', subok=False, shape=None): return zeros_like(prototype, dtype)
def full_like(a, fill_value, dtype=None, order='C', ctx=None, out=None, device=None): return _like('_npi_full_like', a, {'fill_value': fill_value, 'dtype': dtype}, out, ctx or device)


def arange(start, stop=None, step=1, dtype=None, ctx=None, device=None):
    if dtype is None:
        isf = any(isinstance(v, float) for v in (start, stop, step))
        dtype = _np_default_float() if isf else torch.int64
        if not isf and not _state.state.np_default_dtype:
            dtype = torch.float32   # the reference's np.arange defaults to float32 unless set_np(dtype=True)
    return _init('_npi_arange', start=start, stop=stop, step=step, ctx=_ctx_of(ctx, device), dtype=to_torch_dtype(dtype))


def linspace(start, stop, num=50, endpoint=True, retstep=False, dtype=None, axis=0, ctx=None, device=None):
    r = _init('_npi_linspace', start=start, stop=stop, num=num, endpoint=endpoint, ctx=_ctx_of(ctx, device),
              dtype=to_torch_dtype(dtype) or _np_default_float())
    if retstep:
        return r, (stop - start) / (num - 1 if endpoint else num)
    return r


def logspace(start, stop, num=50, endpoint=True, base=10.0, dtype=None, axis=0, ctx=None, device=None):
    return _init('_npi_logspace', start=start, stop=stop, num=num, endpoint=endpoint, base=base, ctx=_ctx_of(ctx, device),
                 dtype=to_torch_dtype(dtype) or _np_default_float())


def eye(N, M=None, k=0, dtype=None, ctx=None, device=None, **kwargs):
    return _init('_npi_eye', N=N, M=M or 0, k=k, ctx=_ctx_of(ctx, device), dtype=to_torch_dtype(dtype) or _np_default_float())


def identity(n, dtype=None, ctx=None, device=None):
    return eye(n, dtype=dtype, ctx=ctx, device=device)


def tri(N, M=None, k=0, dtype=None, ctx=None, device=None):
    return _init('_npi_tri', N=N, M=M, k=k, ctx=_ctx_of(ctx, device), dtype=to_torch_dtype(dtype) or _np_default_float())


def indices(dimensions, dtype=None, ctx=None, device=None):
    return _init('_npi_indices', dimensions=tuple(dimensions), ctx=_ctx_of(ctx, device), dtype=to_torch_dtype(dtype) or torch.int64)


def hanning(M, dtype=None, ctx=None, device=None): return _init('_npi_hanning', M=M, ctx=_ctx_of(ctx, device), dtype=dtype or 'float32')
def hamming(M, dtype=None, ctx=None, device=None): return _init('_npi_hamming', M=M, ctx=_ctx_of(ctx, device), dtype=dtype or 'float32')
def blackman(M, dtype=None, ctx=None, device=None): return _init('_npi_blackman', M=M, ctx=_ctx_of(ctx, device), dtype=dtype or 'float32')


def _wrap_scalar(x, like=None):
    if isinstance(x, NDArray):
        return x
    return array(x, ctx=like._ctx if like is not None else None)


# ---- unary ufuncs ---------------------------------------------------------------------------------
def _make_unary(np_name, opname):
    def fn(x, out=None, **kwargs):
        if not isinstance(x, NDArray):
            return getattr(_np, np_name)(x)
        return _reg.invoke(opname, [x], {}, out=out, kind='np')
    fn.__name__ = np_name
    return fn


for _np_name, _op in [
        ('abs', 'abs'), ('absolute', 'abs'), ('fabs', 'abs'), ('sign', 'sign'), ('sqrt', 'sqrt'), ('cbrt', 'cbrt'),
        ('square', 'square'), ('reciprocal', 'reciprocal'), ('negative', 'negative'), ('positive', 'identity'),
        ('exp', 'exp'), ('expm1', 'expm1'), ('log', 'log'), ('log10', 'log10'), ('log2', 'log2'), ('log1p', 'log1p'),
        ('sin', 'sin'), ('cos', 'cos'), ('tan', 'tan'), ('arcsin', 'arcsin'), ('arccos', 'arccos'), ('arctan', 'arctan'),
        ('sinh', 'sinh'), ('cosh', 'cosh'), ('tanh', 'tanh'), ('arcsinh', 'arcsinh'), ('arccosh', 'arccosh'),
        ('arctanh', 'arctanh'), ('degrees', 'degrees'), ('radians', 'radians'), ('rad2deg', 'degrees'), ('deg2rad', 'radians'),
        ('floor', 'floor'), ('ceil', 'ceil'), ('trunc', 'trunc'), ('rint', 'rint'), ('fix', 'fix'),
        ('isnan', 'isnan'), ('isinf', 'isinf'), ('isfinite', 'isfinite'), ('isposinf', 'isposinf'), ('isneginf', 'isneginf'),
        ('logical_not', '_npi_logical_not'), ('invert', '_npi_invert'), ('bitwise_not', '_npi_invert'),
        ('sinc', '_npi_sinc'), ('i0', '_npi_i0')]:
    globals()[_np_name] = _make_unary(_np_name, _op)


def around(x, decimals=0, out=None): return _reg.invoke('_npi_around', [x], {'decimals': decimals}, out=out, kind='np')
round = around   # pylint: disable=redefined-builtin
round_ = around


# ---- binary ufuncs --------------------------------------------------------------------------------
def _make_binary(np_name, base):
    def fn(x1, x2, out=None, **kwargs):
        a1, a2 = isinstance(x1, NDArray), isinstance(x2, NDArray)
        if a1 and a2:
            return _reg.invoke('_npi_' + base, [x1, x2], {}, out=out, kind='np')
        if a1:
            if isinstance(x2, numeric_types + (_bi.bool,)):
                return _reg.invoke('_npi_%s_scalar' % base, [x1], {'scalar': x2}, out=out, kind='np')
            return fn(x1, array(x2, ctx=x1._ctx), out=out)
        if a2:
            if isinstance(x1, numeric_types + (_bi.bool,)):
                return _reg.invoke('_npi_r%s_scalar' % base, [x2], {'scalar': x1}, out=out, kind='np')
            return fn(array(x1, ctx=x2._ctx), x2, out=out)
        return getattr(_np, np_name)(x1, x2)
    fn.__name__ = np_name
    return fn


for _np_name, _base in [
        ('add', 'add'), ('subtract', 'subtract'), ('multiply', 'multiply'), ('divide', 'true_divide'),
        ('true_divide', 'true_divide'), ('mod', 'mod'), ('remainder', 'mod'), ('power', 'power'),
        ('maximum', 'maximum'), ('minimum', 'minimum'), ('hypot', 'hypot'), ('floor_divide', 'floor_divide'),
        ('equal', 'equal'), ('not_equal', 'not_equal'), ('greater', 'greater'), ('greater_equal', 'greater_equal'),
        ('less', 'less'), ('less_equal', 'less_equal'), ('logical_and', 'logical_and'), ('logical_or', 'logical_or'),
        ('logical_xor', 'logical_xor'), ('bitwise_and', 'bitwise_and'), ('bitwise_or', 'bitwise_or'),
        ('bitwise_xor', 'bitwise_xor'), ('left_shift', 'left_shift'), ('right_shift', 'right_shift')]:
    globals()[_np_name] = _make_binary(_np_name, _base)


def _make_binary_tt(np_name, opname):
    def fn(x1, x2, out=None, **kwargs):
        like = x1 if isinstance(x1, NDArray) else x2
        return _reg.invoke(opname, [_wrap_scalar(x1, like), _wrap_scalar(x2, like)], {}, out=out, kind='np')
    fn.__name__ = np_name
    return fn


for _np_name, _op in [('arctan2', '_npi_arctan2'), ('copysign', '_npi_copysign'), ('ldexp', '_npi_ldexp'),
                      ('lcm', '_npi_lcm'), ('gcd', '_npi_gcd'), ('logaddexp', '_npi_logaddexp'), ('fmax', '_npi_fmax'),
                      ('fmin', '_npi_fmin'), ('fmod', '_npi_fmod'), ('heaviside', '_npi_heaviside')]:
    globals()[_np_name] = _make_binary_tt(_np_name, _op)


def matmul(a, b, out=None): return _reg.invoke('_npi_matmul', [a, b], {}, out=out, kind='np')
def dot(a, b, out=None): return _reg.invoke('_npi_dot', [_wrap_scalar(a), _wrap_scalar(b)], {}, out=out, kind='np')
def vdot(a, b): return _reg.invoke('_npi_vdot', [a, b], {}, kind='np')
def inner(a, b): return _reg.invoke('_npi_inner', [a, b], {}, kind='np')
def outer(a, b): return _reg.invoke('_npi_outer', [a, b], {}, kind='np')
def kron(a, b): return _reg.invoke('_npi_kron', [a, b], {}, kind='np')
def cross(a, b, axisa=-1, axisb=-1, axisc=-1, axis=None):
    if axis is not None:
        axisa = axisb = axisc = axis
    return _reg.invoke('_npi_cross', [a, b], {'axisa': axisa, 'axisb': axisb, 'axisc': axisc}, kind='np')


def tensordot(a, b, axes=2):
    if isinstance(axes, int):
        return _reg.invoke('_npi_tensordot_int_axes', [a, b], {'axes': axes}, kind='np')
    a_ax, b_ax = axes
    a_ax = (a_ax,) if isinstance(a_ax, int) else tuple(a_ax)
    b_ax = (b_ax,) if isinstance(b_ax, int) else tuple(b_ax)
    return _reg.invoke('_npi_tensordot', [a, b], {'a_axes_summed': a_ax, 'b_axes_summed': b_ax}, kind='np')


def einsum(subscripts, *operands, out=None, optimize=False):
    return _reg.invoke('_npi_einsum', list(operands), {'subscripts': subscripts, 'optimize': int(optimize)}, out=out, kind='np')


def trace(a, offset=0, axis1=0, axis2=1, out=None):
    return _reg.invoke('_npi_trace', [a], {'offset': offset, 'axis1': axis1, 'axis2': axis2}, out=out, kind='np')


# ---- reductions -----------------------------------------------------------------------------------
def _make_reduce(np_name, opname):
    def fn(a, axis=None, dtype=None, out=None, keepdims=False, **kwargs):
        if not isinstance(a, NDArray):
            a = array(a)
        attrs = {'axis': axis, 'keepdims': keepdims}
        if dtype is not None:
            attrs['dtype'] = dtype
        return _reg.invoke(opname, [a], attrs, out=out, kind='np')
    fn.__name__ = np_name
    return fn


for _np_name, _op in [('sum', '_npi_sum'), ('mean', '_npi_mean'), ('prod', '_npi_prod'), ('nansum', '_npi_nansum'),
                      ('nanprod', '_npi_nanprod')]:
    globals()[_np_name] = _make_reduce(_np_name, _op)


def _make_reduce_nodtype(np_name, opname):
    def fn(a, axis=None, out=None, keepdims=False, **kwargs):
        if not isinstance(a, NDArray):
            a = array(a)
        return _reg.invoke(opname, [a], {'axis': axis, 'keepdims': keepdims}, out=out, kind='np')
    fn.__name__ = np_name
    return fn


for _np_name, _op in [('max', '_npi_max'), ('amax', '_npi_max'), ('min', '_npi_min'), ('amin', '_npi_min'),
                      ('all', '_npi_all'), ('any', '_npi_any'), ('argmax', '_npi_argmax'), ('argmin', '_npi_argmin')]:
    globals()[_np_name] = _make_reduce_nodtype(_np_name, _op)


def std(a, axis=None, dtype=None, out=None, ddof=0, keepdims=False):
    return _reg.invoke('_npi_std', [a], {'axis': axis, 'ddof': ddof, 'keepdims': keepdims}, out=out, kind='np')


def var(a, axis=None, dtype=None, out=None, ddof=0, keepdims=False):
    return _reg.invoke('_npi_var', [a], {'axis': axis, 'ddof': ddof, 'keepdims': keepdims}, out=out, kind='np')


def cumsum(a, axis=None, dtype=None, out=None): return _reg.invoke('_npi_cumsum', [a], {'axis': axis, 'dtype': dtype}, out=out, kind='np')
def cumprod(a, axis=None, dtype=None, out=None): return _reg.invoke('_npi_cumprod', [a], {'axis': axis, 'dtype': dtype}, out=out, kind='np')
def median(a, axis=None, out=None, overwrite_input=None, keepdims=False): return _reg.invoke('_npi_median', [a], {'axis': axis, 'keepdims': keepdims}, out=out, kind='np')


def percentile(a, q, axis=None, out=None, overwrite_input=None, interpolation='linear', keepdims=False):
    if isinstance(q, NDArray):
        return _reg.invoke('_npi_percentile', [a, q], {'axis': axis, 'interpolation': interpolation, 'keepdims': keepdims}, out=out, kind='np')
    if isinstance(q, (list, tuple)):
        return percentile(a, array(q, dtype=a.dtype, ctx=a._ctx), axis, out, None, interpolation, keepdims)
    return _reg.invoke('_npi_percentile', [a], {'axis': axis, 'interpolation': interpolation, 'keepdims': keepdims, 'q_scalar': q}, out=out, kind='np')


def quantile(a, q, axis=None, out=None, overwrite_input=None, interpolation='linear', keepdims=False):
    return percentile(a, q * 100 if not isinstance(q, (list, tuple)) else [x * 100 for x in q], axis, out, None, interpolation, keepdims)


def average(a, axis=None, weights=None, returned=False, out=None):
    args = [a] if weights is None else [a, weights]
    return _reg.invoke('_npi_average', args, {'axis': axis, 'returned': returned, 'weighted': weights is not None}, kind='np')


def ptp(a, axis=None, keepdims=False): return globals()['max'](a, axis, keepdims=keepdims) - globals()['min'](a, axis, keepdims=keepdims)
def count_nonzero(a, axis=None): return globals()['sum'](not_equal(a, 0).astype('int64'), axis=axis)  # noqa: F821
def cov(m, y=None, rowvar=True, bias=False, ddof=None, fweights=None, aweights=None): return _reg.invoke('_npi_cov', [m], {'rowvar': rowvar, 'bias': bias, 'ddof': ddof}, kind='np')
def corrcoef(x, y=None, rowvar=True): return _reg.invoke('_npi_corrcoef', [x], {}, kind='np')


# ---- shape manipulation ---------------------------------------------------------------------------
def reshape(a, newshape, reverse=False, order='C'): return _reg.invoke('_npi_reshape', [a], {'newshape': _shape(newshape), 'reverse': reverse}, kind='np')
def ravel(x, order='C'): return reshape(x, (-1,))
def transpose(a, axes=None): return _reg.invoke('_npi_transpose', [a], {'axes': tuple(axes) if axes is not None else None}, kind='np')
def swapaxes(a, axis1, axis2): return _reg.invoke('_npi_swapaxes', [a], {'dim1': axis1, 'dim2': axis2}, kind='np')
def moveaxis(a, source, destination): return _reg.invoke('_npi_moveaxis', [a], {'source': source, 'destination': destination}, kind='np')
def rollaxis(a, axis, start=0): return _reg.invoke('_npi_rollaxis', [a], {'axis': axis, 'start': start}, kind='np')
def expand_dims(a, axis): return _reg.invoke('_npi_expand_dims', [a], {'axis': axis}, kind='np')
def squeeze(x, axis=None): return _reg.invoke('_npi_squeeze', [x], {'axis': axis}, kind='np')
def broadcast_to(array, shape): return _reg.invoke('_npi_broadcast_to', [array], {'shape': _shape(shape)}, kind='np')  # pylint: disable=redefined-outer-name


def broadcast_arrays(*args):
    shape = torch.broadcast_shapes(*[a.shape for a in args])
    return [broadcast_to(a, shape) for a in args]


def concatenate(seq, axis=0, out=None): return _reg.invoke('_npi_concatenate', list(seq), {'dim': axis}, out=out, kind='np')
def append(arr, values, axis=None): return concatenate([arr, _wrap_scalar(values, arr)], axis=axis)
def stack(arrays, axis=0, out=None): return _reg.invoke('_npi_stack', list(arrays), {'axis': axis}, out=out, kind='np')
def vstack(arrays, out=None): return _reg.invoke('_npi_vstack', list(arrays), {}, kind='np')
def hstack(arrays): return _reg.invoke('_npi_hstack', list(arrays), {}, kind='np')
def dstack(arrays): return _reg.invoke('_npi_dstack', list(arrays), {}, kind='np')
def column_stack(tup): return _reg.invoke('_npi_column_stack', list(tup), {}, kind='np')
row_stack = vstack


def split(ary, indices_or_sections, axis=0):
    ios = indices_or_sections if isinstance(indices_or_sections, int) else tuple(int(i) for i in indices_or_sections)
    r = _reg.invoke('_npi_split', [ary], {'indices_or_sections': ios, 'axis': axis}, kind='np')
    return r if isinstance(r, list) else [r]


def array_split(ary, indices_or_sections, axis=0):
    ios = indices_or_sections if isinstance(indices_or_sections, int) else tuple(int(i) for i in indices_or_sections)
    r = _reg.invoke('_npi_array_split', [ary], {'indices_or_sections': ios, 'axis': axis}, kind='np')
    return r if isinstance(r, list) else [r]


def hsplit(ary, indices_or_sections): return split(ary, indices_or_sections, 1 if ary.ndim > 1 else 0)
def vsplit(ary, indices_or_sections): return split(ary, indices_or_sections, 0)
def dsplit(ary, indices_or_sections): return split(ary, indices_or_sections, 2)
def tile(A, reps): return _reg.invoke('_npi_tile', [A], {'reps': reps}, kind='np')
def repeat(a, repeats, axis=None): return _reg.invoke('_npi_repeat', [a], {'repeats': repeats, 'axis': axis}, kind='np')
def flip(m, axis=None, out=None): return _reg.invoke('_npi_flip', [m], {'axis': axis}, out=out, kind='np')
def fliplr(m): return flip(m, 1)
def flipud(m): return flip(m, 0)
def roll(a, shift, axis=None): return _reg.invoke('_npi_roll', [a], {'shift': shift, 'axis': axis}, kind='np')
def rot90(m, k=1, axes=(0, 1)): return _reg.invoke('_npi_rot90', [m], {'k': k, 'axes': tuple(axes)}, kind='np')


def _atleast(opname):
    def fn(*arys):
        arys = [_wrap_scalar(a) for a in arys]
        r = _reg.invoke(opname, arys, {'num_args': len(arys)}, kind='np')
        return r[0] if isinstance(r, list) and len(r) == 1 else r
    return fn


atleast_1d, atleast_2d, atleast_3d = _atleast('_npi_atleast_1d'), _atleast('_npi_atleast_2d'), _atleast('_npi_atleast_3d')


def pad(x, pad_width, mode='constant', **kwargs):
    return _reg.invoke('_npi_pad', [x], {'pad_width': pad_width, 'mode': mode,
                                         'constant_values': kwargs.get('constant_values', 0)}, kind='np')


def meshgrid(*xi, indexing='xy', **kwargs):
    return _reg.invoke('_npi_meshgrid', list(xi), {'indexing': indexing, 'num_args': len(xi)}, kind='np')


def shape(a): return a.shape
def ndim(a): return a.ndim
def size(a, axis=None): return a.size if axis is None else a.shape[axis]
def copy(a): return _reg.invoke('_npi_copy', [a], {}, kind='np')
def may_share_memory(a, b, max_work=None): return a._data.data_ptr() == b._data.data_ptr()
shares_memory = may_share_memory
def result_type(*args): return _np.result_type(*[a.dtype if isinstance(a, NDArray) else a for a in args])
def can_cast(from_, to, casting='safe'): return _np.can_cast(from_.dtype if isinstance(from_, NDArray) else from_, to, casting)
def isscalar(x): return _np.isscalar(x)


# ---- indexing / sorting / searching ---------------------------------------------------------------
def take(a, indices, axis=None, mode='raise', out=None):
    if not isinstance(indices, NDArray):
        indices = array(indices, dtype='int64', ctx=a._ctx)
    return _reg.invoke('_npi_take', [a, indices], {'axis': axis, 'mode': 'clip' if mode == 'raise' else mode}, out=out, kind='np')


def take_along_axis(arr, indices, axis):
    if axis is None:
        arr, axis = arr.reshape(-1), 0
    return ndarray._from_tensor(torch.take_along_dim(arr._data, indices._data.long(), axis), arr._ctx)


def where(condition, x=None, y=None):
    if x is None and y is None:
        return nonzero(condition)
    return _reg.invoke('_npi_where', [condition, x, y], {}, kind='np')


def nonzero(a):
    r = _reg.invoke('_npi_nonzero', [a], {}, kind='np')
    return tuple(r[:, i] for i in range(a.ndim))


def argwhere(a): return _reg.invoke('_npi_nonzero', [a], {}, kind='np')
def flatnonzero(a): return _reg.invoke('_npi_flatnonzero', [a], {}, kind='np')
def clip(a, a_min, a_max, out=None): return _reg.invoke('_npi_clip', [a], {'a_min': a_min, 'a_max': a_max}, out=out, kind='np')
def sort(a, axis=-1, kind=None, order=None): return _reg.invoke('_npi_sort', [a], {'axis': axis, 'is_ascend': True}, kind='np')
def argsort(a, axis=-1, kind=None, order=None): return _reg.invoke('_npi_argsort', [a], {'axis': axis, 'is_ascend': True, 'dtype': 'int64'}, kind='np')
def searchsorted(a, v, side='left', sorter=None): return _reg.invoke('_npi_searchsorted', [a, _wrap_scalar(v, a)], {'side': side}, kind='np')
def diag(v, k=0): return _reg.invoke('_npi_diag', [v], {'k': k}, kind='np')
def diagonal(a, offset=0, axis1=0, axis2=1): return _reg.invoke('_npi_diagonal', [a], {'offset': offset, 'axis1': axis1, 'axis2': axis2}, kind='np')
def diagflat(v, k=0): return diag(v.reshape(-1), k)
def tril(m, k=0): return _reg.invoke('_npi_tril', [m], {'k': k}, kind='np')
def triu(m, k=0): return _reg.invoke('_npi_triu', [m], {'k': k}, kind='np')
def tril_indices(n, k=0, m=None): return tuple(_reg.invoke('_npi_tril_indices', [], {'n': n, 'k': k, 'm': m}, kind='np'))
def diff(a, n=1, axis=-1, prepend=None, append=None): return _reg.invoke('_npi_diff', [a], {'n': n, 'axis': axis}, kind='np')  # pylint: disable=redefined-outer-name
def ediff1d(ary, to_end=None, to_begin=None): return _reg.invoke('_npi_ediff1d', [ary], {}, kind='np')
def bincount(x, weights=None, minlength=0): return _reg.invoke('_npi_bincount', [x] + ([weights] if weights is not None else []), {'minlength': minlength}, kind='np')
def nan_to_num(x, copy=True, nan=0.0, posinf=None, neginf=None): return _reg.invoke('_npi_nan_to_num', [x], {'nan': nan, 'posinf': posinf, 'neginf': neginf}, kind='np')  # pylint: disable=redefined-outer-name
def isclose(a, b, rtol=1e-05, atol=1e-08, equal_nan=False): return _reg.invoke('_npi_isclose', [a, _wrap_scalar(b, a)], {'rtol': rtol, 'atol': atol, 'equal_nan': equal_nan}, kind='np')
def allclose(a, b, rtol=1e-05, atol=1e-08, equal_nan=False): return _bi.bool(isclose(a, b, rtol, atol, equal_nan).asnumpy().all())
def array_equal(a1, a2): return a1.shape == a2.shape and _bi.bool((a1 == a2).asnumpy().all())
def polyval(p, x): return _reg.invoke('_npi_polyval', [p, x], {}, kind='np')
def interp(x, xp, fp, left=None, right=None, period=None): return _reg.invoke('_npi_interp', [xp, fp, _wrap_scalar(x, xp)], {'left': left, 'right': right, 'period': period}, kind='np')
def fill_diagonal(a, val, wrap=False):
    a._data.copy_(_reg.invoke('_npi_fill_diagonal', [a], {'val': val, 'wrap': wrap}, kind='np')._data)


def unique(ar, return_index=False, return_inverse=False, return_counts=False, axis=None):
    r = _reg.invoke('_npi_unique', [ar], {'return_index': return_index, 'return_inverse': return_inverse,
                                          'return_counts': return_counts, 'axis': axis}, kind='np')
    return tuple(r) if isinstance(r, list) else r


def histogram(a, bins=10, range=None, normed=None, weights=None, density=None):  # pylint: disable=redefined-builtin
    if isinstance(bins, NDArray):
        r = _reg.invoke('_npi_histogram', [a, bins], {}, kind='np')
    else:
        if range is None:
            range = (float(a.min().asnumpy()), float(a.max().asnumpy()))
        r = _reg.invoke('_npi_histogram', [a], {'bin_cnt': bins, 'range': range}, kind='np')
    return tuple(r)


def insert(arr, obj, values, axis=None):
    r = _np.insert(arr.asnumpy(), obj.asnumpy().astype('int64') if isinstance(obj, NDArray) else obj,
                   values.asnumpy() if isinstance(values, NDArray) else values, axis=axis)
    return array(r, dtype=r.dtype, ctx=arr._ctx)


def delete(arr, obj, axis=None):
    r = _np.delete(arr.asnumpy(), obj.asnumpy().astype('int64') if isinstance(obj, NDArray) else obj, axis=axis)
    return array(r, dtype=r.dtype, ctx=arr._ctx)


def _host_fallback(name):
    """Functions without a device operator run on host NumPy (``python/mxnet/numpy/fallback.py``)."""
    npf = getattr(_np, name)

    def fn(*args, **kwargs):
        ctx = None
        def conv(x):
            nonlocal ctx
            if isinstance(x, NDArray):
                ctx = ctx or x._ctx
                return x.asnumpy()
            if isinstance(x, (list, tuple)):
                return type(x)(conv(v) for v in x)
            return x
        res = npf(*[conv(a) for a in args], **{k: conv(v) for k, v in kwargs.items()})
        def back(r):
            if isinstance(r, _np.ndarray):
                return array(r, dtype=r.dtype if r.dtype != _np.float64 or _state.state.np_default_dtype else 'float32', ctx=ctx)
            if isinstance(r, (list, tuple)):
                return type(r)(back(v) for v in r)
            return r
        return back(res)
    fn.__name__ = name
    return fn


for _n in ['intersect1d', 'union1d', 'setdiff1d', 'setxor1d', 'in1d', 'isin', 'digitize', 'convolve', 'correlate',
           'unwrap', 'gradient', 'partition', 'argpartition', 'lexsort', 'nanmax', 'nanmin', 'nanmean', 'nanstd',
           'nanvar', 'nanargmax', 'nanargmin', 'nancumsum', 'nancumprod', 'nanmedian', 'nanpercentile', 'nanquantile',
           'polyfit', 'poly', 'roots', 'polyadd', 'polysub', 'polymul', 'polydiv', 'polyder', 'polyint', 'vander',
           'triu_indices', 'triu_indices_from', 'tril_indices_from', 'diag_indices_from', 'unravel_index',
           'ravel_multi_index', 'apply_along_axis', 'apply_over_axes', 'piecewise', 'select', 'choose', 'compress',
           'extract', 'place', 'put', 'putmask', 'resize', 'trim_zeros', 'histogram2d', 'histogramdd',
           'histogram_bin_edges', 'packbits', 'unpackbits', 'real', 'imag', 'conj', 'conjugate', 'angle',
           'spacing', 'nextafter', 'modf', 'frexp', 'divmod', 'float_power', 'signbit', 'exp2', 'logaddexp2',
           'geomspace', 'bartlett', 'kaiser', 'trapz', 'cumulative_trapezoid', 'msort', 'sort_complex', 'ix_',
           'diag_indices', 'mask_indices', 'block', 'array_equiv', 'iscomplex', 'isreal', 'iscomplexobj',
           'isrealobj', 'min_scalar_type', 'promote_types', 'common_type', 'tensorinv', 'squeeze_']:
    if hasattr(_np, _n) and _n not in globals():
        globals()[_n] = _host_fallback(_n)


# ---------------------------------------------------------------------------------------------------------
# names of the array API standard (python/mxnet/numpy/multiarray.py: pow, atan2, asin ..., concat, permute_dims,
# bitwise_invert, bitwise_left_shift / bitwise_right_shift, from_dlpack)
# ---------------------------------------------------------------------------------------------------------
pow = power                      # pylint: disable=redefined-builtin
atan2 = arctan2
asin, acos, atan, asinh, acosh, atanh = arcsin, arccos, arctan, arcsinh, arccosh, arctanh
bitwise_invert = invert
bitwise_left_shift, bitwise_right_shift = left_shift, right_shift


def concat(arrays, axis=0, out=None):
    """``concatenate`` under its array-API name; ``axis=None`` joins the flattened inputs."""
    if axis is None:
        return concatenate([a.reshape(-1) for a in arrays], axis=0, out=out)
    return concatenate(arrays, axis=axis, out=out)


def permute_dims(a, axes=None):
    return transpose(a, axes)


def from_dlpack(x):
    """An ndarray sharing memory with any object that implements ``__dlpack__`` (or a DLPack capsule)."""
    import torch
    return ndarray._from_tensor(torch.utils.dlpack.from_dlpack(x))


def genfromtxt(*args, **kwargs):
    """``numpy.genfromtxt`` returning a framework array on ``ctx`` / ``device`` (default: the current device)."""
    ctx = kwargs.pop('ctx', None) or kwargs.pop('device', None)
    ret = _np.genfromtxt(*args, **kwargs)
    return array(ret, dtype=ret.dtype, ctx=ctx)


def set_printoptions(precision=None, threshold=None, **kwarg):
    """Printing of framework arrays goes through NumPy: this sets NumPy's print options."""
    if kwarg:
        raise NotImplementedError('mxnet_b200.numpy.set_printoptions only supports parameters precision and threshold for now.')
    _np.set_printoptions(precision=precision, threshold=threshold)


def _nd_diagonal(self, offset=0, axis1=0, axis2=1):
    return diagonal(self, offset=offset, axis1=axis1, axis2=axis2)


def _nd_reshape_view(self, *shape, **kwargs):
    """A reshaped view sharing memory with this array (a copy only when the layout makes a view impossible)."""
    if len(shape) == 1 and isinstance(shape[0], (list, tuple)):
        shape = tuple(shape[0])
    return ndarray._from_tensor(self._data.reshape(shape), self._ctx)


ndarray.diagonal = _nd_diagonal
ndarray.reshape_view = _nd_reshape_view
ndarray.mT = property(lambda self: swapaxes(self, -1, -2), doc='The array with its last two axes transposed.')

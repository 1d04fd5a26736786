"""``mx.np.linalg`` (``python/mxnet/numpy/linalg.py`` over cuSOLVER/cuBLAS-backed ``_npi_*`` ops)."""
from ..ops import registry as _reg

__all__ = ['norm', 'svd', 'cholesky', 'qr', 'inv', 'det', 'slogdet', 'solve', 'tensorinv', 'tensorsolve', 'pinv',
           'eigvals', 'eig', 'eigvalsh', 'eigh', 'lstsq', 'matrix_rank', 'multi_dot', 'matrix_power', 'cond']


def norm(x, ord=None, axis=None, keepdims=False):  # pylint: disable=redefined-builtin
    return _reg.invoke('_npi_norm', [x], {'ord': ord, 'axis': axis, 'keepdims': keepdims}, kind='np')


def svd(a): return tuple(_reg.invoke('_npi_svd', [a], {}, kind='np'))
def cholesky(a, upper=False): return _reg.invoke('_npi_cholesky', [a], {'upper': upper}, kind='np')
def qr(a, mode='reduced'): return tuple(_reg.invoke('_npi_qr', [a], {}, kind='np'))
def inv(a): return _reg.invoke('_npi_inv', [a], {}, kind='np')
def det(a): return _reg.invoke('_npi_det', [a], {}, kind='np')
def slogdet(a): return tuple(_reg.invoke('_npi_slogdet', [a], {}, kind='np'))
def solve(a, b): return _reg.invoke('_npi_solve', [a, b], {}, kind='np')
def tensorinv(a, ind=2): return _reg.invoke('_npi_tensorinv', [a], {'ind': ind}, kind='np')
def tensorsolve(a, b, axes=None): return _reg.invoke('_npi_tensorsolve', [a, b], {'a_axes': axes}, kind='np')
def pinv(a, rcond=1e-15, hermitian=False): return _reg.invoke('_npi_pinv', [a], {'rcond': rcond, 'hermitian': hermitian}, kind='np')
def eigvals(a): return _reg.invoke('_npi_eigvals', [a], {}, kind='np')
def eig(a): return tuple(_reg.invoke('_npi_eig', [a], {}, kind='np'))
def eigvalsh(a, UPLO='L'): return _reg.invoke('_npi_eigvalsh', [a], {'UPLO': UPLO}, kind='np')
def eigh(a, UPLO='L'): return tuple(_reg.invoke('_npi_eigh', [a], {'UPLO': UPLO}, kind='np'))
def lstsq(a, b, rcond='warn'): return tuple(_reg.invoke('_npi_lstsq', [a, b], {'rcond': None if rcond == 'warn' else rcond}, kind='np'))
def matrix_rank(M, tol=None, hermitian=False): return _reg.invoke('_npi_matrix_rank', [M], {'tol': tol, 'hermitian': hermitian}, kind='np')


def multi_dot(arrays):
    out = arrays[0]
    for a in arrays[1:]:
        out = _reg.invoke('_npi_dot', [out, a], {}, kind='np')
    return out


def matrix_power(a, n):
    from . import multiarray as mnp
    if n == 0:
        return mnp.eye(a.shape[-1], dtype=a.dtype, ctx=a.ctx)
    if n < 0:
        a, n = inv(a), -n
    out = a
    for _ in range(n - 1):
        out = _reg.invoke('_npi_matmul', [out, a], {}, kind='np')
    return out


def cond(x, p=None):
    s = svd(x)[1]
    return s.max(axis=-1) / s.min(axis=-1)


# ---------------------------------------------------------------------------------------------------------
# array-API additions of python/mxnet/numpy/linalg.py
# ---------------------------------------------------------------------------------------------------------
def _mx_np():
    from . import multiarray
    return multiarray


def cross(a, b, axis=-1): return _mx_np().cross(a, b, axis=axis)
def diagonal(a, offset=0): return _mx_np().diagonal(a, offset=offset, axis1=-2, axis2=-1)
def outer(a, b): return _mx_np().outer(a, b)
def tensordot(a, b, axes=2): return _mx_np().tensordot(a, b, axes)
def trace(a, offset=0): return _mx_np().trace(a, offset=offset, axis1=-2, axis2=-1)
def matrix_transpose(a): return _mx_np().swapaxes(a, -1, -2)


def vecdot(a, b, axis=-1):
    """Sum of products over ``axis`` with broadcasting of the other axes."""
    return _mx_np().sum(a * b, axis=axis)


def svdvals(a):
    """Singular values in descending order."""
    return svd(a)[1]


def vector_norm(x, axis=None, keepdims=False, ord=2):  # pylint: disable=redefined-builtin
    np_ = _mx_np()
    if axis is None:
        x, axis = x.reshape(-1), 0
    if isinstance(axis, (tuple, list)) and len(axis) > 1:      # flatten the reduced axes into one
        rest = [d for d in range(x.ndim) if d not in [ax % x.ndim for ax in axis]]
        lead = np_.transpose(x, rest + [ax % x.ndim for ax in axis])
        shape = tuple(x.shape[d] for d in rest)
        out = vector_norm(lead.reshape(shape + (-1,)), axis=-1, keepdims=False, ord=ord)
        if keepdims:
            full = [1 if d in [ax % x.ndim for ax in axis] else x.shape[d] for d in range(x.ndim)]
            out = out.reshape(tuple(full))
        return out
    if isinstance(axis, (tuple, list)):
        axis = axis[0]
    if ord == float('inf'):
        return np_.max(np_.abs(x), axis=axis, keepdims=keepdims)
    if ord == -float('inf'):
        return np_.min(np_.abs(x), axis=axis, keepdims=keepdims)
    if ord == 0:
        return np_.sum((x != 0).astype(x.dtype), axis=axis, keepdims=keepdims)
    if ord == 1:
        return np_.sum(np_.abs(x), axis=axis, keepdims=keepdims)
    if ord == 2:
        return np_.sqrt(np_.sum(x * x, axis=axis, keepdims=keepdims))
    return np_.power(np_.sum(np_.power(np_.abs(x), ord), axis=axis, keepdims=keepdims), 1.0 / ord)


def matrix_norm(x, keepdims=False, ord='fro'):  # pylint: disable=redefined-builtin
    return norm(x, ord=ord, axis=(-2, -1), keepdims=keepdims)


__all__ += ['cross', 'diagonal', 'outer', 'tensordot', 'trace', 'matrix_transpose', 'vecdot', 'svdvals', 'vector_norm',
            'matrix_norm']

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

"""Products of a compressed CSR matrix with a dense matrix on the in-tree kernels (``sparse.cu``)."""
import torch

from . import lib, ptr, stream_ptr, count_launch, check
from ._util import dt

_DT = (torch.float32, torch.float16, torch.bfloat16)


def supported(values, dense):
    return values.is_cuda and dense.is_cuda and values.dtype in _DT and dense.dtype == values.dtype and dense.dim() == 2 and \
        dense.shape[1] < (1 << 31)


def csr_dot_dense(values, indices, indptr, M, K, dense, transposed):
    """``csr[M, K] @ dense[K, N]`` (or ``csr.T @ dense[M, N]``) from the components; int64 indices."""
    dense = dense.contiguous()
    values, indices, indptr = values.contiguous(), indices.contiguous(), indptr.contiguous()
    N = int(dense.shape[1])
    if transposed:
        out = torch.zeros(K, N, dtype=torch.float32, device=dense.device)
    else:
        out = torch.empty(M, N, dtype=dense.dtype, device=dense.device)
    check(lib().mxb_csr_dot_dense(dt(dense), 1 if transposed else 0, ptr(values), ptr(indices), ptr(indptr), ptr(dense), ptr(out),
                                  int(M), N, stream_ptr(dense.device)), 'csr_dot_dense')
    count_launch(1)
    return out.to(dense.dtype) if transposed else out

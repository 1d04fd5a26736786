"""GEMM dispatch: FullyConnected / dot / batch_dot / matmul all land here.

Reference: every dense contraction goes to cuBLAS (``src/operator/linalg_impl.h``:
``cublasGemmEx``/``cublasGemmStridedBatchedEx`` with fp32 accumulation).  Here half-precision
CUDA operands whose sizes meet the tile constraints run on the hand-written tcgen05/TMEM kernel
(``ops/cuda/gemm_tcgen05.cu``); everything else (CPU, fp32/fp64, ragged shapes) is a plain
library GEMM.
"""
import torch

from .. import env


def _kernel_ok(a, b):
    if not (a.is_cuda and b.is_cuda) or a.dtype != b.dtype or a.dtype not in (torch.float16, torch.bfloat16):
        return False
    if not (env.get('MXNET_B200_KERNELS') and env.get('MXNET_B200_GEMM')):
        return False
    from . import cuda
    return cuda.available()


def linear(x, w, bias=None, act=None):
    """``y = x @ w.T + bias`` with optional fused activation ('relu' | 'gelu' | None).

    ``w`` is (N, K) as stored by FullyConnected / Dense, i.e. already K-major for the MMA."""
    if x.dim() == 2 and _kernel_ok(x, w):
        from .cuda import gemm_ops
        if gemm_ops.supported(x.shape[0], w.shape[0], x.shape[1]):
            return gemm_ops.LinearFn.apply(x, w, bias, act)
    y = torch.nn.functional.linear(x, w, bias)
    if act == 'relu':
        y = torch.relu(y)
    elif act == 'gelu':
        y = torch.nn.functional.gelu(y)
    return y


def matmul(a, b):
    """``a @ b`` for 2-D or batched operands."""
    if a.dim() == 2 and b.dim() == 2 and _kernel_ok(a, b):
        from .cuda import gemm_ops
        if gemm_ops.supported(a.shape[0], b.shape[1], a.shape[1]):
            return gemm_ops.MatmulFn.apply(a, b)
    return torch.matmul(a, b)


def batch_matmul(a, b, transpose_a=False, transpose_b=False):
    """``op(a[i]) @ op(b[i])`` over the leading batch axis (``batch_dot``).  Half-precision CUDA operands run as one
    batched launch of the tcgen05 kernel, reading ``a`` / ``b`` in their stored layout whatever the transpose flags."""
    if a.dim() == 3 and b.dim() == 3 and _kernel_ok(a, b):
        from .cuda import gemm_ops
        if gemm_ops.bgemm_supported(a, b):
            return gemm_ops.BatchMatmulFn.apply(a, b, bool(transpose_a), bool(transpose_b))
    return torch.matmul(a.transpose(-1, -2) if transpose_a else a, b.transpose(-1, -2) if transpose_b else b)

"""FullyConnected / matmul on the tcgen05 GEMM kernel (``gemm_tcgen05.cu``).

Forward and the data gradient run on the hand-written kernel (both are "TN" products: the second
operand is stored with the contraction axis contiguous).  The weight gradient contracts over the
row axis of both operands (an "NT" product in row-major terms); it needs MN-major operand
descriptors and is served by the library GEMM for now."""
import torch

from . import lib, ptr, stream_ptr, count_launch, check
from ._util import dt, require

_ACT = {None: 0, 'relu': 1, 'gelu': 2}
_err = {}


def _error_flag(device):
    f = _err.get(device)
    if f is None:
        f = _err[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return f


def check_errors():
    """Raise if any GEMM CTA gave up waiting on a barrier (the result would be incomplete)."""
    for dev, f in _err.items():
        if int(f.item()) != 0:
            f.zero_()
            raise RuntimeError('tcgen05 GEMM reported a barrier time-out on %s' % dev)


def supported(M, N, K):
    return M >= 1 and N >= 8 and K >= 8 and K % 8 == 0 and N % 8 == 0


def gemm_tn(a, b, bias=None, act=None, out=None):
    """``act(a @ b.T + bias)`` with a: [M, K], b: [N, K] (row-major, K contiguous)."""
    if not a.is_contiguous():
        a = a.contiguous()
    if not b.is_contiguous():
        b = b.contiguous()
    M, K = a.shape
    N = b.shape[0]
    require(a, 'a')
    require(b, 'b', dtype=a.dtype, device=a.device, shape=(N, K))
    if out is not None:
        require(out, 'out', dtype=a.dtype, device=a.device, shape=(M, N))
    if bias is not None:
        require(bias, 'bias', numel=N, device=a.device)
    d = out if out is not None else torch.empty(M, N, dtype=a.dtype, device=a.device)
    if bias is not None and bias.dtype != a.dtype:
        bias = bias.to(a.dtype)
    rc = lib().mxb_gemm_tn(dt(a), ptr(a), ptr(b), ptr(d), ptr(bias), M, N, K, K, K, N, _ACT[act],
                           ptr(_error_flag(a.device)), stream_ptr(a.device))
    check(rc, 'gemm_tn')
    count_launch(1)
    return d


class LinearFn(torch.autograd.Function):
    """y = act(x @ w.T + b)."""

    @staticmethod
    def forward(ctx, x, w, bias, act):
        y = gemm_tn(x, w, bias, act)
        ctx.save_for_backward(x, w, y if act is not None else None)
        ctx.act, ctx.has_bias = act, bias is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, y = ctx.saved_tensors
        dy = dy.contiguous()
        if ctx.act == 'relu':
            dy = dy * (y > 0).to(dy.dtype)
        elif ctx.act == 'gelu':
            raise RuntimeError('gelu epilogue has no fused backward; use act=None for training')
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            wt = w.t().contiguous()                    # [K, N]: contraction axis N contiguous
            if supported(dy.shape[0], wt.shape[0], wt.shape[1]):
                dx = gemm_tn(dy, wt)
            else:
                dx = dy @ w
        if ctx.needs_input_grad[1]:
            dw = torch.matmul(dy.t(), x)               # library GEMM (see module docstring)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.float().sum(0).to(ctx.bias_dtype)
        return dx, dw, db, None


class MatmulFn(torch.autograd.Function):
    """c = a @ b for 2-D operands."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return gemm_tn(a, b.t().contiguous())

    @staticmethod
    def backward(ctx, dc):
        a, b = ctx.saved_tensors
        dc = dc.contiguous()
        da = db = None
        if ctx.needs_input_grad[0]:
            da = gemm_tn(dc, b) if supported(dc.shape[0], b.shape[0], b.shape[1]) else dc @ b.t()
        if ctx.needs_input_grad[1]:
            db = torch.matmul(a.t(), dc)
        return da, db

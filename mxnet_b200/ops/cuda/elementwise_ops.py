"""Pointwise, gather and pooling operators on the sm_100a kernels (``elementwise.cu``).

Every function has a ``*_supported`` predicate; callers fall back to tensor operations for layouts the
vector kernels do not cover (sizes that are not multiples of a 16-byte vector, non-contiguous views)."""
import ctypes

import torch

from . import lib, ptr, stream_ptr, count_launch, check
from ._util import DT, dt, require

_seed = {}


def _next_seed(device):
    """Device-resident dropout counter, advanced by a (capturable) tensor op before every call so that graph replays
    draw fresh patterns; forward and backward of one call read the same returned copy."""
    s = _seed.get(device)
    if s is None:
        s = _seed[device] = torch.full((1,), (torch.initial_seed() * 2654435761) & 0x7fffffff, dtype=torch.int32,
                                       device=device)
    s.add_(0x632BE5AB)
    return s.clone()


def _vec(t):
    return 16 // t.element_size()


def pointwise_supported(x, cols=None):
    if not x.is_cuda or x.dtype not in DT or not x.is_contiguous() or x.numel() == 0:
        return False
    v = _vec(x)
    return x.numel() % v == 0 and x.numel() < 2 ** 32 and (cols is None or cols % v == 0) and x.data_ptr() % 16 == 0


# ----------------------------------------------------------------------------------------------- GELU
class _Gelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias):
        C = x.shape[-1]
        y = torch.empty_like(x)
        if bias is not None:
            require(bias, 'bias', numel=C, dtype=x.dtype, device=x.device)
        check(lib().mxb_gelu_forward(dt(x), ptr(x), ptr(bias), ptr(y), x.numel(), C, stream_ptr(x.device)), 'gelu_forward')
        count_launch(1)
        ctx.save_for_backward(x, bias)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, bias = ctx.saved_tensors
        dy = require(dy.contiguous(), 'out_grad', dtype=x.dtype, device=x.device, shape=x.shape)
        dx = torch.empty_like(x)
        check(lib().mxb_gelu_backward(dt(x), ptr(x), ptr(bias), ptr(dy), ptr(dx), x.numel(), x.shape[-1],
                                      stream_ptr(x.device)), 'gelu_backward')
        count_launch(1)
        db = dx.reshape(-1, x.shape[-1]).sum(0).to(bias.dtype) if bias is not None and ctx.needs_input_grad[1] else None
        return dx, db


def gelu(x, bias=None):
    """gelu(x + bias) with the erf form; bias broadcasts over the last axis."""
    return _Gelu.apply(x, bias)


# ----------------------------------------------------------------------------------------------- dropout
class _Dropout(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, residual, p):
        C = x.shape[-1]
        y = torch.empty_like(x)
        if bias is not None:
            require(bias, 'bias', numel=C, dtype=x.dtype, device=x.device)
        if residual is not None:
            require(residual, 'residual', dtype=x.dtype, device=x.device, shape=x.shape)
        seed = _next_seed(x.device) if p > 0 else None
        check(lib().mxb_dropout_forward(dt(x), ptr(x), ptr(bias), ptr(residual), ptr(y), x.numel(), C, float(p), ptr(seed),
                                        stream_ptr(x.device)), 'dropout_forward')
        count_launch(1)
        ctx.save_for_backward(seed)
        ctx.p, ctx.has_bias, ctx.has_res = p, bias is not None, residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        seed, = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty_like(dy)
        check(lib().mxb_dropout_backward(dt(dy), ptr(dy), ptr(dx), dy.numel(), float(ctx.p), ptr(seed),
                                         stream_ptr(dy.device)), 'dropout_backward')
        count_launch(1)
        db = dx.reshape(-1, dy.shape[-1]).sum(0) if ctx.has_bias and ctx.needs_input_grad[1] else None
        return dx, db, (dy if ctx.has_res else None), None


def dropout(x, p, bias=None, residual=None):
    """residual + dropout(x + bias, p): keep mask from a counter hash of a device-resident seed (no mask tensor)."""
    return _Dropout.apply(x, bias, residual, float(p))


# ----------------------------------------------------------------------------------------------- add_n / cast
def add_n_supported(tensors):
    t0 = tensors[0]
    return (pointwise_supported(t0) and all(t.shape == t0.shape and t.dtype == t0.dtype and t.is_contiguous() and
                                            t.device == t0.device and t.data_ptr() % 16 == 0 for t in tensors))


class _AddN(torch.autograd.Function):
    @staticmethod
    def forward(ctx, *tensors):
        ctx.n = len(tensors)
        return _add_n_raw(tensors)

    @staticmethod
    def backward(ctx, dy):
        return (dy,) * ctx.n


def add_n(tensors):
    """Sum of same-shaped tensors in one pass per group of eight (fp32 accumulation)."""
    return _AddN.apply(*tensors)


def _add_n_raw(tensors):
    L = lib()
    kmax = L.mxb_add_n_max()
    out = torch.empty_like(tensors[0])
    pending = list(tensors)
    first = True
    while pending:
        group = pending[:kmax] if first else [out] + pending[:kmax - 1]
        pending = pending[kmax:] if first else pending[kmax - 1:]
        arr = (ctypes.c_void_p * len(group))(*[t.data_ptr() for t in group])
        check(L.mxb_add_n(dt(out), arr, len(group), ptr(out), out.numel(), stream_ptr(out.device)), 'add_n')
        count_launch(1)
        first = False
    return out


def cast_supported(x, dtype):
    return (x.is_cuda and x.dtype in DT and dtype in DT and x.dtype != dtype and x.is_contiguous() and x.numel() > 0
            and x.data_ptr() % 16 == 0)


class _Cast(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dtype):
        ctx.src = x.dtype
        return cast_raw(x, dtype)

    @staticmethod
    def backward(ctx, dy):
        dy = dy.contiguous()
        return (cast_raw(dy, ctx.src) if cast_supported(dy, ctx.src) else dy.to(ctx.src)), None


def cast_raw(x, dtype):
    y = torch.empty(x.shape, dtype=dtype, device=x.device)
    check(lib().mxb_cast(DT[x.dtype], DT[dtype], ptr(x), ptr(y), x.numel(), stream_ptr(x.device)), 'cast')
    count_launch(1)
    return y


def cast(x, dtype):
    return _Cast.apply(x, dtype)


# ----------------------------------------------------------------------------------------------- embedding
def embedding_supported(idx, weight):
    return (weight.is_cuda and weight.dtype in DT and weight.dim() == 2 and weight.is_contiguous() and idx.is_cuda
            and idx.dtype in (torch.int32, torch.int64) and idx.numel() > 0 and weight.shape[1] % _vec(weight) == 0
            and weight.data_ptr() % 16 == 0)


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, idx, weight):
        idx = idx.contiguous()
        rows, D = weight.shape
        out = torch.empty(tuple(idx.shape) + (D,), dtype=weight.dtype, device=weight.device)
        check(lib().mxb_embedding_forward(dt(weight), ptr(idx), 1 if idx.dtype == torch.int64 else 0, ptr(weight), ptr(out),
                                          idx.numel(), D, rows, stream_ptr(weight.device)), 'embedding_forward')
        count_launch(1)
        ctx.save_for_backward(idx)
        ctx.wshape = (rows, D)
        return out

    @staticmethod
    def backward(ctx, dy):
        idx, = ctx.saved_tensors
        rows, D = ctx.wshape
        dy = require(dy.contiguous(), 'out_grad', numel=idx.numel() * D)
        sorted_idx, perm = torch.sort(idx.reshape(-1), stable=True)
        dw = torch.zeros((rows, D), dtype=dy.dtype, device=dy.device)
        partial = torch.empty(((idx.numel() + 31) // 32, 2, D), dtype=torch.float32, device=dy.device)
        check(lib().mxb_embedding_backward(dt(dy), ptr(sorted_idx), 1 if idx.dtype == torch.int64 else 0, ptr(perm), ptr(dy),
                                           ptr(dw), ptr(partial), idx.numel(), D, rows, 0, stream_ptr(dy.device)),
              'embedding_backward')
        count_launch(2)
        return None, dw


def embedding(idx, weight):
    """weight[idx] with a deterministic (sorted, segmented) gradient; indices are clipped to the table."""
    return _Embedding.apply(idx, weight)


# ----------------------------------------------------------------------------------------------- average pooling
def avgpool_supported(x):
    return (x.is_cuda and x.dim() == 4 and x.dtype in DT and x.is_contiguous() and x.numel() > 0
            and x.shape[-1] % _vec(x) == 0 and x.data_ptr() % 16 == 0)


class _AvgPoolNHWC(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, kernel, stride, pad, out_hw, include_pad):
        n, h, w, c = x.shape
        ho, wo = out_hw
        y = torch.empty((n, ho, wo, c), dtype=x.dtype, device=x.device)
        check(lib().mxb_avgpool_forward(dt(x), ptr(x), ptr(y), n, h, w, c, ho, wo, kernel[0], kernel[1], stride[0], stride[1],
                                        pad[0], pad[1], 1 if include_pad else 0, stream_ptr(x.device)), 'avgpool_forward')
        count_launch(1)
        ctx.geom = (n, h, w, c, ho, wo, kernel, stride, pad, include_pad)
        return y

    @staticmethod
    def backward(ctx, dy):
        n, h, w, c, ho, wo, kernel, stride, pad, include_pad = ctx.geom
        dy = require(dy.contiguous(), 'out_grad', shape=(n, ho, wo, c))
        dx = torch.empty((n, h, w, c), dtype=dy.dtype, device=dy.device)
        check(lib().mxb_avgpool_backward(dt(dy), ptr(dy), ptr(dx), n, h, w, c, ho, wo, kernel[0], kernel[1], stride[0],
                                         stride[1], pad[0], pad[1], 1 if include_pad else 0, stream_ptr(dy.device)),
              'avgpool_backward')
        count_launch(1)
        return dx, None, None, None, None, None


def avg_pool2d_nhwc(x, kernel, stride, pad, ceil_mode=False, count_include_pad=True):
    from .pool_ops import out_size
    ho = out_size(x.shape[1], kernel[0], stride[0], pad[0], ceil_mode)
    wo = out_size(x.shape[2], kernel[1], stride[1], pad[1], ceil_mode)
    return _AvgPoolNHWC.apply(x, tuple(kernel), tuple(stride), tuple(pad), (ho, wo), bool(count_include_pad))


def global_avg_pool_nhwc(x):
    return _AvgPoolNHWC.apply(x, (x.shape[1], x.shape[2]), (1, 1), (0, 0), (1, 1), True)


# ----------------------------------------------------------------------------------------------- column sums
def colsum_supported(x):
    return (x.is_cuda and x.dim() == 2 and x.dtype in DT and x.is_contiguous() and x.numel() > 0
            and x.shape[1] % _vec(x) == 0 and x.data_ptr() % 16 == 0)


def colsum(x):
    """fp32 column sums of a 2-D tensor (a bias gradient), two deterministic stages."""
    L = lib()
    rows, C = x.shape
    ny = L.mxb_colsum_chunks(dt(x), rows, C)
    partial = torch.empty((ny, C), dtype=torch.float32, device=x.device)
    out = torch.empty(C, dtype=torch.float32, device=x.device)
    check(L.mxb_colsum(dt(x), ptr(x), ptr(partial), ptr(out), rows, C, stream_ptr(x.device)), 'colsum')
    count_launch(2)
    return out


# ----------------------------------------------------------------------------------------------- transpose
def transpose_supported(x):
    return (x.is_cuda and x.dim() >= 2 and x.element_size() in (2, 4) and x.is_contiguous() and x.numel() > 0
            and x.numel() // (x.shape[-1] * x.shape[-2]) <= 65535 and not x.requires_grad)


def transpose_last2(x):
    """Contiguous copy of ``x`` with its last two axes swapped."""
    r, c = x.shape[-2], x.shape[-1]
    batch = x.numel() // (r * c)
    out = torch.empty(tuple(x.shape[:-2]) + (c, r), dtype=x.dtype, device=x.device)
    check(lib().mxb_transpose(x.element_size(), ptr(x), ptr(out), batch, r, c, stream_ptr(x.device)), 'transpose')
    count_launch(1)
    return out

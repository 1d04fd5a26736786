"""Row softmax and fused softmax cross-entropy on the sm_100a kernels (``softmax.cu``)."""
import torch

from . import lib, ptr, stream_ptr, count_launch, check
from ._util import dt, require


def supported(x):
    return x.dim() >= 1 and x.shape[-1] >= 1 and x.numel() > 0


class _Softmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, log):
        L = lib()
        C = x.shape[-1]
        rows = x.numel() // C
        require(x, 'data')
        y = torch.empty_like(x)
        check(L.mxb_softmax_forward(dt(x), ptr(x), ptr(y), rows, C, 1 if log else 0, stream_ptr(x.device)), 'softmax_forward')
        count_launch(1)
        ctx.save_for_backward(y)
        ctx.log = log
        return y

    @staticmethod
    def backward(ctx, dy):
        y, = ctx.saved_tensors
        L = lib()
        C = y.shape[-1]
        rows = y.numel() // C
        dy = require(dy.contiguous(), 'out_grad', dtype=y.dtype, device=y.device, shape=y.shape)
        dx = torch.empty_like(y)
        check(L.mxb_softmax_backward(dt(y), ptr(y), ptr(dy), ptr(dx), rows, C, 1 if ctx.log else 0, stream_ptr(y.device)),
              'softmax_backward')
        count_launch(1)
        return dx, None


def softmax(x, log=False):
    return _Softmax.apply(x, bool(log))


class _SoftmaxCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, label, ignore_label):
        L = lib()
        C = x.shape[-1]
        rows = x.numel() // C
        require(x, 'data')
        lab = require(label.reshape(-1).to(torch.int64).contiguous(), 'label', numel=rows, device=x.device)
        loss = torch.empty(rows, dtype=torch.float32, device=x.device)
        lse = torch.empty(rows, dtype=torch.float32, device=x.device)
        use_ignore = ignore_label is not None
        check(L.mxb_softmax_ce_forward(dt(x), ptr(x), ptr(lab), ptr(loss), ptr(lse), rows, C,
                                       int(ignore_label) if use_ignore else 0, 1 if use_ignore else 0,
                                       stream_ptr(x.device)), 'softmax_ce_forward')
        count_launch(1)
        ctx.save_for_backward(x, lab, lse)
        ctx.ignore = ignore_label
        return loss.reshape(x.shape[:-1])

    @staticmethod
    def backward(ctx, gout):
        x, lab, lse = ctx.saved_tensors
        L = lib()
        C = x.shape[-1]
        rows = x.numel() // C
        g = require(gout.reshape(-1).float().contiguous(), 'out_grad', numel=rows, device=x.device)
        dx = torch.empty_like(x)
        use_ignore = ctx.ignore is not None
        check(L.mxb_softmax_ce_backward(dt(x), ptr(x), ptr(lab), ptr(lse), ptr(g), ptr(dx), rows, C,
                                        int(ctx.ignore) if use_ignore else 0, 1 if use_ignore else 0,
                                        stream_ptr(x.device)), 'softmax_ce_backward')
        count_launch(1)
        return dx, None, None


def softmax_ce(x, label, ignore_label=None):
    return _SoftmaxCE.apply(x, label, ignore_label)

"""Fused multi-head self-attention on the tcgen05 kernels (``attention.cu``)."""
import torch

from . import lib, ptr, stream_ptr, count_launch, check
from ._util import dt, require

_err = {}
_seed = {}


def _error_flag(device):
    f = _err.get(device)
    if f is None:
        f = _err[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return f


def check_errors():
    for dev, f in _err.items():
        if int(f.item()) != 0:
            f.zero_()
            raise RuntimeError('attention kernel reported a barrier time-out on %s' % dev)


def _next_seed(device):
    """Device-resident dropout counter: advanced by a (capturable) tensor op before every call, so graph replays draw
    fresh patterns; the returned copy is what forward and backward of this call both read."""
    s = _seed.get(device)
    if s is None:
        s = _seed[device] = torch.full((1,), torch.initial_seed() & 0x7fffffff, dtype=torch.int32, device=device)
    s.add_(0x3C6EF35F)
    return s.clone()


def supported(qkv, heads):
    if qkv.dim() != 3 or qkv.shape[2] % 3 or not qkv.is_contiguous() or qkv.numel() == 0:
        return False
    return bool(lib().mxb_attn_supported(int(qkv.shape[1]), int(qkv.shape[2] // 3), int(heads)))


class _SelfAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, mask, heads, dropout):
        N, T, C3 = qkv.shape
        C = C3 // 3
        require(qkv, 'qkv')
        m = None
        if mask is not None:
            m = require(mask.reshape(N, T).float().contiguous(), 'mask', device=qkv.device, shape=(N, T))
        out = torch.empty(N, T, C, dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty(N, heads, T, dtype=torch.float32, device=qkv.device)
        seed = _next_seed(qkv.device) if dropout > 0 else None
        check(lib().mxb_attn_forward(dt(qkv), ptr(qkv), ptr(m), ptr(out), ptr(lse), N, T, C, heads, float(dropout), ptr(seed),
                                     ptr(_error_flag(qkv.device)), stream_ptr(qkv.device)), 'attn_forward')
        count_launch(1)
        ctx.save_for_backward(qkv, m, out, lse, seed)
        ctx.heads, ctx.dropout = heads, float(dropout)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, m, out, lse, seed = ctx.saved_tensors
        N, T, C3 = qkv.shape
        dout = require(dout.contiguous(), 'out_grad', dtype=qkv.dtype, device=qkv.device, shape=out.shape)
        dqkv = torch.empty_like(qkv)
        words = int(lib().mxb_attn_backward_workspace(N, T, C3 // 3))       # per-key-block dQ slots of the streaming kernels
        work = torch.empty(words, dtype=torch.float32, device=qkv.device) if words else None
        check(lib().mxb_attn_backward(dt(qkv), ptr(qkv), ptr(m), ptr(out), ptr(dout), ptr(lse), ptr(dqkv), ptr(work), N, T, C3 // 3,
                                      ctx.heads, ctx.dropout, ptr(seed), ptr(_error_flag(qkv.device)),
                                      stream_ptr(qkv.device)), 'attn_backward')
        count_launch(2 if words else 1)
        return dqkv, None, None, None


def fused_self_attention(qkv, mask, heads, dropout=0.0):
    return _SelfAttention.apply(qkv, mask, int(heads), float(dropout))

"""Contrib operators: transformer attention helpers, detection ops, quantization, misc.

Reference: ``src/operator/contrib/**`` (transformer.cc/.cu interleaved-matmul attention via
strided-batched cuBLAS ``transformer.cu:39-245``; bounding_box, multibox_*, roi_align, proposal;
fft, count_sketch, index_copy, quadratic, STE ops) and ``src/operator/quantization/**``.
The fused multi-head attention entry point :func:`fused_self_attention` replaces the
``interleaved_matmul_selfatt_qk → softmax → dropout → valatt`` chain with a single flash-style
pass that never materialises the (T, T) score matrix in global memory on the GPU.
"""
from __future__ import annotations

import math

import numpy as _np
import torch
import torch.nn.functional as F

from .registry import register, alias
from .. import _state, env
from ..base import to_torch_dtype


# ------------------------------------------------------------------------------------------
# transformer helpers
# ------------------------------------------------------------------------------------------
@register('_contrib_div_sqrt_dim', 'div_sqrt_dim', inputs=('data',))
def div_sqrt_dim(data):
    return data / math.sqrt(data.shape[-1])


def _split_qkv(qkv, heads):
    # (T, N, 3*H*D) interleaved per head as [q_h, k_h, v_h]
    T, N, _ = qkv.shape
    x = qkv.reshape(T, N, heads, 3, -1)
    return x[:, :, :, 0], x[:, :, :, 1], x[:, :, :, 2]


def _batch_matmul(a, b, transpose_a=False, transpose_b=False):
    """The per-head products of the interleaved attention operators: one batched launch of the tcgen05 GEMM for
    half-precision CUDA operands (the reference uses cublasGemmStridedBatchedEx, src/operator/contrib/transformer.cu:39-245)."""
    from . import gemm as _gemm
    return _gemm.batch_matmul(a, b, transpose_a, transpose_b)


@register('_contrib_interleaved_matmul_selfatt_qk', 'interleaved_matmul_selfatt_qk', inputs=('queries_keys_values',),
          defaults={'heads': 1})
def interleaved_matmul_selfatt_qk(queries_keys_values, heads=1):
    q, k, _ = _split_qkv(queries_keys_values, heads)
    T, N, H, D = q.shape
    q2 = q.permute(1, 2, 0, 3).reshape(N * H, T, D)
    k2 = k.permute(1, 2, 0, 3).reshape(N * H, T, D)
    return _batch_matmul(q2 / math.sqrt(D), k2, False, True)


@register('_contrib_interleaved_matmul_selfatt_valatt', 'interleaved_matmul_selfatt_valatt',
          inputs=('queries_keys_values', 'attention'), defaults={'heads': 1})
def interleaved_matmul_selfatt_valatt(queries_keys_values, attention, heads=1):
    _, _, v = _split_qkv(queries_keys_values, heads)
    T, N, H, D = v.shape
    v2 = v.permute(1, 2, 0, 3).reshape(N * H, T, D)
    out = _batch_matmul(attention, v2)
    return out.reshape(N, H, T, D).permute(2, 0, 1, 3).reshape(T, N, H * D)


@register('_contrib_interleaved_matmul_encdec_qk', 'interleaved_matmul_encdec_qk', inputs=('queries', 'keys_values'),
          defaults={'heads': 1})
def interleaved_matmul_encdec_qk(queries, keys_values, heads=1):
    Tq, N, _ = queries.shape
    Tk = keys_values.shape[0]
    q = queries.reshape(Tq, N, heads, -1)
    D = q.shape[-1]
    kv = keys_values.reshape(Tk, N, heads, 2, D)
    q2 = q.permute(1, 2, 0, 3).reshape(N * heads, Tq, D)
    k2 = kv[:, :, :, 0].permute(1, 2, 0, 3).reshape(N * heads, Tk, D)
    return _batch_matmul(q2 / math.sqrt(D), k2, False, True)


@register('_contrib_interleaved_matmul_encdec_valatt', 'interleaved_matmul_encdec_valatt',
          inputs=('keys_values', 'attention'), defaults={'heads': 1})
def interleaved_matmul_encdec_valatt(keys_values, attention, heads=1):
    Tk, N, _ = keys_values.shape
    kv = keys_values.reshape(Tk, N, heads, 2, -1)
    D = kv.shape[-1]
    v2 = kv[:, :, :, 1].permute(1, 2, 0, 3).reshape(N * heads, Tk, D)
    out = _batch_matmul(attention, v2)
    Tq = attention.shape[1]
    return out.reshape(N, heads, Tq, D).permute(2, 0, 1, 3).reshape(Tq, N, heads * D)


def _ew_kernels(t):
    if not (t.is_cuda and env.get('MXNET_B200_KERNELS') and env.get('MXNET_B200_ELEMENTWISE')):
        return None
    from . import cuda
    if not cuda.available():
        return None
    from .cuda import elementwise_ops
    return elementwise_ops


@register('_contrib_dropout_add', 'dropout_add', '_npx_dropout_add', inputs=('data', 'residual', 'bias'),
          defaults={'p': 0.5, 'mode': 'training'})
def dropout_add(data, residual, bias=None, p=0.5, mode='training'):
    """residual + Dropout(data + bias, p) in one pass over the tensors (the sub-layer output of a transformer block;
    the reference composes Dropout (src/operator/nn/dropout-inl.h) and elemwise_add)."""
    active = (mode == 'always') or _state.state.training
    p = float(p) if active else 0.0
    ew = _ew_kernels(data)
    if ew is not None and ew.pointwise_supported(data, data.shape[-1]) and residual.shape == data.shape and \
            residual.dtype == data.dtype and residual.is_contiguous() and \
            (bias is None or (bias.dtype == data.dtype and bias.dim() == 1 and bias.numel() == data.shape[-1])):
        return ew.dropout(data, p, bias, residual)
    x = data if bias is None else data + bias
    return residual + (F.dropout(x, p, True) if p > 0 else x)


@register('_contrib_bias_gelu', 'bias_gelu', '_npx_bias_gelu', inputs=('data', 'bias'))
def bias_gelu(data, bias=None):
    """gelu(data + bias), erf form, bias broadcast over the last axis (one pass; the reference composes broadcast_add
    and LeakyReLU(act_type='gelu'), src/operator/leaky_relu-inl.h)."""
    ew = _ew_kernels(data)
    if ew is not None and ew.pointwise_supported(data, data.shape[-1]) and \
            (bias is None or (bias.dtype == data.dtype and bias.is_contiguous() and bias.dim() == 1 and
                              bias.numel() == data.shape[-1])):
        return ew.gelu(data, bias)
    return F.gelu(data if bias is None else data + bias)


@register('_contrib_fused_self_attention', 'fused_self_attention', '_npx_fused_self_attention',
          inputs=('qkv', 'mask'), defaults={'heads': 1, 'dropout': 0.0, 'layout': 'NTC'})
def fused_self_attention(qkv, mask=None, heads=1, dropout=0.0, layout='NTC'):
    """Multi-head self-attention on a packed projection.

    ``qkv``: (N, T, 3*H*D) for layout 'NTC' (packed as [Q | K | V], each H*D wide) or the
    reference's interleaved (T, N, 3*H*D) for layout 'TNC'.  ``mask``: optional (N, T) validity
    mask of key positions (1 = attend).  Returns (N, T, H*D) / (T, N, H*D)."""
    training = _state.state.training
    p = dropout if training else 0.0
    if layout == 'TNC':
        q, k, v = _split_qkv(qkv, heads)                 # (T, N, H, D)
        q, k, v = (t.permute(1, 2, 0, 3) for t in (q, k, v))
    else:
        N, T, _ = qkv.shape
        x = qkv.reshape(N, T, 3, heads, -1)
        q, k, v = (x[:, :, i].permute(0, 2, 1, 3) for i in range(3))   # (N, H, T, D)
    if qkv.is_cuda and env.get('MXNET_B200_KERNELS') and env.get('MXNET_B200_ATTENTION') and layout == 'NTC' and \
            qkv.dtype in (torch.float16, torch.bfloat16):
        from . import cuda
        if cuda.available():
            from .cuda import attn_ops
            if attn_ops.supported(qkv, heads):
                return attn_ops.fused_self_attention(qkv.contiguous(), mask, heads, p)
    am = None
    if mask is not None:
        am = (mask != 0)[:, None, None, :]
    out = F.scaled_dot_product_attention(q, k, v, attn_mask=am, dropout_p=p)
    if layout == 'TNC':
        return out.permute(2, 0, 1, 3).reshape(out.shape[2], out.shape[0], -1)
    return out.permute(0, 2, 1, 3).reshape(out.shape[0], out.shape[2], -1)


@register('_contrib_sldwin_atten_mask_like', inputs=('score', 'dilation', 'valid_length'),
          defaults={'w': 1, 'symmetric': True})
def sldwin_atten_mask_like(score, dilation, valid_length, w=1, symmetric=True):
    N, T, H, W = score.shape
    i = torch.arange(T, device=score.device)[None, :, None, None]
    j = torch.arange(W, device=score.device)[None, None, None, :]
    off = (j - w) if symmetric else (j - w)
    pos = i + off * dilation.reshape(1, 1, H, 1).to(i.dtype)
    vl = valid_length.reshape(N, 1, 1, 1).to(i.dtype)
    m = (pos >= 0) & (pos < vl) & (i < vl)
    if not symmetric:
        m = m & (off <= 0)
    return m.to(score.dtype)


@register('_contrib_sldwin_atten_score', inputs=('query', 'key', 'dilation'), defaults={'w': 1, 'symmetric': True})
def sldwin_atten_score(query, key, dilation, w=1, symmetric=True):
    N, T, H, D = query.shape
    W = 2 * w + 1 if symmetric else w + 1
    out = query.new_zeros(N, T, H, W)
    for h in range(H):
        d = int(dilation[h].item())
        for j in range(W):
            off = (j - w) * d
            lo, hi = max(0, -off), min(T, T - off)
            if hi > lo:
                out[:, lo:hi, h, j] = (query[:, lo:hi, h] * key[:, lo + off:hi + off, h]).sum(-1)
    return out


@register('_contrib_sldwin_atten_context', inputs=('score', 'value', 'dilation'), defaults={'w': 1, 'symmetric': True})
def sldwin_atten_context(score, value, dilation, w=1, symmetric=True):
    N, T, H, W = score.shape
    out = torch.zeros_like(value)
    for h in range(H):
        d = int(dilation[h].item())
        for j in range(W):
            off = (j - w) * d
            lo, hi = max(0, -off), min(T, T - off)
            if hi > lo:
                out[:, lo:hi, h] += score[:, lo:hi, h, j:j + 1] * value[:, lo + off:hi + off, h]
    return out


# ------------------------------------------------------------------------------------------
# misc contrib
# ------------------------------------------------------------------------------------------
@register('_contrib_quadratic', 'quadratic', inputs=('data',), defaults={'a': 0.0, 'b': 0.0, 'c': 0.0})
def quadratic(data, a=0.0, b=0.0, c=0.0):
    return a * data * data + b * data + c


@register('_contrib_gradientmultiplier', 'gradientmultiplier', inputs=('data',), defaults={'scalar': 1.0})
def gradient_multiplier(data, scalar=1.0):
    return data * scalar + (data * (1 - scalar)).detach()


class _RoundSTE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return torch.round(x)

    @staticmethod
    def backward(ctx, g):
        return g


class _SignSTE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return torch.sign(x)

    @staticmethod
    def backward(ctx, g):
        return g


register('_contrib_round_ste', 'round_ste', inputs=('data',))(lambda data: _RoundSTE.apply(data))
register('_contrib_sign_ste', 'sign_ste', inputs=('data',))(lambda data: _SignSTE.apply(data))


@register('_contrib_index_copy', 'index_copy', inputs=('old_tensor', 'index_vector', 'new_tensor'))
def index_copy(old_tensor, index_vector, new_tensor):
    return old_tensor.index_copy(0, index_vector.long(), new_tensor)


@register('_contrib_index_array', 'index_array', inputs=('data',), defaults={'axes': None})
def index_array(data, axes=None):
    grids = torch.meshgrid(*[torch.arange(s, device=data.device) for s in data.shape], indexing='ij')
    idx = torch.stack(grids, -1)
    if axes is not None:
        idx = idx[..., list(axes)]
    return idx


@register('_npx_index_add', 'index_add', inputs=('a', 'ind', 'val'))
def index_add(a, ind, val):
    out = a.clone()
    idx = ind.long()
    out.index_put_(tuple(idx[i] for i in range(idx.shape[0])), val.expand(idx.shape[1:] + a.shape[idx.shape[0]:]).to(a.dtype),
                   accumulate=True)
    return out


@register('_npx_constraint_check', inputs=('input',), defaults={'msg': 'Constraint violated.'})
def constraint_check(input, msg='Constraint violated.'):   # pylint: disable=redefined-builtin
    """``array(True)`` when every element of the boolean input holds, else ValueError(msg)
    (``src/operator/numpy/np_constraint_check.cc``).  The value is read on the host, like the reference's check."""
    if input.device.type != 'meta' and not bool(input.all()):
        raise ValueError(msg)
    return torch.ones((), dtype=torch.bool, device=input.device)


@register('_npx_index_update', 'index_update', inputs=('a', 'ind', 'val'))
def index_update(a, ind, val):
    out = a.clone()
    idx = ind.long()
    out[tuple(idx[i] for i in range(idx.shape[0]))] = val.to(a.dtype)
    return out


@register('_contrib_allclose', 'allclose', inputs=('a', 'b'), defaults={'rtol': 1e-5, 'atol': 1e-8, 'equal_nan': True})
def allclose(a, b, rtol=1e-5, atol=1e-8, equal_nan=True):
    return torch.tensor([torch.allclose(a, b, rtol, atol, equal_nan)], dtype=torch.int32, device=a.device)


@register('_contrib_dynamic_reshape', inputs=('data', 'shape'))
def dynamic_reshape(data, shape):
    from .tensor import legacy_reshape_shape
    return data.reshape(legacy_reshape_shape(data.shape, [int(v) for v in shape.tolist()]))


@register('_contrib_fft', 'fft', inputs=('data',), defaults={'compute_size': 128})
def fft(data, compute_size=128):
    out = torch.fft.fft(data.float(), dim=-1)
    return torch.stack([out.real, out.imag], -1).reshape(data.shape[:-1] + (-1,)).to(data.dtype)


@register('_contrib_ifft', 'ifft', inputs=('data',), defaults={'compute_size': 128})
def ifft(data, compute_size=128):
    x = data.float().reshape(data.shape[:-1] + (-1, 2))
    out = torch.fft.ifft(torch.complex(x[..., 0], x[..., 1]), dim=-1) * x.shape[-2]
    return out.real.to(data.dtype)


@register('_contrib_count_sketch', 'count_sketch', inputs=('data', 'h', 's'), defaults={'out_dim': 1, 'processing_batch_size': 32})
def count_sketch(data, h, s, out_dim=1, processing_batch_size=32):
    out = data.new_zeros(data.shape[0], out_dim)
    out.index_add_(1, h.reshape(-1).long(), data * s.reshape(1, -1))
    return out


@register('_contrib_hawkesll', 'hawkesll', inputs=('lda', 'alpha', 'beta', 'state', 'lags', 'marks', 'valid_length', 'max_time'), nout=2)
def hawkesll(lda, alpha, beta, state, lags, marks, valid_length, max_time):
    """Log-likelihood of a marked self-exciting Hawkes process (``src/operator/contrib/hawkes_ll-inl.h``)."""
    N, T = lags.shape
    K = lda.shape[1]
    ll = lda.new_zeros(N)
    out_state = state.clone()
    for i in range(N):
        t = 0.0
        last = lda.new_zeros(K)
        st = state[i].clone()
        acc = lda.new_zeros(())
        L = int(valid_length[i].item())
        for j in range(L):
            ci = int(marks[i, j].item())
            t = t + lags[i, j]
            d = t - last[ci]
            ed = torch.exp(-beta[ci] * d)
            lam = lda[i, ci] + alpha[ci] * beta[ci] * st[ci] * ed
            comp = lda[i, ci] * d + alpha[ci] * st[ci] * (1 - ed)
            acc = acc + torch.log(lam) - comp
            st[ci] = 1 + st[ci] * ed
            last[ci] = t
        d = max_time[i] - last
        ed = torch.exp(-beta * d)
        acc = acc - (lda[i] * d + alpha * st * (1 - ed)).sum()
        out_state[i] = st * ed
        ll[i] = acc
    return ll, out_state


# ------------------------------------------------------------------------------------------
# detection
# ------------------------------------------------------------------------------------------
def _iou_matrix(a, b, fmt='corner'):
    if fmt == 'center':
        a = torch.cat([a[..., :2] - a[..., 2:] / 2, a[..., :2] + a[..., 2:] / 2], -1)
        b = torch.cat([b[..., :2] - b[..., 2:] / 2, b[..., :2] + b[..., 2:] / 2], -1)
    tl = torch.maximum(a[..., :, None, :2], b[..., None, :, :2])
    br = torch.minimum(a[..., :, None, 2:], b[..., None, :, 2:])
    wh = (br - tl).clamp(min=0)
    inter = wh[..., 0] * wh[..., 1]
    aa = ((a[..., 2] - a[..., 0]) * (a[..., 3] - a[..., 1]))[..., :, None]
    ab = ((b[..., 2] - b[..., 0]) * (b[..., 3] - b[..., 1]))[..., None, :]
    return inter / (aa + ab - inter).clamp(min=1e-12)


@register('_contrib_box_iou', 'box_iou', inputs=('lhs', 'rhs'), defaults={'format': 'corner'})
def box_iou(lhs, rhs, format='corner'):
    return _iou_matrix(lhs.reshape(-1, 4), rhs.reshape(-1, 4), format).reshape(lhs.shape[:-1] + rhs.shape[:-1])


@register('_contrib_box_nms', 'box_nms', '_contrib_box_non_maximum_suppression', inputs=('data',),
          defaults={'overlap_thresh': 0.5, 'valid_thresh': 0.0, 'topk': -1, 'coord_start': 2, 'score_index': 1,
                    'id_index': -1, 'background_id': -1, 'force_suppress': False, 'in_format': 'corner',
                    'out_format': 'corner'})
def box_nms(data, overlap_thresh=0.5, valid_thresh=0.0, topk=-1, coord_start=2, score_index=1, id_index=-1,
            background_id=-1, force_suppress=False, in_format='corner', out_format='corner'):
    shape = data.shape
    x = data.reshape(-1, shape[-2], shape[-1]).clone()
    out = torch.full_like(x, -1.0)
    for b in range(x.shape[0]):
        d = x[b]
        score = d[:, score_index]
        valid = score > valid_thresh
        if id_index >= 0 and background_id >= 0:
            valid = valid & (d[:, id_index] != background_id)
        idx = torch.nonzero(valid).reshape(-1)
        if idx.numel() == 0:
            continue
        order = idx[torch.argsort(score[idx], descending=True, stable=True)]
        if topk > 0:
            order = order[:topk]
        boxes = d[order, coord_start:coord_start + 4]
        ids = d[order, id_index] if id_index >= 0 else None
        det = _ew_kernels(d)
        if det is not None:
            from .cuda import detection_ops
            corners = boxes if in_format == 'corner' else torch.cat([boxes[:, :2] - boxes[:, 2:] / 2,
                                                                     boxes[:, :2] + boxes[:, 2:] / 2], 1)
            keep = detection_ops.nms_keep(corners, overlap_thresh, None if force_suppress else ids)
        else:
            iou = _iou_matrix(boxes, boxes, in_format)
            keep = torch.ones(order.numel(), dtype=torch.bool, device=d.device)
            for i in range(order.numel()):
                if not keep[i]:
                    continue
                sup = iou[i] > overlap_thresh
                if ids is not None and not force_suppress:
                    sup = sup & (ids == ids[i])
                sup[:i + 1] = False
                keep = keep & ~sup
        kept = d[order[keep]]
        if in_format != out_format:
            c = kept[:, coord_start:coord_start + 4]
            if out_format == 'center':
                c = torch.cat([(c[:, :2] + c[:, 2:]) / 2, c[:, 2:] - c[:, :2]], 1)
            else:
                c = torch.cat([c[:, :2] - c[:, 2:] / 2, c[:, :2] + c[:, 2:] / 2], 1)
            kept = kept.clone()
            kept[:, coord_start:coord_start + 4] = c
        out[b, :kept.shape[0]] = kept
    return out.reshape(shape)


@register('_contrib_bipartite_matching', 'bipartite_matching', inputs=('data',), nout=2,
          defaults={'is_ascend': False, 'threshold': 0.0, 'topk': -1})
def bipartite_matching(data, is_ascend=False, threshold=0.0, topk=-1):
    shape = data.shape
    x = data.reshape(-1, shape[-2], shape[-1])
    rows = torch.full((x.shape[0], shape[-2]), -1.0, device=data.device)
    cols = torch.full((x.shape[0], shape[-1]), -1.0, device=data.device)
    for b in range(x.shape[0]):
        flat = x[b].reshape(-1)
        order = torch.argsort(flat, descending=not is_ascend)
        cnt = 0
        for o in order.tolist():
            r, c = divmod(o, shape[-1])
            v = flat[o].item()
            if (v < threshold and not is_ascend) or (v > threshold and is_ascend):
                break
            if rows[b, r] < 0 and cols[b, c] < 0:
                rows[b, r], cols[b, c] = c, r
                cnt += 1
                if 0 < topk <= cnt:
                    break
    return rows.reshape(shape[:-1]), cols.reshape(shape[:-2] + shape[-1:])


@register('_contrib_ROIAlign', 'ROIAlign', inputs=('data', 'rois'),
          defaults={'pooled_size': (1, 1), 'spatial_scale': 1.0, 'sample_ratio': -1, 'position_sensitive': False, 'aligned': False})
def roi_align(data, rois, pooled_size=(1, 1), spatial_scale=1.0, sample_ratio=-1, position_sensitive=False, aligned=False):
    """Average of bilinear samples per output bin (``src/operator/contrib/roi_align.cc``): sampling points more than one
    pixel outside the map count as zero, points in the one-pixel border are clamped onto the edge."""
    ph, pw = pooled_size
    N, CI, H, W = data.shape
    C = CI // (ph * pw) if position_sensitive else CI
    if _ew_kernels(data) is not None:
        from .cuda import detection_ops
        if detection_ops.roi_align_supported(data, rois):
            return detection_ops.roi_align(data, rois, (ph, pw), spatial_scale, sample_ratio, position_sensitive, aligned)
    outs = []
    off = 0.5 if aligned else 0.0
    rois_host = rois.detach().float().cpu()
    dev = data.device
    for r in rois_host:
        b = int(r[0].item())
        if b < 0:
            outs.append(data.new_zeros(C, ph, pw))
            continue
        x1, y1, x2, y2 = [(float(v) * spatial_scale - off) for v in r[1:5]]
        rw, rh = x2 - x1, y2 - y1
        if not aligned:
            rw, rh = max(rw, 1.0), max(rh, 1.0)
        sh = sample_ratio if sample_ratio > 0 else max(int(math.ceil(rh / ph)), 1)
        sw = sample_ratio if sample_ratio > 0 else max(int(math.ceil(rw / pw)), 1)
        ys = y1 + (torch.arange(ph * sh, device=dev, dtype=torch.float32) + 0.5) * (rh / (ph * sh))
        xs = x1 + (torch.arange(pw * sw, device=dev, dtype=torch.float32) + 0.5) * (rw / (pw * sw))

        def axis(v, n):
            inside = (v >= -1.0) & (v <= n)
            v = v.clamp(min=0)
            lo = v.floor().long()
            top = lo >= n - 1
            lo = torch.where(top, torch.full_like(lo, n - 1), lo)
            hi = torch.where(top, lo, lo + 1)
            frac = torch.where(top, torch.zeros_like(v), v - lo)
            return lo, hi, frac, inside
        y0, y1i, ly, iny = axis(ys, H)
        x0, x1i, lx, inx = axis(xs, W)
        plane = data[b].float()                                          # (CI, H, W)
        top_rows, bot_rows = plane[:, y0], plane[:, y1i]                 # (CI, Sy, W)
        val = ((1 - ly)[None, :, None] * ((1 - lx) * top_rows[:, :, x0] + lx * top_rows[:, :, x1i]) +
               ly[None, :, None] * ((1 - lx) * bot_rows[:, :, x0] + lx * bot_rows[:, :, x1i]))
        val = val * (iny[:, None] & inx[None, :]).to(val.dtype)
        pooled = val.reshape(CI, ph, sh, pw, sw).mean((2, 4))
        if position_sensitive:
            pooled = pooled.reshape(C, ph, pw, ph, pw)
            ii, jj = torch.arange(ph, device=dev), torch.arange(pw, device=dev)
            pooled = pooled[:, ii[:, None], jj[None, :], ii[:, None], jj[None, :]]
        outs.append(pooled.to(data.dtype))
    return torch.stack(outs, 0) if outs else data.new_zeros(0, C, ph, pw)


def _bilinear_points(plane, y, x):
    """Bilinear samples of plane (C, H, W) at points (y, x) with the ROIAlign boundary rules: points more than one pixel
    outside the map give zero, points in the border are clamped onto the edge."""
    C, H, W = plane.shape
    inside = (y >= -1.0) & (y <= H) & (x >= -1.0) & (x <= W)
    y, x = y.clamp(min=0), x.clamp(min=0)
    y0, x0 = y.floor().long(), x.floor().long()
    ty, tx = y0 >= H - 1, x0 >= W - 1
    y0 = torch.where(ty, torch.full_like(y0, H - 1), y0)
    x0 = torch.where(tx, torch.full_like(x0, W - 1), x0)
    y1, x1 = torch.where(ty, y0, y0 + 1), torch.where(tx, x0, x0 + 1)
    ly, lx = torch.where(ty, torch.zeros_like(y), y - y0), torch.where(tx, torch.zeros_like(x), x - x0)
    flat = plane.reshape(C, H * W)
    val = ((1 - ly) * (1 - lx) * flat[:, y0 * W + x0] + (1 - ly) * lx * flat[:, y0 * W + x1] +
           ly * (1 - lx) * flat[:, y1 * W + x0] + ly * lx * flat[:, y1 * W + x1])
    return val * inside.to(val.dtype)


@register('_contrib_RROIAlign', 'RROIAlign', inputs=('data', 'rois'), defaults={'pooled_size': (1, 1), 'spatial_scale': 1.0, 'sampling_ratio': -1})
def rroi_align(data, rois, pooled_size=(1, 1), spatial_scale=1.0, sampling_ratio=-1):
    """ROIAlign over rotated boxes (batch index, centre x, centre y, width, height, angle in degrees): the sampling grid
    of every bin is rotated around the box centre (``src/operator/contrib/rroi_align.cc``)."""
    ph, pw = pooled_size
    N, C, H, W = data.shape
    dev = data.device
    outs = []
    for r in rois.detach().float().cpu():
        b = int(r[0].item())
        cx, cy = float(r[1]) * spatial_scale, float(r[2]) * spatial_scale
        rw, rh = max(float(r[3]) * spatial_scale, 1.0), max(float(r[4]) * spatial_scale, 1.0)
        theta = float(r[5]) * math.pi / 180.0
        gh = sampling_ratio if sampling_ratio > 0 else max(int(math.ceil(rh / ph)), 1)
        gw = sampling_ratio if sampling_ratio > 0 else max(int(math.ceil(rw / pw)), 1)
        yy = -rh / 2 + (torch.arange(ph * gh, device=dev, dtype=torch.float32) + 0.5) * (rh / (ph * gh))
        xx = -rw / 2 + (torch.arange(pw * gw, device=dev, dtype=torch.float32) + 0.5) * (rw / (pw * gw))
        yy, xx = torch.meshgrid(yy, xx, indexing='ij')
        x = xx * math.cos(theta) + yy * math.sin(theta) + cx
        y = yy * math.cos(theta) - xx * math.sin(theta) + cy
        val = _bilinear_points(data[b].float(), y.reshape(-1), x.reshape(-1))
        outs.append(val.reshape(C, ph, gh, pw, gw).mean((2, 4)).to(data.dtype))
    return torch.stack(outs, 0) if outs else data.new_zeros(0, C, ph, pw)


@register('_contrib_MultiBoxPrior', 'MultiBoxPrior', inputs=('data',),
          defaults={'sizes': (1.0,), 'ratios': (1.0,), 'clip': False, 'steps': (-1.0, -1.0), 'offsets': (0.5, 0.5)})
def multibox_prior(data, sizes=(1.0,), ratios=(1.0,), clip=False, steps=(-1.0, -1.0), offsets=(0.5, 0.5)):
    H, W = data.shape[2], data.shape[3]
    sy = steps[0] if steps[0] > 0 else 1.0 / H
    sx = steps[1] if steps[1] > 0 else 1.0 / W
    cy = (torch.arange(H, dtype=torch.float32, device=data.device) + offsets[0]) * sy
    cx = (torch.arange(W, dtype=torch.float32, device=data.device) + offsets[1]) * sx
    whs = [(s * H / W / 2 if False else s / 2 * math.sqrt(ratios[0]) * H / W, s / 2 / math.sqrt(ratios[0])) for s in sizes]
    whs += [(sizes[0] / 2 * math.sqrt(r) * H / W, sizes[0] / 2 / math.sqrt(r)) for r in ratios[1:]]
    gy, gx = torch.meshgrid(cy, cx, indexing='ij')
    anchors = []
    for w, h in whs:
        anchors.append(torch.stack([gx - w, gy - h, gx + w, gy + h], -1))
    out = torch.stack(anchors, 2).reshape(1, -1, 4)
    return out.clamp(0, 1) if clip else out


@register('_contrib_MultiBoxTarget', 'MultiBoxTarget', inputs=('anchor', 'label', 'cls_pred'), nout=3,
          defaults={'overlap_threshold': 0.5, 'ignore_label': -1.0, 'negative_mining_ratio': -1.0,
                    'negative_mining_thresh': 0.5, 'minimum_negative_samples': 0, 'variances': (0.1, 0.1, 0.2, 0.2)})
def multibox_target(anchor, label, cls_pred, overlap_threshold=0.5, ignore_label=-1.0, negative_mining_ratio=-1.0,
                    negative_mining_thresh=0.5, minimum_negative_samples=0, variances=(0.1, 0.1, 0.2, 0.2)):
    anchors = anchor.reshape(-1, 4)
    A = anchors.shape[0]
    B = label.shape[0]
    loc_t = anchors.new_zeros(B, A * 4)
    loc_m = anchors.new_zeros(B, A * 4)
    cls_t = anchors.new_zeros(B, A)
    aw, ah = anchors[:, 2] - anchors[:, 0], anchors[:, 3] - anchors[:, 1]
    ax, ay = (anchors[:, 0] + anchors[:, 2]) / 2, (anchors[:, 1] + anchors[:, 3]) / 2
    for b in range(B):
        gt = label[b]
        gt = gt[gt[:, 0] >= 0]
        if gt.shape[0] == 0:
            continue
        iou = _iou_matrix(anchors, gt[:, 1:5])
        best_gt = iou.argmax(1)
        best_iou = iou.max(1)[0]
        pos = best_iou > overlap_threshold
        force = iou.argmax(0)
        pos[force] = True
        best_gt[force] = torch.arange(gt.shape[0], device=anchor.device)
        g = gt[best_gt]
        gw, gh = g[:, 3] - g[:, 1], g[:, 4] - g[:, 2]
        gx, gy = (g[:, 1] + g[:, 3]) / 2, (g[:, 2] + g[:, 4]) / 2
        t = torch.stack([(gx - ax) / aw / variances[0], (gy - ay) / ah / variances[1],
                         torch.log(gw / aw) / variances[2], torch.log(gh / ah) / variances[3]], 1)
        m = pos.float()[:, None].expand(-1, 4)
        loc_t[b] = (t * m).reshape(-1)
        loc_m[b] = m.reshape(-1)
        cls_t[b] = torch.where(pos, g[:, 0] + 1, torch.zeros_like(g[:, 0]))
        if negative_mining_ratio > 0:
            npos = int(pos.sum().item())
            nneg = max(int(npos * negative_mining_ratio), minimum_negative_samples)
            bg = torch.softmax(cls_pred[b], 0)[0]
            cand = (~pos) & (best_iou < negative_mining_thresh)
            score = torch.where(cand, -bg, torch.full_like(bg, -float('inf')))
            keep = torch.zeros_like(pos)
            if nneg > 0:
                keep[torch.topk(score, min(nneg, A))[1]] = True
            keep = keep & cand
            cls_t[b] = torch.where(pos | keep, cls_t[b], torch.full_like(cls_t[b], ignore_label))
    return loc_t, loc_m, cls_t


@register('_contrib_MultiBoxDetection', 'MultiBoxDetection', inputs=('cls_prob', 'loc_pred', 'anchor'),
          defaults={'clip': True, 'threshold': 0.01, 'background_id': 0, 'nms_threshold': 0.5, 'force_suppress': False,
                    'variances': (0.1, 0.1, 0.2, 0.2), 'nms_topk': -1})
def multibox_detection(cls_prob, loc_pred, anchor, clip=True, threshold=0.01, background_id=0, nms_threshold=0.5,
                       force_suppress=False, variances=(0.1, 0.1, 0.2, 0.2), nms_topk=-1):
    B, C, A = cls_prob.shape
    anchors = anchor.reshape(-1, 4)
    aw, ah = anchors[:, 2] - anchors[:, 0], anchors[:, 3] - anchors[:, 1]
    ax, ay = (anchors[:, 0] + anchors[:, 2]) / 2, (anchors[:, 1] + anchors[:, 3]) / 2
    loc = loc_pred.reshape(B, A, 4)
    cx = loc[..., 0] * variances[0] * aw + ax
    cy = loc[..., 1] * variances[1] * ah + ay
    w = torch.exp(loc[..., 2] * variances[2]) * aw / 2
    h = torch.exp(loc[..., 3] * variances[3]) * ah / 2
    boxes = torch.stack([cx - w, cy - h, cx + w, cy + h], -1)
    if clip:
        boxes = boxes.clamp(0, 1)
    fg = torch.cat([cls_prob[:, :background_id], cls_prob[:, background_id + 1:]], 1)
    score, cid = fg.max(1)
    cid = torch.where(score > threshold, cid.float(), torch.full_like(score, -1.0))
    det = torch.cat([cid[..., None], score[..., None], boxes], -1)
    return box_nms(det, nms_threshold, threshold, nms_topk, 2, 1, 0, -1, force_suppress)


# ------------------------------------------------------------------------------------------
# quantization (src/operator/quantization/*)
# ------------------------------------------------------------------------------------------
def _qrange(out_type):
    return (0.0, 255.0, torch.uint8) if out_type == 'uint8' else (-127.0, 127.0, torch.int8)


@register('_contrib_quantize', 'quantize', inputs=('data', 'min_range', 'max_range'), nout=3, defaults={'out_type': 'uint8'})
def quantize(data, min_range, max_range, out_type='uint8'):
    lo, hi, dt = _qrange(out_type)
    mn, mx = min_range.reshape(()).float(), max_range.reshape(()).float()
    if out_type == 'uint8':
        scale = (hi - lo) / (mx - mn)
        q = torch.round((data.float() - mn) * scale).clamp(lo, hi).to(dt)
        return q, mn.reshape(1), mx.reshape(1)
    real = torch.maximum(mn.abs(), mx.abs())
    q = torch.round(data.float() * (hi / real)).clamp(lo, hi).to(dt)
    return q, (-real).reshape(1), real.reshape(1)


@register('_contrib_quantize_v2', 'quantize_v2', inputs=('data',), nout=3,
          defaults={'out_type': 'int8', 'min_calib_range': None, 'max_calib_range': None})
def quantize_v2(data, out_type='int8', min_calib_range=None, max_calib_range=None):
    if out_type == 'auto':
        out_type = 'uint8' if (min_calib_range is not None and min_calib_range >= 0) else 'int8'
    mn = torch.as_tensor(min_calib_range if min_calib_range is not None else data.min().item(), dtype=torch.float32, device=data.device)
    mx = torch.as_tensor(max_calib_range if max_calib_range is not None else data.max().item(), dtype=torch.float32, device=data.device)
    return quantize(data, mn, mx, out_type)


@register('_contrib_dequantize', 'dequantize', inputs=('data', 'min_range', 'max_range'), defaults={'out_type': 'float32'})
def dequantize(data, min_range, max_range, out_type='float32'):
    mn, mx = min_range.reshape(()).float(), max_range.reshape(()).float()
    if data.dtype == torch.uint8:
        return data.float() * ((mx - mn) / 255.0) + mn
    if data.dtype == torch.int32:
        return data.float() * (torch.maximum(mn.abs(), mx.abs()) / 2147483647.0)
    return data.float() * (torch.maximum(mn.abs(), mx.abs()) / 127.0)


@register('_contrib_requantize', 'requantize', inputs=('data', 'min_range', 'max_range'), nout=3,
          defaults={'out_type': 'int8', 'min_calib_range': None, 'max_calib_range': None})
def requantize(data, min_range, max_range, out_type='int8', min_calib_range=None, max_calib_range=None):
    real = dequantize(data, min_range, max_range)
    if min_calib_range is not None:
        mn = torch.as_tensor(min_calib_range, dtype=torch.float32, device=data.device)
        mx = torch.as_tensor(max_calib_range, dtype=torch.float32, device=data.device)
    else:
        mn, mx = real.min(), real.max()
    return quantize(real, mn, mx, 'int8')


def _int8_kernel_ok(x, w):
    if not (x.is_cuda and x.dtype == torch.int8 and w.dtype == torch.int8):
        return False
    if not (env.get('MXNET_B200_KERNELS') and env.get('MXNET_B200_GEMM')):
        return False
    from . import cuda
    from .cuda import gemm_ops
    return cuda.available() and gemm_ops.gemm_i8_supported(x, w)


@register('_contrib_quantized_fully_connected', inputs=('data', 'weight', 'bias', 'min_data', 'max_data', 'min_weight',
                                                        'max_weight', 'min_bias', 'max_bias'), nout=3,
          defaults={'num_hidden': 0, 'no_bias': False, 'flatten': True})
def quantized_fully_connected(data, weight, bias=None, min_data=None, max_data=None, min_weight=None, max_weight=None,
                              min_bias=None, max_bias=None, num_hidden=0, no_bias=False, flatten=True):
    x = data.reshape(data.shape[0], -1) if flatten else data
    sd = torch.maximum(min_data.abs(), max_data.abs()).reshape(()) / 127.0
    sw = torch.maximum(min_weight.abs(), max_weight.abs()).reshape(()) / 127.0
    qbias = None
    if bias is not None and not no_bias:
        sb = torch.maximum(min_bias.abs(), max_bias.abs()).reshape(()) / 127.0
        qbias = torch.round(bias.float() * sb / (sd * sw))
    out_range = sd * sw * 2147483647.0
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if _int8_kernel_ok(x2, weight):
        # tensor-core path: exact int8 x int8 products with int32 accumulation (tcgen05.mma.kind::i8)
        from .cuda import gemm_ops
        acc = gemm_ops.gemm_i8(x2, weight, qbias.to(torch.int32) if qbias is not None else None)
    else:
        # integer-valued float arithmetic: exact while the sums stay below 2**24 (fp32) / 2**53 (fp64 for long rows)
        ft = torch.float32 if x2.shape[-1] * 127 * 127 < (1 << 24) else torch.float64
        acc = torch.matmul(x2.to(ft), weight.to(ft).t())
        if qbias is not None:
            acc = acc + qbias.to(ft)
        acc = acc.to(torch.int32)
    return acc.reshape(*lead, weight.shape[0]), (-out_range).reshape(1), out_range.reshape(1)


@register('_contrib_quantized_conv', inputs=('data', 'weight', 'bias', 'min_data', 'max_data', 'min_weight', 'max_weight',
                                             'min_bias', 'max_bias'), nout=3,
          defaults={'kernel': (), 'stride': (), 'dilate': (), 'pad': (), 'num_filter': 0, 'num_group': 1, 'no_bias': False,
                    'layout': None})
def quantized_conv(data, weight, bias=None, min_data=None, max_data=None, min_weight=None, max_weight=None,
                   min_bias=None, max_bias=None, kernel=(), stride=(), dilate=(), pad=(), num_filter=0, num_group=1,
                   no_bias=False, layout=None, **_):
    sd = torch.maximum(min_data.abs(), max_data.abs()).reshape(()) / 127.0
    sw = torch.maximum(min_weight.abs(), max_weight.abs()).reshape(()) / 127.0
    qbias = None
    if bias is not None and not no_bias:
        sb = torch.maximum(min_bias.abs(), max_bias.abs()).reshape(()) / 127.0
        qbias = torch.round(bias.float() * sb / (sd * sw))
    out_range = sd * sw * 2147483647.0
    acc = _quantized_conv_i8(data, weight, qbias, stride, dilate, pad, num_group)
    if acc is None:
        # integer-valued float arithmetic (exact while the sums stay below 2**24)
        acc = F.conv2d(data.float(), weight.float(), None, tuple(stride) or 1, tuple(pad) or 0, tuple(dilate) or 1, num_group)
        if qbias is not None:
            acc = acc + qbias.reshape(1, -1, 1, 1)
        acc = acc.to(torch.int32)
    return acc, (-out_range).reshape(1), out_range.reshape(1)


def _quantized_conv_i8(data, weight, qbias, stride, dilate, pad, num_group):
    """2-D int8 convolution (NCHW) on the int8 tensor-core GEMM (``tcgen05.mma.kind::i8``, exact int32 accumulation): the
    receptive fields are gathered into rows (a strided view, one int8 copy: 1/4 of the bytes of the fp32 detour) and
    multiplied with the filter matrix.  Returns None where the kernel does not apply (reference: cuDNN int8 convolution,
    src/operator/quantization/quantized_conv.cu)."""
    if data.dim() != 4 or num_group != 1 or not (data.is_cuda and data.dtype == torch.int8 and weight.dtype == torch.int8):
        return None
    sh, sw_ = (tuple(stride) or (1, 1)) if not isinstance(stride, int) else (stride, stride)
    ph, pw = (tuple(pad) or (0, 0)) if not isinstance(pad, int) else (pad, pad)
    dil = (tuple(dilate) or (1, 1)) if not isinstance(dilate, int) else (dilate, dilate)
    if tuple(dil) != (1, 1):
        return None
    cout, cin, kh, kw = weight.shape
    if (cin * kh * kw) % 16 or cin != data.shape[1]:
        return None
    x = F.pad(data, (pw, pw, ph, ph)) if (ph or pw) else data
    if x.shape[2] < kh or x.shape[3] < kw:
        return None
    cols = x.unfold(2, kh, sh).unfold(3, kw, sw_)                     # [N, C, Ho, Wo, kh, kw], a view
    n, _, ho, wo = cols.shape[:4]
    a = cols.permute(0, 2, 3, 1, 4, 5).reshape(n * ho * wo, cin * kh * kw)
    b = weight.reshape(cout, cin * kh * kw)
    if not _int8_kernel_ok(a, b):
        return None
    from .cuda import gemm_ops
    acc = gemm_ops.gemm_i8(a, b, qbias.to(torch.int32) if qbias is not None else None)
    return acc.reshape(n, ho, wo, cout).permute(0, 3, 1, 2)


def _passthrough_q(name, fn):
    def op(data, min_data, max_data, **kw):
        return fn(data, **kw), min_data, max_data
    register('_contrib_quantized_' + name, inputs=('data', 'min_data', 'max_data'), nout=3)(op)


_passthrough_q('flatten', lambda d: d.reshape(d.shape[0], -1))
_passthrough_q('act', lambda d, act_type='relu': torch.relu(d))
_passthrough_q('reshape', lambda d, shape=(), **k: d.reshape(tuple(shape)))
_passthrough_q('transpose', lambda d, axes=None: d.permute(tuple(axes)) if axes else d.t())


@register('_contrib_quantized_pooling', inputs=('data', 'min_data', 'max_data'), nout=3)
def quantized_pooling(data, min_data, max_data, **kw):
    from .nn import pooling
    return pooling(data.float(), **kw).to(data.dtype), min_data, max_data


@register('_contrib_quantized_elemwise_add', inputs=('lhs', 'rhs', 'lhs_min', 'lhs_max', 'rhs_min', 'rhs_max'), nout=3)
def quantized_elemwise_add(lhs, rhs, lhs_min, lhs_max, rhs_min, rhs_max):
    a = dequantize(lhs, lhs_min, lhs_max)
    b = dequantize(rhs, rhs_min, rhs_max)
    s = a + b
    r = s.abs().max()
    return torch.round(s * (2147483647.0 / r)).to(torch.int32) if False else torch.round(s / r * 127).to(torch.int8), (-r).reshape(1), r.reshape(1)


@register('_contrib_calibrate_entropy', 'calibrate_entropy', inputs=('hist', 'hist_edges'), nout=2,
          defaults={'num_quantized_bins': 255})
def calibrate_entropy(hist, hist_edges, num_quantized_bins=255):
    """KL-divergence threshold search of the entropy calibration (``quantization/calibrate.cc``)."""
    h = hist.detach().cpu().numpy().astype(_np.float64)
    edges = hist_edges.detach().cpu().numpy()
    nbins = h.size
    zero = nbins // 2
    nhalf = num_quantized_bins // 2
    best, best_t = float('inf'), float(edges[-1])
    for i in range(nhalf, zero + 1):
        lo, hi = zero - i, zero + i + 1
        p = h[lo:hi].copy()
        p[0] += h[:lo].sum()
        p[-1] += h[hi:].sum()
        nz = p != 0
        nm = p.size // num_quantized_bins
        q = _np.zeros_like(p)
        for j in range(num_quantized_bins):
            s, e = j * nm, (j + 1) * nm if j < num_quantized_bins - 1 else p.size
            cnt = nz[s:e].sum()
            if cnt:
                q[s:e] = _np.where(nz[s:e], h[lo + s:lo + e].sum() / cnt, 0)
        ps, qs = p / max(p.sum(), 1e-12), q / max(q.sum(), 1e-12)
        mask = ps > 0
        kl = _np.sum(ps[mask] * _np.log(ps[mask] / _np.maximum(qs[mask], 1e-12)))
        if kl < best:
            best, best_t = kl, float(edges[hi]) if hi < edges.size else float(edges[-1])
    return torch.tensor([best_t], dtype=torch.float32), torch.tensor([best], dtype=torch.float32)


# ------------------------------------------------------------------------------------------
# Region-proposal, position-sensitive pooling and deformable convolution operators
# (src/operator/contrib/{proposal,multi_proposal,psroi_pooling,deformable_psroi_pooling,deformable_convolution,
#  modulated_deformable_convolution,mrcnn_mask_target}*).  Cold-path detection operators: tensor operations and the
#  library's detection primitives; differentiable with respect to the feature maps through autograd.
# ------------------------------------------------------------------------------------------
def _rpn_anchors(feature_stride, ratios, scales, device):
    """Base anchors of the region-proposal network (proposal-inl.h:188-226): for every ratio, then every scale."""
    base = float(feature_stride)
    ctr = 0.5 * (base - 1.0)
    out = []
    for ratio in ratios:
        size_ratios = math.floor(base * base / ratio)
        for scale in scales:
            w = math.floor(math.sqrt(size_ratios) + 0.5) * scale
            h = math.floor((w / scale * ratio) + 0.5) * scale
            out.append([ctr - 0.5 * (w - 1.0), ctr - 0.5 * (h - 1.0), ctr + 0.5 * (w - 1.0), ctr + 0.5 * (h - 1.0)])
    return torch.tensor(out, dtype=torch.float32, device=device)


def _greedy_nms(boxes, thresh, max_keep):
    """Greedy suppression in score order with the +1 pixel area convention (proposal.cc:204-256)."""
    n = boxes.shape[0]
    if _ew_kernels(boxes) is not None and n > 0:
        from .cuda import detection_ops
        keep = detection_ops.nms_keep(boxes, thresh, None, max_keep, plus_one=True)
        return torch.nonzero(keep).reshape(-1).tolist()
    area = (boxes[:, 2] - boxes[:, 0] + 1) * (boxes[:, 3] - boxes[:, 1] + 1)
    xx1 = torch.maximum(boxes[:, None, 0], boxes[None, :, 0])
    yy1 = torch.maximum(boxes[:, None, 1], boxes[None, :, 1])
    xx2 = torch.minimum(boxes[:, None, 2], boxes[None, :, 2])
    yy2 = torch.minimum(boxes[:, None, 3], boxes[None, :, 3])
    inter = (xx2 - xx1 + 1).clamp(min=0) * (yy2 - yy1 + 1).clamp(min=0)
    over = (inter / (area[:, None] + area[None, :] - inter) > thresh).cpu()
    suppressed = torch.zeros(n, dtype=torch.bool)
    keep = []
    for i in range(n):
        if len(keep) >= max_keep:
            break
        if suppressed[i]:
            continue
        keep.append(i)
        suppressed[i + 1:] |= over[i, i + 1:]
    return keep


def _proposal_one(scores, deltas, im_info, pre_n, post_n, threshold, min_size, scales, ratios, stride, iou_loss):
    A, H, W = scores.shape
    dev = scores.device
    anchors = _rpn_anchors(stride, ratios, scales, dev)                                   # (A, 4)
    shift_x = torch.arange(W, device=dev, dtype=torch.float32) * stride
    shift_y = torch.arange(H, device=dev, dtype=torch.float32) * stride
    shifts = torch.stack([shift_x[None, :].expand(H, W), shift_y[:, None].expand(H, W)] * 2, -1)   # (H, W, 4)
    boxes = (anchors[None, None] + shifts[:, :, None]).reshape(-1, 4)                     # index = (h*W + w)*A + a
    d = deltas.float().reshape(A, 4, H, W).permute(2, 3, 0, 1).reshape(-1, 4)
    score = scores.float().permute(1, 2, 0).reshape(-1).clone()
    im_h, im_w, im_scale = float(im_info[0]), float(im_info[1]), float(im_info[2])
    if iou_loss:
        pred = boxes + d
    else:
        w = boxes[:, 2] - boxes[:, 0] + 1.0
        h = boxes[:, 3] - boxes[:, 1] + 1.0
        cx = boxes[:, 0] + 0.5 * (w - 1.0)
        cy = boxes[:, 1] + 0.5 * (h - 1.0)
        pcx, pcy = d[:, 0] * w + cx, d[:, 1] * h + cy
        pw, ph = torch.exp(d[:, 2]) * w, torch.exp(d[:, 3]) * h
        pred = torch.stack([pcx - 0.5 * (pw - 1.0), pcy - 0.5 * (ph - 1.0), pcx + 0.5 * (pw - 1.0), pcy + 0.5 * (ph - 1.0)], 1)
    pred = torch.stack([pred[:, 0].clamp(0, im_w - 1), pred[:, 1].clamp(0, im_h - 1),
                        pred[:, 2].clamp(0, im_w - 1), pred[:, 3].clamp(0, im_h - 1)], 1)
    # positions beyond the real (unpadded) image get score -1
    real_h, real_w = int(im_h / stride), int(im_w / stride)
    hh = torch.arange(H, device=dev)[:, None, None].expand(H, W, A).reshape(-1)
    ww = torch.arange(W, device=dev)[None, :, None].expand(H, W, A).reshape(-1)
    score[(hh >= real_h) | (ww >= real_w)] = -1.0
    # boxes below the minimum size are grown by min_size/2 on every side and demoted
    ms = min_size * im_scale
    small = ((pred[:, 2] - pred[:, 0] + 1.0) < ms) | ((pred[:, 3] - pred[:, 1] + 1.0) < ms)
    grow = torch.tensor([-ms / 2, -ms / 2, ms / 2, ms / 2], device=dev)
    pred = torch.where(small[:, None], pred + grow, pred)
    score[small] = -1.0
    count = score.numel()
    pre_n = count if pre_n <= 0 else min(pre_n, count)
    post_n_eff = min(post_n, pre_n)
    order = torch.sort(score, descending=True, stable=True)[1][:pre_n]
    props, sc = pred[order], score[order]
    keep = _greedy_nms(props, threshold, post_n_eff)
    idx = torch.tensor([keep[i] if i < len(keep) else keep[i % len(keep)] for i in range(post_n)], device=dev)
    return props[idx], sc[idx]


def _proposal_nout(attrs):
    return 2 if attrs.get('output_score') in (True, 'True', 1, '1') else 1


_PROPOSAL_DEFAULTS = {'rpn_pre_nms_top_n': 6000, 'rpn_post_nms_top_n': 300, 'threshold': 0.7, 'rpn_min_size': 16,
                      'scales': (4.0, 8.0, 16.0, 32.0), 'ratios': (0.5, 1.0, 2.0), 'feature_stride': 16,
                      'output_score': False, 'iou_loss': False}


@register('_contrib_MultiProposal', 'MultiProposal', '_contrib_Proposal', 'Proposal', inputs=('cls_prob', 'bbox_pred', 'im_info'),
          nout=_proposal_nout, defaults=_PROPOSAL_DEFAULTS)
def multi_proposal(cls_prob, bbox_pred, im_info, rpn_pre_nms_top_n=6000, rpn_post_nms_top_n=300, threshold=0.7,
                   rpn_min_size=16, scales=(4.0, 8.0, 16.0, 32.0), ratios=(0.5, 1.0, 2.0), feature_stride=16,
                   output_score=False, iou_loss=False):
    """Region proposals from RPN scores and box deltas: anchors -> decoded boxes -> clip -> min-size filter -> top-k ->
    greedy NMS -> fixed-size output (batch index, x1, y1, x2, y2), padded by cycling through the kept boxes.
    ``Proposal`` is the single-image form of the same computation."""
    N, A2, H, W = cls_prob.shape
    A = A2 // 2
    rois, scores = [], []
    with torch.no_grad():
        for b in range(N):
            r, s = _proposal_one(cls_prob[b, A:], bbox_pred[b], im_info[b].tolist(), int(rpn_pre_nms_top_n),
                                 int(rpn_post_nms_top_n), float(threshold), float(rpn_min_size), tuple(scales), tuple(ratios),
                                 int(feature_stride), bool(iou_loss))
            rois.append(torch.cat([torch.full((r.shape[0], 1), float(b), device=r.device), r], 1))
            scores.append(s[:, None])
    rois = torch.cat(rois, 0).to(cls_prob.dtype)
    if output_score:
        return rois, torch.cat(scores, 0).to(cls_prob.dtype)
    return rois


@register('_contrib_PSROIPooling', 'PSROIPooling', inputs=('data', 'rois'),
          defaults={'spatial_scale': 1.0, 'output_dim': 1, 'pooled_size': 1, 'group_size': 0})
def psroi_pooling(data, rois, spatial_scale=1.0, output_dim=1, pooled_size=1, group_size=0):
    """Position-sensitive ROI average pooling (R-FCN): output channel c of bin (ph, pw) averages input channel
    (c * G + gh) * G + gw over the bin (psroi_pooling.cu:36-90)."""
    P = int(pooled_size)
    G = int(group_size) or P
    N, C, H, W = data.shape
    out = data.new_zeros((rois.shape[0], int(output_dim), P, P))
    r_cpu = rois.detach().float().cpu()
    ctop = torch.arange(int(output_dim), device=data.device)
    for n in range(rois.shape[0]):
        b = int(r_cpu[n, 0])
        x1 = round(float(r_cpu[n, 1])) * spatial_scale
        y1 = round(float(r_cpu[n, 2])) * spatial_scale
        x2 = (round(float(r_cpu[n, 3])) + 1.0) * spatial_scale
        y2 = (round(float(r_cpu[n, 4])) + 1.0) * spatial_scale
        rw, rh = max(x2 - x1, 0.1), max(y2 - y1, 0.1)
        bh, bw = rh / P, rw / P
        for ph in range(P):
            hs = min(max(int(math.floor(ph * bh + y1)), 0), H)
            he = min(max(int(math.ceil((ph + 1) * bh + y1)), 0), H)
            gh = min(max(int(math.floor(ph * G / P)), 0), G - 1)
            for pw in range(P):
                ws = min(max(int(math.floor(pw * bw + x1)), 0), W)
                we = min(max(int(math.ceil((pw + 1) * bw + x1)), 0), W)
                gw = min(max(int(math.floor(pw * G / P)), 0), G - 1)
                if he <= hs or we <= ws:
                    continue
                chan = (ctop * G + gh) * G + gw
                out[n, :, ph, pw] = data[b, chan, hs:he, ws:we].float().mean((1, 2)).to(data.dtype)
    return out


def _bilinear_at(plane, h, w):
    """plane: (K, H, W); bilinear value at the (already clamped) real position (h, w)."""
    H, W = plane.shape[-2:]
    h0, w0 = int(math.floor(h)), int(math.floor(w))
    h1, w1 = min(h0 + 1, H - 1), min(w0 + 1, W - 1)
    dh, dw = h - h0, w - w0
    return (plane[:, h0, w0] * (1 - dh) * (1 - dw) + plane[:, h0, w1] * (1 - dh) * dw +
            plane[:, h1, w0] * dh * (1 - dw) + plane[:, h1, w1] * dh * dw)


@register('_contrib_DeformablePSROIPooling', 'DeformablePSROIPooling', inputs=('data', 'rois', 'trans'),
          defaults={'spatial_scale': 1.0, 'output_dim': 1, 'group_size': 1, 'pooled_size': 1, 'part_size': 0,
                    'sample_per_part': 1, 'trans_std': 0.0, 'no_trans': False})
def deformable_psroi_pooling(data, rois, trans=None, spatial_scale=1.0, output_dim=1, group_size=1, pooled_size=1,
                             part_size=0, sample_per_part=1, trans_std=0.0, no_trans=False):
    """Position-sensitive ROI pooling whose bins are shifted by learned normalised offsets and sampled bilinearly
    (deformable_psroi_pooling.cu:45-140)."""
    P, G, S = int(pooled_size), int(group_size), int(sample_per_part)
    part = int(part_size) or P
    no_trans = bool(no_trans) or trans is None
    N, C, H, W = data.shape
    D = int(output_dim)
    ncls = 1 if no_trans else trans.shape[1] // 2
    per_cls = D if no_trans else D // ncls
    x = data.float()
    out = x.new_zeros((rois.shape[0], D, P, P))
    r_cpu = rois.detach().float().cpu()
    t_cpu = None if no_trans else trans.detach().float().cpu()
    ctop = torch.arange(D, device=data.device)
    cls_of = (ctop // per_cls).cpu()
    for n in range(rois.shape[0]):
        b = int(r_cpu[n, 0])
        x1 = round(float(r_cpu[n, 1])) * spatial_scale - 0.5
        y1 = round(float(r_cpu[n, 2])) * spatial_scale - 0.5
        x2 = (round(float(r_cpu[n, 3])) + 1.0) * spatial_scale - 0.5
        y2 = (round(float(r_cpu[n, 4])) + 1.0) * spatial_scale - 0.5
        rw, rh = max(x2 - x1, 0.1), max(y2 - y1, 0.1)
        bh, bw = rh / P, rw / P
        sh, sw = bh / S, bw / S
        for ph in range(P):
            gh = min(max(int(math.floor(ph * G / P)), 0), G - 1)
            p_h = int(math.floor(ph / P * part))
            for pw in range(P):
                gw = min(max(int(math.floor(pw * G / P)), 0), G - 1)
                p_w = int(math.floor(pw / P * part))
                chan = (ctop * G + gh) * G + gw
                for cls in range(ncls):
                    sel = (cls_of == cls).nonzero().reshape(-1).to(data.device)
                    if sel.numel() == 0:
                        continue
                    tx = 0.0 if no_trans else float(t_cpu[n, cls * 2, p_h, p_w]) * trans_std
                    ty = 0.0 if no_trans else float(t_cpu[n, cls * 2 + 1, p_h, p_w]) * trans_std
                    ws = pw * bw + x1 + tx * rw
                    hs = ph * bh + y1 + ty * rh
                    total, cnt = 0.0, 0
                    for ih in range(S):
                        for iw in range(S):
                            w_, h_ = ws + iw * sw, hs + ih * sh
                            if w_ < -0.5 or w_ > W - 0.5 or h_ < -0.5 or h_ > H - 0.5:
                                continue
                            w_, h_ = min(max(w_, 0.0), W - 1.0), min(max(h_, 0.0), H - 1.0)
                            total = total + _bilinear_at(x[b, chan[sel]], h_, w_)
                            cnt += 1
                    if cnt:
                        out[n, sel, ph, pw] = total / cnt
    return out.to(data.dtype)


@register('_contrib_DeformableConvolution', 'DeformableConvolution', inputs=('data', 'offset', 'weight', 'bias'),
          defaults={'kernel': (), 'stride': (), 'dilate': (), 'pad': (), 'num_filter': 0, 'num_group': 1,
                    'num_deformable_group': 1, 'workspace': 1024, 'no_bias': False, 'layout': None})
def deformable_convolution(data, offset, weight, bias=None, kernel=(), stride=(), dilate=(), pad=(), num_filter=0,
                           num_group=1, num_deformable_group=1, workspace=1024, no_bias=False, layout=None):
    """Convolution whose sampling grid is displaced by per-position (dy, dx) offsets, bilinear sampling
    (deformable_im2col.cuh + GEMM in the reference; the library's deformable convolution here)."""
    from torchvision.ops import deform_conv2d
    stride = tuple(stride) or (1, 1)
    dilate = tuple(dilate) or (1, 1)
    pad = tuple(pad) or (0, 0)
    b = None if no_bias else bias
    return deform_conv2d(data, offset.to(data.dtype), weight, b, stride, pad, dilate)


@register('_contrib_ModulatedDeformableConvolution', 'ModulatedDeformableConvolution',
          inputs=('data', 'offset', 'mask', 'weight', 'bias'),
          defaults={'kernel': (), 'stride': (), 'dilate': (), 'pad': (), 'num_filter': 0, 'num_group': 1,
                    'num_deformable_group': 1, 'workspace': 1024, 'no_bias': False, 'im2col_step': 64, 'layout': None})
def modulated_deformable_convolution(data, offset, mask, weight, bias=None, kernel=(), stride=(), dilate=(), pad=(),
                                     num_filter=0, num_group=1, num_deformable_group=1, workspace=1024, no_bias=False,
                                     im2col_step=64, layout=None):
    """Deformable convolution v2: every sampled value is additionally scaled by a learned mask
    (modulated_deformable_im2col.cuh)."""
    from torchvision.ops import deform_conv2d
    stride = tuple(stride) or (1, 1)
    dilate = tuple(dilate) or (1, 1)
    pad = tuple(pad) or (0, 0)
    b = None if no_bias else bias
    return deform_conv2d(data, offset.to(data.dtype), weight, b, stride, pad, dilate, mask.to(data.dtype))


@register('_contrib_mrcnn_mask_target', 'mrcnn_mask_target', inputs=('rois', 'gt_masks', 'matches', 'cls_targets'), nout=2,
          defaults={'num_rois': 0, 'num_classes': 0, 'mask_size': (14, 14), 'sample_ratio': 2, 'aligned': False})
def mrcnn_mask_target(rois, gt_masks, matches, cls_targets, num_rois=0, num_classes=0, mask_size=(14, 14), sample_ratio=2,
                      aligned=False):
    """Mask R-CNN training targets: the matched ground-truth mask of every ROI resampled to `mask_size` with ROIAlign,
    repeated over classes, and a one-hot class weight of the same shape (mrcnn_mask_target.cu)."""
    from torchvision.ops import roi_align as tv_roi_align
    B, N = rois.shape[0], rois.shape[1]
    C = int(num_classes)
    ms = tuple(mask_size) if not isinstance(mask_size, int) else (mask_size, mask_size)
    targets = []
    for b in range(B):
        m = gt_masks[b].float()[matches[b].long()][:, None]                      # (N, 1, H, W)
        boxes = torch.cat([torch.arange(N, device=rois.device, dtype=torch.float32)[:, None], rois[b].float()], 1)
        t = tv_roi_align(m, boxes, ms, 1.0, int(sample_ratio), bool(aligned))    # (N, 1, ms, ms)
        targets.append(t[:, 0])
    t = torch.stack(targets, 0)[:, :, None].expand(B, N, C, ms[0], ms[1]).contiguous()
    cls = (cls_targets.long()[:, :, None] == torch.arange(C, device=rois.device)[None, None, :])
    w = cls[:, :, :, None, None].expand(B, N, C, ms[0], ms[1]).to(t.dtype).contiguous()
    return t.to(gt_masks.dtype), w.to(gt_masks.dtype)

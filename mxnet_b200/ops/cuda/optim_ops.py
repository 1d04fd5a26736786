"""Multi-tensor optimizer / reduction launches (``optim.cu``)."""
import ctypes as C

import torch

from . import lib, ptr, stream_ptr, count_launch, check
from ._util import DT, require


def _parr(tensors):
    return (C.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def multi_sgd(ws, gs, moms, w32, lrs, wds, momentum, rescale, clip):
    L = lib()
    cap = L.mxb_max_tensors()
    dtype = ws[0].dtype
    for i in range(0, len(ws), cap):
        sl = slice(i, i + cap)
        w, g = ws[sl], gs[sl]
        n = len(w)
        dev = w[0].device
        for j in range(n):
            require(w[j], 'weight', dtype=dtype, device=dev)
            require(g[j], 'grad', numel=w[j].numel(), dtype=dtype, device=dev)
            if moms is not None:
                require(moms[i + j], 'mom', numel=w[j].numel(), dtype=torch.float32, device=dev)
            if w32 is not None:
                require(w32[i + j], 'weight32', numel=w[j].numel(), dtype=torch.float32, device=dev)
        m = _parr(moms[sl]) if moms is not None else None
        mp = _parr(w32[sl]) if w32 is not None else None
        check(L.mxb_multi_sgd(DT[dtype], n, _parr(w), _parr(g), m, mp, (C.c_float * n)(*lrs[sl]), (C.c_float * n)(*wds[sl]),
                              (C.c_int64 * n)(*[t.numel() for t in w]), float(momentum), float(rescale),
                              float(-1.0 if clip is None else clip), stream_ptr(w[0].device)), 'multi_sgd')
        count_launch(1)


def multi_adam(ws, gs, means, vars_, w32, lrs, wds, etas, beta1, beta2, eps, clip, rescale, decoupled):
    """Adam (decoupled=False) or AdamW over lists of tensors; `rescale` is a float or a one-element fp32 device tensor
    (a zero or non-finite value skips the update on the device, without a host synchronisation)."""
    L = lib()
    cap = L.mxb_max_tensors()
    dtype = ws[0].dtype
    rs_ptr, rs_host = (ptr(rescale), 1.0) if isinstance(rescale, torch.Tensor) else (None, float(rescale))
    if isinstance(rescale, torch.Tensor):
        require(rescale, 'rescale_grad', numel=1, dtype=torch.float32, device=ws[0].device)
    for i in range(0, len(ws), cap):
        sl = slice(i, i + cap)
        w, g = ws[sl], gs[sl]
        n = len(w)
        dev = w[0].device
        for j in range(n):
            require(w[j], 'weight', dtype=dtype, device=dev)
            require(g[j], 'grad', numel=w[j].numel(), dtype=dtype, device=dev)
            require(means[i + j], 'mean', numel=w[j].numel(), dtype=torch.float32, device=dev)
            require(vars_[i + j], 'var', numel=w[j].numel(), dtype=torch.float32, device=dev)
            if w32 is not None:
                require(w32[i + j], 'weight32', numel=w[j].numel(), dtype=torch.float32, device=dev)
        mp = _parr(w32[sl]) if w32 is not None else None
        et = (C.c_float * n)(*etas[sl]) if etas is not None else None
        check(L.mxb_multi_adam(DT[dtype], n, _parr(w), _parr(g), _parr(means[sl]), _parr(vars_[sl]), mp,
                               (C.c_float * n)(*lrs[sl]), (C.c_float * n)(*wds[sl]), et,
                               (C.c_int64 * n)(*[t.numel() for t in w]), float(beta1), float(beta2), float(eps),
                               float(-1.0 if clip is None else clip), rs_ptr, rs_host, 1 if decoupled else 0,
                               stream_ptr(dev)), 'multi_adam')
        count_launch(1)


def multi_all_finite(tensors):
    L = lib()
    cap = L.mxb_max_tensors()
    out = torch.empty(1, dtype=torch.float32, device=tensors[0].device)
    for i in range(0, len(tensors), cap):
        ts = [t if t.is_contiguous() else t.contiguous() for t in tensors[i:i + cap]]
        n = len(ts)
        check(L.mxb_multi_all_finite(n, _parr(ts), (C.c_int64 * n)(*[t.numel() for t in ts]),
                                     (C.c_int * n)(*[DT[t.dtype] for t in ts]), ptr(out), 1 if i == 0 else 0,
                                     stream_ptr(out.device)), 'multi_all_finite')
        count_launch(2 if i == 0 else 1)
    return out


def multi_sum_sq(tensors):
    L = lib()
    cap = L.mxb_max_tensors()
    out = torch.empty(len(tensors), dtype=torch.float32, device=tensors[0].device)
    for i in range(0, len(tensors), cap):
        ts = [t if t.is_contiguous() else t.contiguous() for t in tensors[i:i + cap]]
        n = len(ts)
        sizes = (C.c_int64 * n)(*[t.numel() for t in ts])
        scratch = torch.empty(max(1, L.mxb_sum_sq_chunks(n, sizes)), dtype=torch.float32, device=out.device)
        check(L.mxb_multi_sum_sq(n, _parr(ts), sizes, (C.c_int * n)(*[DT[t.dtype] for t in ts]), ptr(scratch), ptr(out), i,
                                 stream_ptr(out.device)), 'multi_sum_sq')
        count_launch(2)
    return out


def multi_add_(dsts, srcs):
    """``dsts[i] += srcs[i]`` for lists of same-dtype contiguous CUDA tensors, 48 tensors per launch (the
    parameter-gradient accumulation that ends a captured backward pass: one launch per 48 parameters instead of one
    tensor-library launch per parameter)."""
    L = lib()
    cap = L.mxb_max_tensors()
    groups = {}
    for d, s in zip(dsts, srcs):
        if d.dtype != s.dtype or d.shape != s.shape or not d.is_contiguous() or not s.is_contiguous() or d.dtype not in DT:
            d.add_(s)                       # anything irregular keeps the tensor library's add
            continue
        groups.setdefault((d.device, d.dtype), []).append((d, s))
    for (dev, dtype), pairs in groups.items():
        for i in range(0, len(pairs), cap):
            part = pairs[i:i + cap]
            n = len(part)
            sizes = (C.c_int64 * n)(*[d.numel() for d, _ in part])
            check(L.mxb_multi_add_inplace(DT[dtype], n, _parr([d for d, _ in part]), _parr([s for _, s in part]), sizes,
                                          stream_ptr(dev)), 'multi_add_inplace')
            count_launch(1)

"""``mx.nd.save`` / ``mx.nd.load`` / ``load_frombuffer`` over the native ``.params`` container.

Reference: ``python/mxnet/ndarray/utils.py:149-271`` → ``MXNDArrayLegacySave`` /
``MXNDArrayLoad`` (``src/c_api/c_api.cc:2259-2348``), which sniffs zip (npz), ``.npy`` and the
legacy magic.  The byte layout is implemented natively in ``csrc/ndarray_io.cc``.
"""
from __future__ import annotations

import ctypes
import io
import zipfile

import numpy as _np
import torch

from .. import _state
from ..base import MXNetError, dtype_flag, flag_to_torch
from ..device import Device, current_device
from .ndarray import NDArray

__all__ = ['save', 'load', 'load_frombuffer', 'zeros_like_shape']


def zeros_like_shape(shape, dtype='float32', ctx=None):
    from .ndarray import zeros
    return zeros(shape, ctx=ctx, dtype=dtype)


def _rt():
    from ..csrc import runtime
    return runtime.lib()


def _host(t):
    t = t.detach()
    if t.is_cuda:
        t = t.cpu()
    return t.contiguous()


def _add_array(L, w, arr, np_shape):
    c_i64 = ctypes.c_int64
    stype = getattr(arr, '_stype', 'default')
    t = _host(arr._data)
    flag = dtype_flag(t.dtype)
    dev_type, dev_id = 1, 0     # arrays are written from host memory, like the reference's CPU copy
    raw = t.view(torch.uint8).reshape(-1) if t.numel() else torch.empty(0, dtype=torch.uint8)
    if t.dtype == torch.bool:
        raw = t.to(torch.uint8).reshape(-1)
    shape = (c_i64 * max(t.dim(), 1))(*t.shape)
    if stype == 'default':
        legacy_none = (not np_shape) and t.dim() == 0
        if legacy_none:
            # legacy semantics cannot express 0-d arrays: promote to shape (1,)
            shape = (c_i64 * 1)(1)
            L.mxb_ndwriter_add_dense(w, 0, shape, 1, dev_type, dev_id, flag, raw.data_ptr(), raw.numel(), 0)
        else:
            L.mxb_ndwriter_add_dense(w, 1 if np_shape else 0, shape, t.dim(), dev_type, dev_id, flag,
                                     raw.data_ptr(), raw.numel(), 0)
        return
    if stype == 'row_sparse':
        idx = _host(arr.indices._data).long()
        data = _host(arr.data._data)
        auxs = [idx]
    else:
        data = _host(arr.data._data)
        auxs = [_host(arr.indptr._data).long(), _host(arr.indices._data).long()]
    draw = data.view(torch.uint8).reshape(-1) if data.numel() else torch.empty(0, dtype=torch.uint8)
    sshape = (c_i64 * max(data.dim(), 1))(*data.shape)
    aux_ptrs = (ctypes.c_void_p * len(auxs))(*[a.data_ptr() for a in auxs])
    aux_len = (c_i64 * len(auxs))(*[a.numel() for a in auxs])
    L.mxb_ndwriter_add_sparse(w, 1 if stype == 'row_sparse' else 2, shape, t.dim(), sshape, data.dim(), dev_type,
                              dev_id, flag, draw.data_ptr(), draw.numel(), len(auxs), aux_ptrs, aux_len)


def _build_writer(data):
    L = _rt()
    if isinstance(data, NDArray):
        data = [data]
    names = None
    if isinstance(data, dict):
        names = list(data.keys())
        arrays = [data[k] for k in names]
    elif isinstance(data, (list, tuple)):
        arrays = list(data)
    else:
        raise ValueError('data needs to either be a NDArray, dict of str, NDArray pairs or a list of NDarrays.')
    for a in arrays:
        if not isinstance(a, NDArray):
            raise TypeError('save only accept dict str->NDArray or list of NDArray')
    np_shape = _state.state.np_shape
    w = L.mxb_ndwriter_create()
    for a in arrays:
        _add_array(L, w, a, np_shape and getattr(a, '_stype', 'default') == 'default')
    if names is not None:
        for n in names:
            b = n.encode('utf-8')
            L.mxb_ndwriter_add_name(w, b, len(b))
    return L, w


def _save_now(fname, data):
    L, w = _build_writer(data)
    try:
        rc = L.mxb_ndwriter_save(w, str(fname).encode())
    finally:
        L.mxb_ndwriter_free(w)
    if rc != 0:
        raise MXNetError('cannot write %s' % fname)


def save(fname, data):
    """Save arrays (list or ``{name: array}``) in the legacy binary container.

    The write runs as a task of the host engine that READS the arrays: it starts after every pending host task that
    writes one of them (an asynchronous load, a prefetch) and host tasks pushed later that write them wait for it; the
    call returns when the file is complete and raises what the writer raised (``MXNDArraySave`` waits on its arrays the
    same way, src/c_api/c_api.cc)."""
    from .. import engine
    arrays = [a for a in (data.values() if isinstance(data, dict) else
                          (data if isinstance(data, (list, tuple)) else [data])) if isinstance(a, NDArray)]
    if engine.in_task():
        return _save_now(fname, data)
    done = engine.native().new_var()
    engine.push(lambda: _save_now(fname, data), reads=arrays, writes=[done], name='ndarray_save')
    engine.native().wait_for_var(done)


def save_tobuffer(data):
    L, w = _build_writer(data)
    try:
        n = L.mxb_ndwriter_size(w)
        buf = ctypes.create_string_buffer(n)
        L.mxb_ndwriter_to_buffer(w, buf)
    finally:
        L.mxb_ndwriter_free(w)
    return buf.raw


def _tensor_from(ptr, nbytes, flag, shape):
    td = flag_to_torch(flag)
    if nbytes == 0:
        return torch.empty(tuple(shape), dtype=td)
    raw = (ctypes.c_ubyte * nbytes).from_address(ptr)
    a = _np.frombuffer(raw, dtype=_np.uint8).copy()
    t = torch.from_numpy(a)
    if td == torch.bool:
        return t.reshape(tuple(shape)).bool()
    return t.view(td).reshape(tuple(shape))


def _read_list(L, h, ctx, cls):
    err = L.mxb_ndlist_error(h)
    if err:
        raise MXNetError(err.decode())
    n = L.mxb_ndlist_count(h)
    arrays = []
    c_i64 = ctypes.c_int64
    for i in range(n):
        meta = (c_i64 * 8)()
        L.mxb_ndlist_meta(h, i, meta)
        none, stype, ndim, _, _, flag, n_aux, sndim = list(meta)
        if none:
            arrays.append(None)
            continue
        shape = (c_i64 * max(ndim, 1))()
        L.mxb_ndlist_shape(h, i, shape)
        shape = list(shape)[:ndim]
        nbytes = ctypes.c_uint64(0)
        ptr = L.mxb_ndlist_data(h, i, ctypes.byref(nbytes))
        if stype == 0:
            t = _tensor_from(ptr, nbytes.value, flag, shape)
            arrays.append(cls._from_tensor(t.to(ctx.torch_device), ctx))
            continue
        sshape = (c_i64 * max(sndim, 1))()
        L.mxb_ndlist_storage_shape(h, i, sshape)
        data = _tensor_from(ptr, nbytes.value, flag, list(sshape)[:sndim])
        auxs = []
        for k in range(n_aux):
            m2 = (c_i64 * 2)()
            ashape = (c_i64 * 8)()
            ab = ctypes.c_uint64(0)
            ap = L.mxb_ndlist_aux(h, i, k, m2, ashape, ctypes.byref(ab))
            auxs.append(_tensor_from(ap, ab.value, m2[0], list(ashape)[:m2[1]]).long())
        from . import sparse
        if stype == 1:
            arrays.append(sparse.row_sparse_array((data.numpy(), auxs[0].numpy()), shape=tuple(shape), ctx=ctx,
                                                  dtype=data.numpy().dtype))
        else:
            arrays.append(sparse.csr_matrix((data.numpy(), auxs[1].numpy(), auxs[0].numpy()), shape=tuple(shape),
                                            ctx=ctx, dtype=data.numpy().dtype))
    k = L.mxb_ndlist_num_names(h)
    if k == 0:
        return arrays
    out = {}
    for i in range(k):
        ln = c_i64(0)
        p = L.mxb_ndlist_name(h, i, ctypes.byref(ln))
        out[ctypes.string_at(p, ln.value).decode('utf-8')] = arrays[i]
    return out


def _load_npz(src, ctx, cls):
    z = _np.load(src, allow_pickle=False)
    if isinstance(z, _np.ndarray):                 # a .npy file holds one array (Fortran order becomes C order)
        return cls(_np.ascontiguousarray(z), ctx=ctx, dtype=z.dtype if z.dtype != _np.float64 else None)
    out, sparse_parts = {}, {}
    for k in z.files:
        if '/' in k and k.rsplit('/', 1)[1] in ('data', 'indices', 'indptr', 'shape', 'format'):
            base, part = k.rsplit('/', 1)
            sparse_parts.setdefault(base, {})[part] = z[k]
        else:
            a = z[k]
            out[k] = cls(a, ctx=ctx, dtype=a.dtype)
    from . import sparse
    for base, p in sparse_parts.items():
        fmt = bytes(p['format']).decode() if p['format'].dtype.kind in 'SU' or p['format'].dtype == _np.uint8 \
            else str(p['format'])
        shape = tuple(int(s) for s in p['shape'])
        if 'csr' in fmt:
            out[base] = sparse.csr_matrix((p['data'], p['indices'], p['indptr']), shape=shape, ctx=ctx, dtype=p['data'].dtype)
        else:
            out[base] = sparse.row_sparse_array((p['data'], p['indices']), shape=shape, ctx=ctx, dtype=p['data'].dtype)
    return out            # a dict in every case: positional members of savez keep numpy's names arr_0, arr_1, ...


def _sniff(head):
    if head[:4] == b'PK\x03\x04' or head[:4] == b'PK\x05\x06':
        return 'npz'
    if head[:6] == b'\x93NUMPY':
        return 'npy'
    return 'legacy'


def load(fname, ctx=None, cls=None):
    """Load arrays saved by :func:`save`, ``npx.save`` / ``npx.savez`` or the reference."""
    ctx = ctx or Device('cpu', 0)
    cls = cls or NDArray
    with open(fname, 'rb') as f:
        kind = _sniff(f.read(8))
    if kind in ('npz', 'npy'):
        return _load_npz(fname, ctx, cls)
    L = _rt()
    h = L.mxb_ndlist_load_file(str(fname).encode())
    try:
        return _read_list(L, h, ctx, cls)
    finally:
        L.mxb_ndlist_free(h)


def load_frombuffer(buf, ctx=None, cls=None):
    ctx = ctx or Device('cpu', 0)
    cls = cls or NDArray
    if not isinstance(buf, (bytes, bytearray)):
        raise TypeError('buf required to be a string or bytes')
    kind = _sniff(bytes(buf[:8]))
    if kind in ('npz', 'npy'):
        return _load_npz(io.BytesIO(bytes(buf)), ctx, cls)
    L = _rt()
    b = bytes(buf)
    h = L.mxb_ndlist_load_buffer(b, len(b))
    try:
        return _read_list(L, h, ctx, cls)
    finally:
        L.mxb_ndlist_free(h)

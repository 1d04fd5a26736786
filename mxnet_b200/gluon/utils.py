"""Gluon utilities (``python/mxnet/gluon/utils.py``): batch splitting, global-norm clipping, downloads."""
import hashlib
import math
import os
import warnings

import numpy as np
import torch

from ..ndarray.ndarray import NDArray
from ..util import is_np_array

__all__ = ['split_data', 'split_and_load', 'clip_global_norm', 'check_sha1', 'download', 'replace_file',
           'shape_is_known', 'split_rnn_params']


def split_data(data, num_slice, batch_axis=0, even_split=True):
    size = data.shape[batch_axis]
    if even_split and size % num_slice != 0:
        raise ValueError("data with shape %s cannot be evenly split into %d slices along axis %d. Use a batch size "
                         "that's multiple of %d or set even_split=False to allow uneven partitioning of data." % (
                             str(data.shape), num_slice, batch_axis, num_slice))
    # uneven partitions follow numpy.array_split: the first (size % num_slice) slices get one element more
    n_each, extras = divmod(size, num_slice)
    sizes = extras * [n_each + 1] + (num_slice - extras) * [n_each]
    slices, lo = [], 0
    for n in sizes:
        idx = [slice(None)] * data.ndim
        idx[batch_axis] = slice(lo, lo + n)
        slices.append(data[tuple(idx)])
        lo += n
    return slices


def split_and_load(data, ctx_list=None, batch_axis=0, even_split=True, device_list=None):
    """Split a batch along ``batch_axis`` and place one slice on every device (``utils.py:86``)."""
    ctx_list = ctx_list if ctx_list is not None else device_list
    if not isinstance(data, NDArray):
        if is_np_array():
            from .. import numpy as mnp
            data = mnp.array(data, ctx=ctx_list[0])
        else:
            from .. import ndarray as nd
            data = nd.array(data, ctx=ctx_list[0])
    if len(ctx_list) == 1:
        return [data.as_in_context(ctx_list[0])]
    slices = split_data(data, len(ctx_list), batch_axis, even_split)
    return [i.as_in_context(ctx) for i, ctx in zip(slices, ctx_list)]


def clip_global_norm(arrays, max_norm, check_isfinite=True):
    """Rescale arrays so that the 2-norm of their concatenation is at most ``max_norm``
    (``utils.py:116-167``): ``scale = min(1, max_norm / (total + 1e-8))``."""
    assert len(arrays) > 0
    from ..ops import registry as _reg
    dev = arrays[0]._data.device
    sq = _reg.get('multi_sum_sq').fn(*[a._data for a in arrays], num_arrays=len(arrays))
    total = torch.sqrt(sq.float().to(dev).sum())
    scale = torch.clamp(max_norm / (total + 1e-8), max=1.0)
    if check_isfinite:
        total_f = float(total.item())
        if not math.isfinite(total_f):
            warnings.warn(UserWarning('nan or inf is detected. Clipping results will be undefined.'), stacklevel=2)
    with torch.no_grad():
        torch._foreach_mul_([a._data for a in arrays], [scale.to(a._data.device, a._data.dtype) for a in arrays]) \
            if len({a._data.device for a in arrays}) > 1 else \
            [a._data.mul_(scale.to(a._data.dtype)) for a in arrays]
    if check_isfinite:
        return total_f
    return arrays[0].__class__._from_tensor(total.reshape(1) if not is_np_array() else total)


def check_sha1(filename, sha1_hash):
    sha1 = hashlib.sha1()
    with open(filename, 'rb') as f:
        while True:
            data = f.read(1048576)
            if not data:
                break
            sha1.update(data)
    return sha1.hexdigest() == sha1_hash


def replace_file(src, dst):
    os.replace(src, dst)


def download(url, path=None, overwrite=False, sha1_hash=None, retries=5, verify_ssl=True):
    """Download a file.  Files already present (and matching ``sha1_hash``) are used as they are."""
    if path is None:
        fname = url.split('/')[-1]
    else:
        path = os.path.expanduser(path)
        fname = os.path.join(path, url.split('/')[-1]) if os.path.isdir(path) else path
    if not overwrite and os.path.exists(fname) and (not sha1_hash or check_sha1(fname, sha1_hash)):
        return fname
    import requests
    dirname = os.path.dirname(os.path.abspath(os.path.expanduser(fname)))
    os.makedirs(dirname, exist_ok=True)
    last = None
    for _ in range(max(retries, 0) + 1):
        try:
            r = requests.get(url, stream=True, verify=verify_ssl, timeout=30)
            if r.status_code != 200:
                raise RuntimeError('Failed downloading url {}'.format(url))
            tmp = fname + '.part'
            with open(tmp, 'wb') as f:
                for chunk in r.iter_content(chunk_size=1048576):
                    if chunk:
                        f.write(chunk)
            os.replace(tmp, fname)
            if sha1_hash and not check_sha1(fname, sha1_hash):
                raise UserWarning('File {} is downloaded but the content hash does not match.'.format(fname))
            return fname
        except Exception as e:  # pylint: disable=broad-except
            last = e
    raise last


def shape_is_known(shape):
    if shape is None:
        return False
    from .. import _state
    unknown = -1 if _state.state.np_shape else 0
    if len(shape) == 0:
        return unknown == -1
    return all(d != unknown and d >= 0 for d in shape)


def split_rnn_params(param, mode, num_layers, input_size, hidden_size, bidirectional=False, projection_size=None):
    """Split the flat fused-RNN parameter vector into named per-gate-block arrays (``utils.py:509``)."""
    from ..ops.nn import rnn_unpack
    pieces = rnn_unpack(param._data, mode, num_layers, input_size, hidden_size, bidirectional, projection_size)
    d = 2 if bidirectional else 1
    out = {}
    for idx, (w_ih, w_hh, w_hr, b_ih, b_hh) in enumerate(pieces):
        layer, direction = idx // d, 'lr'[idx % d]
        pre = '%s%d_' % (direction, layer)
        cls = param.__class__
        out[pre + 'i2h_weight'] = cls._from_tensor(w_ih, param._ctx)
        out[pre + 'h2h_weight'] = cls._from_tensor(w_hh, param._ctx)
        if w_hr is not None:
            out[pre + 'h2r_weight'] = cls._from_tensor(w_hr, param._ctx)
        out[pre + 'i2h_bias'] = cls._from_tensor(b_ih, param._ctx)
        out[pre + 'h2h_bias'] = cls._from_tensor(b_hh, param._ctx)
    return out


class HookHandle(object):
    """A handle that can attach a hook to a dict of hooks and detach it again (also usable in a ``with`` block)."""

    def __init__(self):
        self._hooks_dict_ref, self._id = None, None

    def attach(self, hooks_dict, hook):
        import weakref
        assert not self._hooks_dict_ref, 'The same handle cannot be attached twice.'
        self._id = id(hook)
        hooks_dict[self._id] = hook
        self._hooks_dict_ref = weakref.ref(hooks_dict) if not isinstance(hooks_dict, dict) else (lambda d=hooks_dict: d)

    def detach(self):
        hooks = self._hooks_dict_ref() if self._hooks_dict_ref else None
        if hooks is not None and self._id in hooks:
            del hooks[self._id]

    def __enter__(self):
        return self

    def __exit__(self, ptype, value, trace):
        self.detach()

"""``mx.npx``: operators beyond NumPy's API with NumPy-semantics arrays
(``python/mxnet/numpy_extension/_op.py``) plus the mode switches and ``save/savez/load``."""
import numpy as _onp

from ..ops import registry as _reg
from ..util import set_np, reset_np, is_np_shape, is_np_array, is_np_default_dtype, use_np, use_np_shape, use_np_array, \
    np_shape, np_array   # noqa: F401
from ..device import cpu, gpu, cpu_pinned, num_gpus, current_device, gpu_memory_info, Device   # noqa: F401
from ..ops.random import seed   # noqa: F401
from ..ndarray.ndarray import waitall, NDArray   # noqa: F401
from ..ndarray import contrib_ext as _cf
from . import random, image   # noqa: F401

current_context = current_device


def _np_frontend(name):
    return _reg.make_frontend(_reg.get(name), 'np')


for _name in _reg.list_ops():
    if _name.startswith('_npx_'):
        globals()[_name[5:].lstrip('_')] = _np_frontend(_name)

for _pub, _opn in [('relu', 'relu'), ('sigmoid', 'sigmoid'), ('log_sigmoid', 'log_sigmoid'), ('mish', 'mish'),
                   ('gamma', 'gamma'), ('gammaln', 'gammaln'), ('digamma', 'digamma'), ('erf', 'erf'), ('erfinv', 'erfinv'),
                   ('smooth_l1', 'smooth_l1'), ('gather_nd', 'gather_nd'), ('scatter_nd', 'scatter_nd'),
                   ('reshape_like', 'reshape_like'), ('broadcast_like', 'broadcast_like'), ('slice', 'slice'),
                   ('slice_axis', 'slice_axis'), ('slice_like', 'slice_like'), ('batch_flatten', 'Flatten'),
                   ('cast', '_npi_cast'), ('shape_array', 'shape_array'), ('sequence_last', 'SequenceLast'),
                   ('sequence_reverse', 'SequenceReverse'), ('roi_pooling', 'ROIPooling'), ('softmin', 'softmin'),
                   ('multibox_prior', '_contrib_MultiBoxPrior'), ('multibox_target', '_contrib_MultiBoxTarget'),
                   ('multibox_detection', '_contrib_MultiBoxDetection'), ('box_nms', '_contrib_box_nms'),
                   ('box_iou', '_contrib_box_iou'), ('roi_align', '_contrib_ROIAlign'), ('bilinear_resize2d', '_contrib_BilinearResize2D'),
                   ('interleaved_matmul_selfatt_qk', '_contrib_interleaved_matmul_selfatt_qk'),
                   ('interleaved_matmul_selfatt_valatt', '_contrib_interleaved_matmul_selfatt_valatt'),
                   ('interleaved_matmul_encdec_qk', '_contrib_interleaved_matmul_encdec_qk'),
                   ('interleaved_matmul_encdec_valatt', '_contrib_interleaved_matmul_encdec_valatt'),
                   ('div_sqrt_dim', '_contrib_div_sqrt_dim'), ('sldwin_atten_score', '_contrib_sldwin_atten_score'),
                   ('sldwin_atten_context', '_contrib_sldwin_atten_context'), ('sldwin_atten_mask_like', '_contrib_sldwin_atten_mask_like'),
                   ('softmax_ce_loss', '_npx_softmax_ce_loss'), ('norm', 'norm'), ('amp_cast', 'amp_cast'),
                   ('amp_multicast', 'amp_multicast'), ('all_finite', 'all_finite'), ('multi_all_finite', 'multi_all_finite'),
                   ('multi_sum_sq', 'multi_sum_sq'), ('quantize', '_contrib_quantize'), ('dequantize', '_contrib_dequantize'),
                   ('index_add', '_npx_index_add'), ('index_update', '_npx_index_update'), ('depth_to_space', 'depth_to_space'),
                   ('space_to_depth', 'space_to_depth')]:
    if _pub not in globals():
        globals()[_pub] = _np_frontend(_opn)

foreach, while_loop, cond = _cf.foreach, _cf.while_loop, _cf.cond


def nonzero(a):
    return _reg.invoke('_npi_nonzero', [a], {}, kind='np')


def save(file, arr):
    """Save arrays to ``.npy``/``.npz`` (np mode) – ``MXNDArraySave`` → ``npz::save_array``
    (``src/serialization/cnpy.cc:470-505``): uncompressed zip of ``.npy`` members; sparse arrays as
    ``name/data``, ``name/indices``, ``name/indptr``, ``name/shape``, ``name/format``."""
    if isinstance(arr, NDArray):
        with open(file, 'wb') as f:
            _onp.save(f, arr.asnumpy(), allow_pickle=False)
        return
    savez(file, *arr) if isinstance(arr, (list, tuple)) else savez(file, **arr)


def savez(file, *args, **kwds):
    members = {}
    for i, a in enumerate(args):
        members['arr_%d' % i] = a
    members.update(kwds)
    flat = {}
    for k, a in members.items():
        st = getattr(a, '_stype', 'default')
        if st == 'default':
            flat[k] = a.asnumpy() if isinstance(a, NDArray) else _onp.asarray(a)
        else:
            flat[k + '/data'] = a.data.asnumpy()
            flat[k + '/indices'] = a.indices.asnumpy()
            if st == 'csr':
                flat[k + '/indptr'] = a.indptr.asnumpy()
            flat[k + '/shape'] = _onp.asarray(a.shape, dtype=_onp.int64)
            flat[k + '/format'] = _onp.asarray('csr' if st == 'csr' else 'row_sparse')
    with open(file, 'wb') as f:
        _onp.savez(f, **flat)


def load(file):
    from ..ndarray.utils import load as _load
    from ..numpy.multiarray import ndarray
    return _load(file, cls=ndarray)


# ---- utilities of python/mxnet/numpy_extension/utils.py -----------------------------------------------------------------
from ..util import set_np_default_dtype, get_cuda_compute_capability   # noqa: E402,F401
from ..ndarray import contrib_ext as control_flow   # noqa: E402,F401  (foreach / while_loop / cond)


def from_dlpack(dlpack):
    """An ``mx.np.ndarray`` that shares memory with a DLPack capsule (or any object with ``__dlpack__``)."""
    import torch
    from ..numpy.multiarray import ndarray
    return ndarray._from_tensor(torch.utils.dlpack.from_dlpack(dlpack))


def from_numpy(array, zero_copy=True):
    """An ``mx.np.ndarray`` from a ``numpy.ndarray``; with ``zero_copy`` the two share memory (the array must be C-contiguous)."""
    import torch
    from ..numpy.multiarray import ndarray
    if zero_copy and not array.flags['C_CONTIGUOUS']:
        raise ValueError('Only c-contiguous arrays are supported for zero-copy')
    return ndarray._from_tensor(torch.from_numpy(array if zero_copy else array.copy()))


def to_dlpack_for_read(data):
    """DLPack capsule of the array once every pending write has finished."""
    return data.to_dlpack_for_read()


def to_dlpack_for_write(data):
    """DLPack capsule of the array once every pending read and write has finished."""
    return data.to_dlpack_for_write()

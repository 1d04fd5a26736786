"""``mx.contrib.tensorrt`` (``python/mxnet/contrib/tensorrt.py``).  The TensorRT sub-graph back end is a third-party
integration of the reference that this build does not carry: inference graphs run through the in-tree kernels and CUDA
graphs instead.  The functions exist so that code probing for the back end gets a clear answer."""
from ..base import MXNetError

_use_fp16 = True


def set_use_fp16(status):
    """Remember the requested precision (read back by ``get_use_fp16``); it has no effect without the back end."""
    global _use_fp16
    _use_fp16 = bool(status)


def get_use_fp16():
    return _use_fp16


def init_tensorrt_params(sym, arg_params, aux_params):
    raise MXNetError('the TensorRT back end is not part of this build; run the symbol directly '
                     '(hybridize(static_alloc=True, static_shape=True) captures CUDA graphs)')

"""Loader of the ahead-of-time compiled sm_100a kernel library (``libmxb200_kernels.so``).

The kernels are plain ``extern "C"`` launchers taking raw device pointers and a stream, built
in-tree by ``build.py`` (``nvcc -gencode arch=compute_100a,code=sm_100a``) and bound with ctypes.
On a machine with a GPU a missing library is an error, not a silent fallback: the framework's hot
paths are these kernels.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, 'libmxb200_kernels.so')
_lib = None
_checked = False


def lib():
    """The loaded kernel library (raises if it is missing or fails to load)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError('sm_100a kernel library not built: run `python -m mxnet_b200.ops.cuda.build` '
                               '(expected %s)' % LIB_PATH)
        _lib = ctypes.CDLL(LIB_PATH)
        from . import _signatures
        _signatures.declare(_lib)
    return _lib


def available():
    """True when CUDA tensors should be routed to the hand-written kernels."""
    global _checked
    if not torch.cuda.is_available():
        return False
    if not _checked:
        lib()           # fail loudly on a GPU box without the library
        _checked = True
    return True


def stream_ptr(device=None):
    """The current stream of ``device`` as a raw handle for a kernel launch that follows immediately.  The launchers
    of the kernel library start their kernels on the CURRENT device, so this also makes ``device`` current when it is
    not (a process that drives several GPUs runs operators on arrays of any of them; the tensor library's own
    operators switch devices by themselves, the raw launchers cannot)."""
    if device is not None:
        index = device.index if isinstance(device, torch.device) else int(device)
        if index is not None and index != torch.cuda.current_device():
            torch.cuda.set_device(index)
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


_launch_count = 0


def count_launch(n=1):
    """Counter of kernel launches issued through this library (reported by the benchmark)."""
    global _launch_count
    _launch_count += n


def launches():
    return _launch_count


def check(code, what):
    if code != 0:
        raise RuntimeError('%s failed with CUDA error %d' % (what, code))

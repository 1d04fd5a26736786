"""Run-time compiled CUDA modules (``python/mxnet/rtc.py`` ``CudaModule``/``CudaKernel`` over NVRTC,
``src/common/rtc.cc``).  Source is compiled for the running device's architecture with NVRTC
(through the CUDA Python bindings) and launched on the current stream.
"""
import ctypes
import re

import numpy as np
import torch

from .base import MXNetError
from .ndarray.ndarray import NDArray

_DTYPE_CPP_TO_NP = {'float': np.float32, 'double': np.float64, '__half': np.float16, 'uint8_t': np.uint8,
                    'int': np.int32, 'int32_t': np.int32, 'int8_t': np.int8, 'char': np.int8, 'int64_t': np.int64}


def _include_dirs():
    """Directories holding the toolkit's device headers (``cuda_fp16.h`` and friends): NVRTC searches none by itself."""
    import os
    found = []
    roots = [os.environ.get('CUDA_HOME'), os.environ.get('CUDA_PATH'), '/usr/local/cuda']
    try:
        import nvidia.cuda_runtime as rt   # the pip wheel of the runtime ships the same headers
        roots.append(os.path.dirname(rt.__file__))
    except Exception:   # pylint: disable=broad-except
        pass
    for root in roots:
        inc = os.path.join(root, 'include') if root else None
        if inc and os.path.isfile(os.path.join(inc, 'cuda_fp16.h')) and inc not in found:
            found.append(inc)
    return found


class CudaModule(object):
    def __init__(self, source, options=(), exports=()):
        try:
            try:
                from cuda.bindings import nvrtc   # cuda-python >= 12.8
            except ImportError:
                from cuda import nvrtc
        except Exception as e:   # pylint: disable=broad-except
            raise MXNetError('NVRTC bindings are unavailable: %s' % e)
        self._nvrtc = nvrtc
        if not torch.cuda.is_available():
            raise MXNetError('CudaModule needs a GPU')
        major, minor = torch.cuda.get_device_capability()
        arch = 'sm_%d%d%s' % (major, minor, 'a' if major >= 9 else '')
        err, prog = nvrtc.nvrtcCreateProgram(source.encode(), b'mxb_rtc.cu', 0, [], [])
        opts = [('--gpu-architecture=' + arch).encode()] + [('--include-path=' + d).encode() for d in _include_dirs()]
        opts += [o.encode() for o in options]
        err, = nvrtc.nvrtcCompileProgram(prog, len(opts), opts)
        if int(err) != 0:
            _, n = nvrtc.nvrtcGetProgramLogSize(prog)
            log = b' ' * n
            nvrtc.nvrtcGetProgramLog(prog, log)
            raise MXNetError('NVRTC compilation failed:\n' + log.decode(errors='replace'))
        _, n = nvrtc.nvrtcGetCUBINSize(prog)
        cubin = b' ' * n
        nvrtc.nvrtcGetCUBIN(prog, cubin)
        try:
            from cuda.bindings import driver as cu
        except ImportError:
            from cuda import cuda as cu
        self._cu = cu
        torch.cuda.current_stream()   # make sure a context exists
        err, self._module = cu.cuModuleLoadData(cubin)
        if int(err) != 0:
            raise MXNetError('cuModuleLoadData failed: %s' % err)
        self._exports = list(exports)

    def get_kernel(self, name, signature):
        pattern = re.compile(r'^\s*(const)?\s*([\w_]+)\s*(\*)?\s*([\w_]+)?\s*$')
        args = []
        for arg in re.sub(r'\s+', ' ', signature).split(','):
            m = pattern.match(arg)
            if not m or m.groups()[1] == 'const':
                raise ValueError('Invalid function prototype "%s"' % arg)
            is_const, dtype, is_ptr, _ = m.groups()
            if dtype not in _DTYPE_CPP_TO_NP:
                raise TypeError('Unsupported kernel argument type %s' % arg)
            args.append((bool(is_ptr), bool(is_const), _DTYPE_CPP_TO_NP[dtype]))
        err, fn = self._cu.cuModuleGetFunction(self._module, name.encode())
        if int(err) != 0:
            raise MXNetError('kernel %s not found' % name)
        return CudaKernel(self._cu, fn, name, args)


class CudaKernel(object):
    def __init__(self, cu, fn, name, args):
        self._cu, self._fn, self._name, self._args = cu, fn, name, args

    def launch(self, args, ctx, grid_dims, block_dims, shared_mem=0):
        assert ctx.device_type == 'gpu', 'Cuda kernel can only be launched on GPU'
        assert len(args) == len(self._args)
        holders, ptrs = [], []
        for a, (is_ptr, _, dt) in zip(args, self._args):
            if is_ptr:
                assert isinstance(a, NDArray)
                holders.append(ctypes.c_void_p(a._data.data_ptr()))
            else:
                holders.append(np.array(a, dtype=dt))
        arr = (ctypes.c_void_p * len(holders))()
        for i, h in enumerate(holders):
            arr[i] = ctypes.addressof(h) if isinstance(h, ctypes.c_void_p) else h.ctypes.data
        stream = torch.cuda.current_stream(ctx.device_id).cuda_stream
        err, = self._cu.cuLaunchKernel(self._fn, *grid_dims, *block_dims, shared_mem, stream, ctypes.addressof(arr), 0)
        if int(err) != 0:
            raise MXNetError('launch of %s failed: %s' % (self._name, err))

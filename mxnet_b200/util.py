"""NumPy-semantics switches and small helpers (``python/mxnet/util.py``)."""
import functools
import os

from . import _state

__all__ = ['set_np', 'reset_np', 'is_np_shape', 'is_np_array', 'is_np_default_dtype', 'np_shape', 'np_array',
           'use_np', 'use_np_shape', 'use_np_array', 'set_np_shape', 'makedirs', 'get_gpu_count', 'get_gpu_memory',
           'getenv', 'setenv', 'default_array', 'get_cuda_compute_capability', 'set_module', 'wrap_ctx_to_device_func']


def makedirs(d):
    os.makedirs(d, exist_ok=True)


def get_gpu_count():
    from .device import num_gpus
    return num_gpus()


def get_gpu_memory(gpu_dev_id):
    from .device import gpu_memory_info
    return gpu_memory_info(gpu_dev_id)


def get_cuda_compute_capability(ctx):
    import torch
    major, minor = torch.cuda.get_device_capability(ctx.device_id)
    return major * 10 + minor


def getenv(name):
    return os.environ.get(name)


def setenv(name, value):
    from . import env
    env.set(name, value)


def set_np_shape(active):
    prev = _state.state.np_shape
    _state.state.np_shape = bool(active)
    return prev


def is_np_shape():
    return _state.state.np_shape


def is_np_array():
    return _state.state.np_array


def is_np_default_dtype():
    return _state.state.np_default_dtype


def set_np(shape=True, array=True, dtype=False):
    """Turn on NumPy semantics: zero-dim/zero-size shapes, ``mx.np.ndarray`` outputs, optional
    float64 default dtype (``python/mxnet/util.py`` ``set_np``)."""
    if not shape and array:
        raise ValueError('NumPy Shape semantics is required in using NumPy array semantics.')
    _state.state.np_shape = bool(shape)
    _state.state.np_array = bool(array)
    _state.state.np_default_dtype = bool(dtype)


def reset_np():
    set_np(shape=False, array=False, dtype=False)


class _NumpyScope(object):
    def __init__(self, field, active):
        self._field, self._active, self._prev = field, active, None

    def __enter__(self):
        self._prev = getattr(_state.state, self._field)
        setattr(_state.state, self._field, self._active)
        return self

    def __exit__(self, *a):
        setattr(_state.state, self._field, self._prev)


def np_shape(active=True):
    return _NumpyScope('np_shape', active)


def np_array(active=True):
    return _NumpyScope('np_array', active)


def _wrap_scope(fn_or_cls, scopes):
    if isinstance(fn_or_cls, type):
        for name, m in list(vars(fn_or_cls).items()):
            if callable(m) and not name.startswith('__') or name in ('__init__', '__call__'):
                if callable(m) and not isinstance(m, (staticmethod, classmethod, type)):
                    setattr(fn_or_cls, name, _wrap_scope(m, scopes))
        return fn_or_cls

    @functools.wraps(fn_or_cls)
    def wrapper(*args, **kwargs):
        saved = [(f, getattr(_state.state, f)) for f in scopes]
        for f in scopes:
            setattr(_state.state, f, True)
        try:
            return fn_or_cls(*args, **kwargs)
        finally:
            for f, v in saved:
                setattr(_state.state, f, v)
    return wrapper


def use_np_shape(func):
    return _wrap_scope(func, ['np_shape'])


def use_np_array(func):
    return _wrap_scope(func, ['np_array'])


def use_np(func):
    return _wrap_scope(func, ['np_shape', 'np_array'])


def default_array(source_array, ctx=None, dtype=None):
    if is_np_array():
        from . import numpy as _mnp
        return _mnp.array(source_array, ctx=ctx, dtype=dtype)
    from . import ndarray as _nd
    return _nd.array(source_array, ctx=ctx, dtype=dtype)


def set_module(module):
    def deco(f):
        if module is not None:
            f.__module__ = module
        return f
    return deco


def wrap_ctx_to_device_func(func):
    @functools.wraps(func)
    def wrapper(*args, **kwargs):
        if 'ctx' in kwargs and 'device' not in kwargs:
            kwargs['device'] = kwargs.pop('ctx')
        return func(*args, **kwargs)
    return wrapper

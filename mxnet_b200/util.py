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


# ---------------------------------------------------------------------------------------------------------
# decorators and switches of python/mxnet/util.py used by the NumPy front end and by run-time compilation
# ---------------------------------------------------------------------------------------------------------
_np_ufunc_default_kwargs = {'where': True, 'casting': 'same_kind', 'order': 'K', 'dtype': None, 'subok': True}


def np_ufunc_legal_option(key, value):
    """Whether ``key=value`` is a valid ufunc option at all (valid but non-default options are "not implemented",
    anything else is a type error)."""
    import numpy as _np
    if key == 'where':
        return True
    if key == 'casting':
        return value in ('no', 'equiv', 'safe', 'same_kind', 'unsafe')
    if key == 'order':
        return isinstance(value, str)
    if key == 'dtype':
        return value in (_np.int8, _np.uint8, _np.int32, _np.int64, _np.float16, _np.float32, _np.float64,
                         'int8', 'uint8', 'int32', 'int64', 'float16', 'float32', 'float64')
    if key == 'subok':
        return isinstance(value, bool)
    return False


def _check_ufunc_kwargs(func, kwargs):
    for key, value in kwargs.items():
        if key not in _np_ufunc_default_kwargs:
            raise TypeError("{} is an invalid keyword to function '{}'".format(key, func.__name__))
        if value != _np_ufunc_default_kwargs[key]:
            if np_ufunc_legal_option(key, value):
                raise NotImplementedError('{}={} is not implemented yet for operator {}'.format(key, str(value), func.__name__))
            raise TypeError('{}={} not understood for operator {}'.format(key, value, func.__name__))


def wrap_np_unary_func(func):
    """Uniform handling of the ufunc keyword arguments (where, casting, order, dtype, subok) for unary functions."""
    @functools.wraps(func)
    def _wrap_np_unary_func(x, out=None, **kwargs):
        _check_ufunc_kwargs(func, kwargs)
        return func(x, out=out)
    return _wrap_np_unary_func


def wrap_np_binary_func(func):
    @functools.wraps(func)
    def _wrap_np_binary_func(x1, x2, out=None, **kwargs):
        _check_ufunc_kwargs(func, kwargs)
        return func(x1, x2, out=out)
    return _wrap_np_binary_func


def wrap_data_api_statical_func(func):
    """``ddof=`` of NumPy accepted for the array-API ``correction=``."""
    @functools.wraps(func)
    def _wrap(*args, **kwargs):
        correction = kwargs.pop('ddof', None)
        if correction is not None:
            kwargs['correction'] = correction
        return func(*args, **kwargs)
    return _wrap


def wrap_data_api_linalg_func(func):
    """``UPLO=`` / ``rcond=`` / ``tol=`` of NumPy accepted for the array-API ``upper=`` / ``rtol=``."""
    @functools.wraps(func)
    def _wrap(*args, **kwargs):
        uplo, rcond, tol = kwargs.pop('UPLO', None), kwargs.pop('rcond', None), kwargs.pop('tol', None)
        if uplo is not None:
            kwargs['upper'] = uplo == 'U'
        if rcond is not None:
            kwargs['rtol'] = rcond
        if tol is not None:
            kwargs['rtol'] = tol
        return func(*args, **kwargs)
    return _wrap


def wrap_sort_functions(func):
    """``kind='stable'`` of NumPy accepted for the array-API ``stable=``; ``order=`` is not supported."""
    @functools.wraps(func)
    def _wrap(*args, **kwargs):
        kind, order = kwargs.pop('kind', None), kwargs.pop('order', None)
        if kind is not None:
            kwargs['stable'] = kind == 'stable'
        if order is not None:
            raise NotImplementedError('order not supported here')
        return func(*args, **kwargs)
    return _wrap


def numpy_fallback(func):
    """Run ``func`` on official NumPy arrays: framework arrays among the arguments are copied to the host, NumPy results
    come back as framework arrays on the device of the inputs."""
    import numpy as _np

    def to_host(obj, dev):
        if hasattr(obj, 'asnumpy'):
            return obj.asnumpy(), (dev[0] or obj.context,)
        if isinstance(obj, (list, tuple)):
            out = []
            for o in obj:
                v, dev = to_host(o, dev)
                out.append(v)
            return obj.__class__(out), dev
        if isinstance(obj, dict):
            out = {}
            for k, o in obj.items():
                out[k], dev = to_host(o, dev)
            return out, dev
        return obj, dev

    def to_device(obj, dev):
        from . import numpy as mxnp
        if isinstance(obj, _np.ndarray):
            return mxnp.array(obj, dtype=obj.dtype, ctx=dev)
        if isinstance(obj, (list, tuple)):
            return obj.__class__([to_device(o, dev) for o in obj])
        if isinstance(obj, dict):
            return {k: to_device(o, dev) for k, o in obj.items()}
        return obj

    @functools.wraps(func)
    def _fallback(*args, **kwargs):
        a, dev = to_host(args, (None,))
        k, dev = to_host(kwargs, dev)
        return to_device(func(*a, **k), dev[0])
    return _fallback


def np_default_dtype(active=True):
    """Scope in which creation functions default to float64 / int64 like NumPy (instead of float32)."""
    return _NumpyScope('np_default_dtype', active)


def use_np_default_dtype(func):
    """Decorator form of :func:`np_default_dtype` for a function or every method of a class."""
    return _wrap_scope(func, ['np_default_dtype'])


def set_np_default_dtype(is_np_default_dtype=True):   # pylint: disable=redefined-outer-name
    """Switch the NumPy default-dtype semantics globally; returns the previous setting."""
    prev = _state.state.np_default_dtype
    _state.state.np_default_dtype = bool(is_np_default_dtype)
    return prev


def get_max_supported_compute_capability():
    """Highest compute capability (major * 10 + minor) the run-time compiler of this installation can target."""
    try:
        try:
            from cuda.bindings import nvrtc
        except ImportError:
            from cuda import nvrtc
        err, n = nvrtc.nvrtcGetNumSupportedArchs()
        err, archs = nvrtc.nvrtcGetSupportedArchs()
        return int(max(archs))
    except Exception:   # pylint: disable=broad-except
        return 100


def get_rtc_compile_opts(device):
    """NVRTC options for code that is to run on ``device``: machine code for its architecture when the compiler knows it,
    otherwise PTX for the newest architecture it knows (the driver finishes the compilation)."""
    cc = get_cuda_compute_capability(device)
    max_cc = get_max_supported_compute_capability()
    to_sass = cc <= max_cc
    arch = cc if to_sass else max_cc
    suffix = 'a' if to_sass and arch >= 90 else ''
    return ['--gpu-architecture={}_{}{}'.format('sm' if to_sass else 'compute', arch, suffix)]


def set_flush_denorms(value):
    """Flush denormal floats to zero in host arithmetic (the tensor library's switch); returns the previous state."""
    import torch
    prev = bool(getattr(set_flush_denorms, '_state', False))
    ok = torch.set_flush_denormal(bool(value))
    set_flush_denorms._state = bool(value) and ok
    return prev


def dtype_from_number(number):
    """The dtype a Python or NumPy scalar gets as an array: bool, int64 (int32 for np.int32), float32 or float64 under
    NumPy default-dtype semantics."""
    import numpy as _np
    if isinstance(number, (bool, _np.bool_)):
        return _np.bool_
    if isinstance(number, (int, _np.integer)) and not isinstance(number, _np.generic):
        return _np.int64
    if isinstance(number, float):
        return _np.float64 if is_np_default_dtype() else _np.float32
    if isinstance(number, _np.generic):
        return number.dtype.type
    raise TypeError('type {} not supported'.format(str(type(number))))


from tempfile import TemporaryDirectory   # noqa: E402,F401  (kept for code written against the reference's util module)

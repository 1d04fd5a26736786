"""Base definitions shared by every module: error hierarchy, dtype tables, small helpers.

Parity targets in the reference: ``python/mxnet/base.py`` (``MXNetError``, ``_Null``,
``NotImplementedForSymbol``), ``python/mxnet/error.py`` (error registry) and the dtype enum of
``3rdparty/mshadow/mshadow/base.h:352-364`` (``kFloat32=0 … kBfloat16=12``), which is the integer
written into ``.params`` files and therefore has to keep its numbering.
"""
from __future__ import annotations

import os
import numpy as _np
import torch

__all__ = ['MXNetError', 'NotImplementedForSymbol', 'NotSupportedForSparseNDArray', '_Null',
           'string_types', 'numeric_types', 'integer_types', 'classproperty']

string_types = (str,)
numeric_types = (float, int, _np.generic)
integer_types = (int, _np.integer)


class _NullType(object):
    """Placeholder for "argument not given" (distinct from ``None``, which is a legal value)."""

    def __repr__(self):
        return '_Null'

    def __bool__(self):
        return False


_Null = _NullType()


class MXNetError(RuntimeError):
    """Default error raised by the framework (reference: ``python/mxnet/base.py:93``)."""


class NotImplementedForSymbol(MXNetError):
    """Raised when an NDArray-only facility is used on a Symbol."""

    def __init__(self, function, alias, *args):
        super().__init__()
        self.function = getattr(function, '__name__', str(function))
        self.alias = alias
        self.args = [str(type(a)) for a in args]

    def __str__(self):
        msg = 'Function {}'.format(self.function)
        if self.alias:
            msg += ' (namely operator "{}")'.format(self.alias)
        if self.args:
            msg += ' with arguments ({})'.format(', '.join(self.args))
        msg += ' is not implemented for Symbol and only available in NDArray.'
        return msg


class NotSupportedForSparseNDArray(MXNetError):
    """Raised when a dense-only facility is used on a sparse array."""

    def __init__(self, function, alias, *args):
        super().__init__()
        self.function = getattr(function, '__name__', str(function))
        self.alias = alias
        self.args = [str(type(a)) for a in args]

    def __str__(self):
        return 'Function {} is not supported for SparseNDArray'.format(self.function)


class classproperty(object):
    def __init__(self, fget):
        self.fget = fget

    def __get__(self, obj, owner):
        return self.fget(owner)


# --------------------------------------------------------------------------------------------
# dtype tables.  The integer flag is the on-disk encoding (mshadow TypeFlag).
# --------------------------------------------------------------------------------------------
_DTYPE_NP_TO_MX = {
    None: -1,
    _np.dtype('float32'): 0,
    _np.dtype('float64'): 1,
    _np.dtype('float16'): 2,
    _np.dtype('uint8'): 3,
    _np.dtype('int32'): 4,
    _np.dtype('int8'): 5,
    _np.dtype('int64'): 6,
    _np.dtype('bool'): 7,
    _np.dtype('int16'): 8,
    _np.dtype('uint16'): 9,
    _np.dtype('uint32'): 10,
    _np.dtype('uint64'): 11,
    # 12 is bfloat16; numpy has no native bf16 so it is keyed by name below
}
_DTYPE_MX_TO_NP = {v: k for k, v in _DTYPE_NP_TO_MX.items() if k is not None}
BFLOAT16_FLAG = 12

_TORCH_TO_NP = {
    torch.float32: _np.dtype('float32'), torch.float64: _np.dtype('float64'),
    torch.float16: _np.dtype('float16'), torch.uint8: _np.dtype('uint8'),
    torch.int32: _np.dtype('int32'), torch.int8: _np.dtype('int8'),
    torch.int64: _np.dtype('int64'), torch.bool: _np.dtype('bool'),
    torch.int16: _np.dtype('int16'),
}
for _name in ('uint16', 'uint32', 'uint64'):
    if hasattr(torch, _name):
        _TORCH_TO_NP[getattr(torch, _name)] = _np.dtype(_name)
_NP_TO_TORCH = {v: k for k, v in _TORCH_TO_NP.items()}

_TORCH_TO_FLAG = {t: _DTYPE_NP_TO_MX[n] for t, n in _TORCH_TO_NP.items()}
_TORCH_TO_FLAG[torch.bfloat16] = BFLOAT16_FLAG
_FLAG_TO_TORCH = {v: k for k, v in _TORCH_TO_FLAG.items()}


class _BFloat16Name(str):
    """Stand-in dtype object for bfloat16 (NumPy has none).  Compares equal to 'bfloat16'."""
    name = 'bfloat16'
    itemsize = 2
    kind = 'f'


bfloat16 = _BFloat16Name('bfloat16')


def to_torch_dtype(dtype):
    """Accepts numpy dtypes, python types, strings, torch dtypes; returns a torch dtype."""
    if dtype is None:
        return None
    if isinstance(dtype, torch.dtype):
        return dtype
    if isinstance(dtype, str) and dtype == 'bfloat16':
        return torch.bfloat16
    if dtype is bool:
        return torch.bool
    if dtype is int:
        return torch.int64
    if dtype is float:
        return torch.float64
    try:
        return _NP_TO_TORCH[_np.dtype(dtype)]
    except (KeyError, TypeError):
        raise TypeError('unsupported dtype %r' % (dtype,))


def to_numpy_dtype(dtype):
    """Inverse of :func:`to_torch_dtype`; bfloat16 maps to the :data:`bfloat16` stand-in."""
    if dtype is None:
        return None
    if isinstance(dtype, torch.dtype):
        if dtype == torch.bfloat16:
            return bfloat16
        return _TORCH_TO_NP[dtype]
    if isinstance(dtype, str) and dtype == 'bfloat16':
        return bfloat16
    return _np.dtype(dtype)


def dtype_name(dtype):
    d = to_numpy_dtype(dtype)
    return d.name if d is not None else 'None'


def dtype_flag(dtype):
    """mshadow type flag for a dtype (any accepted spelling)."""
    return _TORCH_TO_FLAG[to_torch_dtype(dtype)]


def flag_to_torch(flag):
    return _FLAG_TO_TORCH[int(flag)]


def is_float_dtype(dtype):
    return to_torch_dtype(dtype) in (torch.float16, torch.bfloat16, torch.float32, torch.float64)


def check_call(ret):
    """Kept for API familiarity: native calls here raise directly, so a non-zero code is an error."""
    if ret != 0:
        raise MXNetError('native call failed with code %d' % ret)


def data_dir_default():
    """Default directory for downloaded files: ``~/.mxnet`` (``%APPDATA%/mxnet`` on Windows)."""
    import platform
    if platform.system() == 'Windows':
        return os.path.join(os.environ.get('APPDATA'), 'mxnet')
    return os.path.join(os.path.expanduser('~'), '.mxnet')


def data_dir():
    """Directory for downloaded models and data sets: ``$MXNET_HOME`` or the default."""
    return os.getenv('MXNET_HOME', data_dir_default())


def c_str(string):
    """A ``ctypes`` char pointer for a Python string."""
    import ctypes
    return ctypes.c_char_p(string.encode('utf-8'))


def c_str_array(strings):
    import ctypes
    arr = (ctypes.c_char_p * len(strings))()
    arr[:] = [s.encode('utf-8') for s in strings]
    return arr


def c_array(ctype, values):
    """A ``ctypes`` array of ``ctype`` from a Python sequence."""
    out = (ctype * len(values))()
    out[:] = values
    return out


def c_array_buf(ctype, buf):
    """A ``ctypes`` array of ``ctype`` over an object with the buffer interface (no copy)."""
    return (ctype * len(buf)).from_buffer(buf)


def c_handle_array(objs):
    import ctypes
    arr = (ctypes.c_void_p * len(objs))()
    arr[:] = [getattr(o, 'handle', None) for o in objs]
    return arr


def ctypes2buffer(cptr, length):
    """Bytes of ``length`` copied from a ``ctypes`` char pointer."""
    import ctypes
    if not isinstance(cptr, ctypes.POINTER(ctypes.c_char)):
        raise TypeError('expected char pointer')
    res = bytearray(length)
    rptr = (ctypes.c_char * length).from_buffer(res)
    if not ctypes.memmove(rptr, cptr, length):
        raise RuntimeError('memmove failed')
    return res


def ctypes2numpy_shared(cptr, shape):
    """A float32 NumPy view of the memory behind a ``ctypes`` float pointer."""
    import ctypes
    if not isinstance(cptr, ctypes.POINTER(ctypes.c_float)):
        raise RuntimeError('expected float pointer')
    size = 1
    for s in shape:
        size *= s
    dbuffer = (ctypes.c_float * size).from_address(ctypes.addressof(cptr.contents))
    return _np.frombuffer(dbuffer, dtype=_np.float32).reshape(shape)


def build_param_doc(arg_names, arg_types, arg_descs, remove_dup=True):
    """The "Parameters" section of a generated operator docstring."""
    seen, lines = set(), []
    for name, type_info, desc in zip(arg_names, arg_types, arg_descs):
        if name in seen and remove_dup or name == 'num_args':
            continue
        seen.add(name)
        line = '%s : %s' % (name, type_info)
        if desc:
            line += '\n    ' + desc
        lines.append(line)
    return 'Parameters\n----------\n%s\n' % '\n'.join(lines)


def add_fileline_to_docstring(module, incursive=True):
    """The reference appends "From:<file>:<line>" of the C++ definition to operator docstrings; operators here are defined
    in Python, where that information is part of every traceback, so docstrings stay as written."""
    return None


_registered_errors = {}


def register_error(func_name=None, cls=None):
    """Register an exception class under a name so that errors raised by native code with that prefix map to it."""
    if callable(func_name):
        cls, func_name = func_name, func_name.__name__

    def register(mycls):
        _registered_errors[func_name if isinstance(func_name, str) else mycls.__name__] = mycls
        return mycls
    return register(cls) if cls is not None else register


# ---- small names scripts import from ``mxnet.base`` ----------------------------------------------------------------------
def py_str(x):
    """Text of a bytes object (``c_char_p`` results in the reference's ctypes layer)."""
    return x.decode('utf-8') if isinstance(x, (bytes, bytearray)) else str(x)


def _as_list(obj):
    """``obj`` if it is a list or tuple, else ``[obj]``."""
    return obj if isinstance(obj, (list, tuple)) else [obj]


def c2pyerror(err_msg):
    """(message, error class) of an error string produced by the native side: ``'ValueError: ...'`` selects a registered
    Python error class, anything else is an :class:`MXNetError`."""
    head, _, rest = str(err_msg).partition(':')
    cls = error_types.get(head.strip()) if head.strip().isidentifier() else None
    return (rest.strip() if cls is not None else str(err_msg)), (cls or MXNetError)


def get_last_ffi_error():
    """The last error recorded by the native runtime as an exception object."""
    from . import csrc
    try:
        msg = csrc.runtime.last_error()
    except Exception:   # pylint: disable=broad-except
        msg = ''
    text, cls = c2pyerror(msg)
    return cls(text)


import numpy as _np   # noqa: E402
mx_real_t = _np.float32
import ctypes as _ct
mx_uint, mx_int, mx_float = _ct.c_uint, _ct.c_int, _ct.c_float
error_types = _registered_errors      # the reference's name for the registry filled by register_error

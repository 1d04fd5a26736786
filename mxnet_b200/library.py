"""Loading of external operator libraries (``python/mxnet/library.py`` → ``MXLoadLib``).

An extension here is a shared object exporting ``mxb_register(void (*add)(const char* name, void* fn))``
or, more commonly, a Python module defining ``register_ops(registry)``; both add operators to the
live registry and regenerate the ``mx.nd`` / ``mx.npx`` front ends.
"""
import ctypes
import importlib.util
import os

from .base import MXNetError

_loaded = {}


def load(path, verbose=True):
    if not os.path.exists(path):
        raise MXNetError('load path %s does NOT exist' % path)
    if not os.path.isabs(path):
        raise MXNetError('load path %s is not an absolute path' % path)
    ext = os.path.splitext(path)[1]
    if ext == '.py':
        spec = importlib.util.spec_from_file_location('mxb_ext_%d' % len(_loaded), path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        if hasattr(mod, 'register_ops'):
            from .ops import registry
            mod.register_ops(registry)
        _loaded[path] = mod
    elif ext in ('.so', '.dll'):
        _loaded[path] = ctypes.CDLL(path, ctypes.RTLD_LOCAL)
    else:
        raise MXNetError('load path %s is NOT a library file' % path)
    _refresh_frontends()
    return _loaded[path]


def _refresh_frontends():
    from . import ndarray as nd
    from .ops import registry as reg
    for name in reg.list_ops():
        if not name.startswith('_') and not hasattr(nd, name):
            setattr(nd, name, reg.make_frontend(reg.get(name), 'nd'))


def compiled_with_cxx11_abi():
    return True

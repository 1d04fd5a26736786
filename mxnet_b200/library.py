"""Loading of external operator libraries (``python/mxnet/library.py`` -> ``MXLoadLib``, ``src/c_api/c_api.cc``).

Two kinds of extension are accepted by :func:`load`:

* a shared object that follows the C ABI of ``mxnet_b200/include/mxb_lib_api.h`` (the counterpart of the
  reference's ``include/mxnet/lib_api.h``): every operator descriptor the library exports becomes a registered
  operator with shape/type inference, forward, optional backward through autograd and optional per-call state;
* a Python module defining ``register_ops(registry)``.

Either way the ``mx.nd`` / ``mx.sym`` / ``mx.npx`` front ends are regenerated so the new operators are callable by
name.  A shared object without the ABI's entry points is only mapped into the process (its static initialisers run).
"""
import ctypes
import importlib.util
import os

import torch

from .base import MXNetError, _FLAG_TO_TORCH, _TORCH_TO_FLAG

API_VERSION = 1
MAX_NDIM = 8
_loaded = {}


class _Tensor(ctypes.Structure):
    _fields_ = [('data', ctypes.c_void_p), ('shape', ctypes.c_int64 * MAX_NDIM), ('ndim', ctypes.c_int32),
                ('dtype', ctypes.c_int32), ('dev_type', ctypes.c_int32), ('dev_id', ctypes.c_int32)]


class _Attrs(ctypes.Structure):
    _fields_ = [('num', ctypes.c_int32), ('keys', ctypes.POINTER(ctypes.c_char_p)), ('vals', ctypes.POINTER(ctypes.c_char_p))]


_i32p = ctypes.POINTER(ctypes.c_int32)
_i64p = ctypes.POINTER(ctypes.c_int64)
_INFER_SHAPE = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(_Attrs), ctypes.c_int32, ctypes.POINTER(_i64p), _i32p,
                                ctypes.c_int32, ctypes.POINTER(_i64p), _i32p)
_INFER_TYPE = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(_Attrs), ctypes.c_int32, _i32p, ctypes.c_int32, _i32p)
_FORWARD = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(_Attrs), ctypes.c_int32, ctypes.POINTER(_Tensor), ctypes.c_int32,
                            ctypes.POINTER(_Tensor), ctypes.c_void_p, ctypes.c_void_p)
_BACKWARD = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(_Attrs), ctypes.c_int32, ctypes.POINTER(_Tensor), ctypes.c_int32,
                             ctypes.POINTER(_Tensor), ctypes.POINTER(_Tensor), ctypes.POINTER(_Tensor), ctypes.c_void_p,
                             ctypes.c_void_p)
_CREATE_STATE = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(_Attrs), ctypes.POINTER(ctypes.c_void_p))
_DESTROY_STATE = ctypes.CFUNCTYPE(None, ctypes.c_void_p)


_PASS_RUN = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_char_p, ctypes.POINTER(_Attrs), ctypes.POINTER(ctypes.c_char_p))


class _PassDesc(ctypes.Structure):
    _fields_ = [('name', ctypes.c_char_p), ('run', _PASS_RUN)]


class _OpDesc(ctypes.Structure):
    _fields_ = [('name', ctypes.c_char_p), ('doc', ctypes.c_char_p), ('num_inputs', ctypes.c_int32),
                ('num_outputs', ctypes.c_int32), ('input_names', ctypes.POINTER(ctypes.c_char_p)),
                ('infer_shape', _INFER_SHAPE), ('infer_type', _INFER_TYPE), ('forward', _FORWARD), ('backward', _BACKWARD),
                ('create_state', _CREATE_STATE), ('destroy_state', _DESTROY_STATE)]


def _pack_attrs(attrs):
    """Attribute dict -> (_Attrs, keep-alive list); values are written the way a Symbol serialises them."""
    from .symbol.symbol import _fmt_attr
    items = [(str(k).encode(), _fmt_attr(v).encode()) for k, v in attrs.items()]
    n = len(items)
    keys = (ctypes.c_char_p * max(n, 1))(*[k for k, _ in items])
    vals = (ctypes.c_char_p * max(n, 1))(*[v for _, v in items])
    return _Attrs(n, keys, vals), (keys, vals, items)


def _pack_tensors(tensors):
    arr = (_Tensor * max(len(tensors), 1))()
    for i, t in enumerate(tensors):
        if t.dim() > MAX_NDIM:
            raise MXNetError('extension operators take at most %d dimensions, got %d' % (MAX_NDIM, t.dim()))
        arr[i].data = t.data_ptr()
        for d, s in enumerate(t.shape):
            arr[i].shape[d] = s
        arr[i].ndim = t.dim()
        arr[i].dtype = _TORCH_TO_FLAG[t.dtype]
        arr[i].dev_type = 2 if t.is_cuda else 1
        arr[i].dev_id = t.device.index or 0
    return arr


def _stream_of(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream) if t.is_cuda else ctypes.c_void_p(0)


class _ExtOp(object):
    """One operator of a loaded library, as a callable over tensors for the operator registry."""

    def __init__(self, lib, desc, path):
        self.lib, self.desc, self.path = lib, desc, path
        self.name = desc.name.decode()
        self.nin, self.nout = int(desc.num_inputs), int(desc.num_outputs)
        if desc.input_names:
            self.input_names = tuple(desc.input_names[i].decode() for i in range(self.nin))
        else:
            self.input_names = tuple('data%d' % i for i in range(self.nin)) if self.nin != 1 else ('data',)
        self.stateful = bool(desc.create_state)
        self.differentiable = bool(desc.backward)

    def _fail(self, what, rc):
        msg = ''
        if hasattr(self.lib, 'mxb_lib_last_error'):
            self.lib.mxb_lib_last_error.restype = ctypes.c_char_p
            m = self.lib.mxb_lib_last_error()
            msg = ': ' + m.decode() if m else ''
        raise MXNetError('%s of operator %s from %s returned %d%s' % (what, self.name, self.path, rc, msg))

    def infer(self, in_shapes, in_dtypes, attrs):
        """Output shapes and torch dtypes for the given input shapes and dtypes."""
        cattrs, _keep = _pack_attrs(attrs)
        d = self.desc
        if d.infer_shape:
            bufs_in = [(ctypes.c_int64 * max(len(s), 1))(*s) for s in in_shapes]
            pin = (_i64p * max(self.nin, 1))(*[ctypes.cast(b, _i64p) for b in bufs_in])
            nd_in = (ctypes.c_int32 * max(self.nin, 1))(*[len(s) for s in in_shapes])
            bufs_out = [(ctypes.c_int64 * MAX_NDIM)() for _ in range(self.nout)]
            pout = (_i64p * max(self.nout, 1))(*[ctypes.cast(b, _i64p) for b in bufs_out])
            nd_out = (ctypes.c_int32 * max(self.nout, 1))()
            rc = d.infer_shape(ctypes.byref(cattrs), self.nin, pin, nd_in, self.nout, pout, nd_out)
            if rc != 0:
                self._fail('infer_shape', rc)
            out_shapes = [tuple(bufs_out[i][k] for k in range(nd_out[i])) for i in range(self.nout)]
        else:
            out_shapes = [tuple(in_shapes[0])] * self.nout
        if d.infer_type:
            tin = (ctypes.c_int32 * max(self.nin, 1))(*[_TORCH_TO_FLAG[t] for t in in_dtypes])
            tout = (ctypes.c_int32 * max(self.nout, 1))()
            rc = d.infer_type(ctypes.byref(cattrs), self.nin, tin, self.nout, tout)
            if rc != 0:
                self._fail('infer_type', rc)
            out_dtypes = [_FLAG_TO_TORCH[tout[i]] for i in range(self.nout)]
        else:
            out_dtypes = [in_dtypes[0]] * self.nout
        return out_shapes, out_dtypes

    def forward(self, inputs, attrs, state):
        shapes, dtypes = self.infer([tuple(t.shape) for t in inputs], [t.dtype for t in inputs], attrs)
        dev = inputs[0].device
        outs = [torch.empty(s, dtype=t, device=dev) for s, t in zip(shapes, dtypes)]
        if dev.type == 'meta':                       # symbolic shape inference stops here
            return outs
        cattrs, _keep = _pack_attrs(attrs)
        cin, cout = _pack_tensors(inputs), _pack_tensors(outs)
        rc = self.desc.forward(ctypes.byref(cattrs), self.nin, cin, self.nout, cout, _stream_of(inputs[0]), state)
        if rc != 0:
            self._fail('forward', rc)
        return outs

    def backward(self, ograds, inputs, outputs, attrs, state):
        igrads = [torch.empty_like(t) for t in inputs]
        cattrs, _keep = _pack_attrs(attrs)
        rc = self.desc.backward(ctypes.byref(cattrs), self.nout, _pack_tensors(ograds), self.nin, _pack_tensors(inputs),
                                _pack_tensors(outputs), _pack_tensors(igrads), _stream_of(inputs[0]), state)
        if rc != 0:
            self._fail('backward', rc)
        return igrads

    def new_state(self, attrs):
        if not self.stateful:
            return None
        cattrs, _keep = _pack_attrs(attrs)
        h = ctypes.c_void_p()
        rc = self.desc.create_state(ctypes.byref(cattrs), ctypes.byref(h))
        if rc != 0:
            self._fail('create_state', rc)
        return _State(self, h)

    def __call__(self, *tensors, **attrs):
        if len(tensors) != self.nin:
            raise MXNetError('operator %s takes %d array inputs, got %d' % (self.name, self.nin, len(tensors)))
        inputs = [t.contiguous() for t in tensors]
        state = self.new_state(attrs) if inputs[0].device.type != 'meta' else None
        handle = state.handle if state is not None else ctypes.c_void_p(0)
        needs_grad = self.differentiable and torch.is_grad_enabled() and any(
            t.requires_grad for t in inputs if t.is_floating_point())
        if needs_grad:
            outs = _ExtFunction.apply(self, attrs, state, *inputs)
        else:
            with torch.no_grad():
                outs = self.forward(inputs, attrs, handle)
        outs = tuple(outs)
        return outs[0] if self.nout == 1 else outs


class _State(object):
    """Owner of one ``MXBOpState``: destroyed with the last reference (the autograd record or the call)."""

    def __init__(self, op, handle):
        self.op, self.handle = op, handle

    def __del__(self):
        if self.handle and self.op.desc.destroy_state:
            self.op.desc.destroy_state(self.handle)
            self.handle = None


class _ExtFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, op, attrs, state, *inputs):
        outs = op.forward(list(inputs), attrs, state.handle if state is not None else ctypes.c_void_p(0))
        ctx.op, ctx.attrs, ctx.state, ctx.nin = op, attrs, state, len(inputs)
        ctx.save_for_backward(*inputs, *outs)
        for o in outs:
            if not o.is_floating_point():
                ctx.mark_non_differentiable(o)
        return tuple(outs)

    @staticmethod
    def backward(ctx, *ograds):
        saved = ctx.saved_tensors
        inputs, outputs = list(saved[:ctx.nin]), list(saved[ctx.nin:])
        og = [g.contiguous() if g is not None else torch.zeros_like(o) for g, o in zip(ograds, outputs)]
        handle = ctx.state.handle if ctx.state is not None else ctypes.c_void_p(0)
        igrads = ctx.op.backward(og, inputs, outputs, ctx.attrs, handle)
        return (None, None, None) + tuple(g if t.is_floating_point() else None for g, t in zip(igrads, inputs))


def _load_shared_object(path, verbose):
    lib = ctypes.CDLL(path, ctypes.RTLD_LOCAL)
    if not hasattr(lib, 'mxb_lib_api_version'):
        return lib, []
    version = lib.mxb_lib_api_version()
    if version != API_VERSION:
        raise MXNetError('library %s was built for extension API version %d, this framework speaks version %d'
                         % (path, version, API_VERSION))
    if hasattr(lib, 'mxb_lib_init'):
        from .libinfo import __version__
        parts = (__version__.split('.') + ['0', '0'])[:3]
        number = int(parts[0]) * 10000 + int(parts[1]) * 100 + int(''.join(c for c in parts[2] if c.isdigit()) or 0)
        rc = lib.mxb_lib_init(ctypes.c_int(number))
        if rc != 0:
            raise MXNetError('library %s failed to initialise (mxb_lib_init returned %d)' % (path, rc))
    lib.mxb_lib_num_ops.restype = ctypes.c_int
    lib.mxb_lib_op.restype = ctypes.POINTER(_OpDesc)
    lib.mxb_lib_op.argtypes = [ctypes.c_int]
    from .ops import registry
    names = []
    for i in range(lib.mxb_lib_num_ops()):
        desc = lib.mxb_lib_op(i).contents
        if not desc.name or not desc.forward:
            raise MXNetError('library %s: operator %d has no name or no forward function' % (path, i))
        op = _ExtOp(lib, desc, path)
        if registry.has(op.name) and not isinstance(registry.get(op.name).fn, _ExtOp):
            raise MXNetError('library %s: operator name %s is already registered by the framework' % (path, op.name))
        registry._OPS[op.name] = registry.OpDef(op.name, op, op.input_names, nout=op.nout,
                                                doc=desc.doc.decode() if desc.doc else None)
        names.append(op.name)
        if verbose:
            print('loaded operator %s (%d inputs, %d outputs%s%s) from %s' % (
                op.name, op.nin, op.nout, ', differentiable' if op.differentiable else '',
                ', stateful' if op.stateful else '', os.path.basename(path)))
    if hasattr(lib, 'mxb_lib_num_passes'):
        from .symbol import passes
        lib.mxb_lib_pass.restype = ctypes.POINTER(_PassDesc)
        lib.mxb_lib_pass.argtypes = [ctypes.c_int]
        for i in range(lib.mxb_lib_num_passes()):
            desc = lib.mxb_lib_pass(i).contents
            pname = desc.name.decode()
            passes.register_backend(pname, _ExtPass(lib, desc, path))
            names.append(pname)
            if verbose:
                print('loaded graph pass %s from %s' % (pname, os.path.basename(path)))
    return lib, names


class _ExtPass(object):
    """A graph pass of a loaded library as a partitioning backend: Symbol -> JSON -> library -> JSON -> Symbol."""

    def __init__(self, lib, desc, path):
        self.lib, self.desc, self.path = lib, desc, path

    def __call__(self, sym, args=None, aux=None, **options):
        from .symbol import load_json
        cattrs, _keep = _pack_attrs(options)
        out = ctypes.c_char_p()
        rc = self.desc.run(sym.tojson().encode(), ctypes.byref(cattrs), ctypes.byref(out))
        if rc != 0 or not out.value:
            msg = ''
            if hasattr(self.lib, 'mxb_lib_last_error'):
                self.lib.mxb_lib_last_error.restype = ctypes.c_char_p
                m = self.lib.mxb_lib_last_error()
                msg = ': ' + m.decode() if m else ''
            raise MXNetError('graph pass %s from %s returned %d%s' % (self.desc.name.decode(), self.path, rc, msg))
        return load_json(out.value.decode())


def load(path, verbose=True):
    """Load an operator library and register what it provides; returns the loaded module or library handle."""
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
        lib, names = _load_shared_object(path, verbose)
        lib._mxb_ops = names
        _loaded[path] = lib
    else:
        raise MXNetError('load path %s is NOT a library file' % path)
    _refresh_frontends()
    return _loaded[path]


def loaded_libraries():
    """Paths of the libraries loaded so far."""
    return list(_loaded)


def include_dir():
    """Directory of ``mxb_lib_api.h`` for building an operator library (``-I`` argument)."""
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), 'include')


def _refresh_frontends():
    from . import ndarray as nd
    from . import symbol as sym
    from . import numpy_extension as npx
    from .ops import registry as reg
    from .symbol import _op_frontend
    for name in reg.list_ops():
        if name.startswith('_'):
            continue
        op = reg.get(name)
        ext = isinstance(op.fn, _ExtOp)
        if ext or not hasattr(nd, name):
            fn = reg.make_frontend(op, 'nd')
            setattr(nd, name, fn)
            setattr(nd.op, name, fn)
        if ext or not hasattr(sym, name):
            setattr(sym, name, _op_frontend(op))
        if ext:
            setattr(npx, name, reg.make_frontend(op, 'np'))


def compiled_with_cxx11_abi():
    return True


def compiled_with_gcc_cxx11_abi():
    """Whether the native libraries use the C++11 ABI of libstdc++ (they are built in-tree with the system g++)."""
    return True

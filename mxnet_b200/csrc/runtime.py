"""ctypes bindings of the native runtime library ``libmxb200_rt.so`` (engine, storage pools,
``.params`` container, RecordIO, profiler back end).

The library is built in-tree from the ``.cc`` files next to this module (``build_runtime``); it is
compiled on first import when missing so a fresh checkout works on a CPU-only machine.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import threading

from ..base import MXNetError

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, 'libmxb200_rt.so')
SOURCES = ['engine.cc', 'storage.cc', 'ndarray_io.cc', 'recordio.cc', 'profiler.cc', 'c_api.cc']
_lib = None
_lock = threading.Lock()

c_i64, c_u64, c_vp, c_cp, c_int = ctypes.c_int64, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int


def build_runtime(force=False):
    srcs = [os.path.join(_HERE, s) for s in SOURCES]
    if not force and os.path.exists(LIB_PATH) and \
            all(os.path.getmtime(LIB_PATH) >= os.path.getmtime(s) for s in srcs):
        return LIB_PATH
    cmd = ['g++', '-O2', '-std=c++17', '-fPIC', '-shared', '-pthread'] + srcs + ['-o', LIB_PATH + '.tmp', '-ldl', '-lrt']
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise MXNetError('building the native runtime failed:\n' + r.stderr)
    os.replace(LIB_PATH + '.tmp', LIB_PATH)
    return LIB_PATH


TASK_FN = ctypes.CFUNCTYPE(c_int, c_vp, ctypes.c_char_p, c_int)
_RAW_TASK_FN = ctypes.CFUNCTYPE(c_int, c_vp, c_vp, c_int)


def lib():
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                override = os.environ.get('MXNET_LIBRARY_PATH')
                path = override if override else build_runtime()
                L = ctypes.CDLL(path)
                _declare(L)
                _lib = L
    return _lib


def _declare(L):
    def sig(name, res, *args):
        f = getattr(L, name)
        f.restype = res
        f.argtypes = list(args)
    sig('mxb_engine_create', c_vp, c_int, c_int)
    sig('mxb_engine_create_ex', c_vp, c_int, c_int, c_int)
    sig('mxb_engine_destroy', None, c_vp)
    sig('mxb_engine_new_var', c_vp, c_vp)
    sig('mxb_engine_delete_var', None, c_vp, c_vp)
    sig('mxb_engine_var_version', c_u64, c_vp)
    sig('mxb_engine_push', None, c_vp, _RAW_TASK_FN, c_vp, ctypes.POINTER(c_vp), c_int, ctypes.POINTER(c_vp), c_int, c_int, c_cp)
    sig('mxb_engine_wait_var', c_int, c_vp, c_vp, ctypes.c_char_p, c_int)
    sig('mxb_engine_wait_all', c_int, c_vp, ctypes.c_char_p, c_int)
    sig('mxb_engine_num_pending', c_i64, c_vp)
    sig('mxb_pool_create', c_vp, c_int, c_int, c_int, c_u64, c_u64, c_int, c_int)
    sig('mxb_pool_destroy', None, c_vp)
    sig('mxb_pool_alloc', c_vp, c_vp, c_u64, c_int, ctypes.POINTER(c_u64))
    sig('mxb_pool_free', None, c_vp, c_vp, c_u64)
    sig('mxb_pool_direct_free', None, c_vp, c_vp, c_u64)
    sig('mxb_pool_release_all', None, c_vp)
    sig('mxb_pool_round', c_u64, c_vp, c_u64)
    sig('mxb_pool_stats', None, c_vp, ctypes.POINTER(c_i64))
    sig('mxb_cuda_runtime_found', c_int)
    sig('mxb_shm_open', c_vp, c_cp, c_u64, c_int, ctypes.POINTER(c_u64))
    sig('mxb_shm_close', c_int, c_cp, c_vp)
    sig('mxb_shm_detach', c_int, c_vp)
    sig('mxb_shm_adopt', c_vp, c_cp, ctypes.POINTER(c_u64))
    sig('mxb_ndlist_load_file', c_vp, c_cp)
    sig('mxb_ndlist_load_buffer', c_vp, c_vp, c_u64)
    sig('mxb_ndlist_free', None, c_vp)
    sig('mxb_ndlist_error', c_cp, c_vp)
    sig('mxb_ndlist_count', c_i64, c_vp)
    sig('mxb_ndlist_num_names', c_i64, c_vp)
    sig('mxb_ndlist_name', c_vp, c_vp, c_i64, ctypes.POINTER(c_i64))
    sig('mxb_ndlist_meta', None, c_vp, c_i64, ctypes.POINTER(c_i64))
    sig('mxb_ndlist_shape', None, c_vp, c_i64, ctypes.POINTER(c_i64))
    sig('mxb_ndlist_storage_shape', None, c_vp, c_i64, ctypes.POINTER(c_i64))
    sig('mxb_ndlist_data', c_vp, c_vp, c_i64, ctypes.POINTER(c_u64))
    sig('mxb_ndlist_aux', c_vp, c_vp, c_i64, c_int, ctypes.POINTER(c_i64), ctypes.POINTER(c_i64), ctypes.POINTER(c_u64))
    sig('mxb_ndwriter_create', c_vp)
    sig('mxb_ndwriter_free', None, c_vp)
    sig('mxb_ndwriter_add_dense', None, c_vp, c_int, ctypes.POINTER(c_i64), c_int, c_int, c_int, c_int, c_vp, c_u64, c_int)
    sig('mxb_ndwriter_add_sparse', None, c_vp, c_int, ctypes.POINTER(c_i64), c_int, ctypes.POINTER(c_i64), c_int, c_int,
        c_int, c_int, c_vp, c_u64, c_int, ctypes.POINTER(c_vp), ctypes.POINTER(c_i64))
    sig('mxb_ndwriter_add_name', None, c_vp, c_cp, c_u64)
    sig('mxb_ndwriter_save', c_int, c_vp, c_cp)
    sig('mxb_ndwriter_size', c_u64, c_vp)
    sig('mxb_ndwriter_to_buffer', None, c_vp, c_vp)
    sig('mxb_rec_writer_open', c_vp, c_cp, c_int)
    sig('mxb_rec_writer_tell', c_i64, c_vp)
    sig('mxb_rec_writer_write', c_int, c_vp, c_vp, c_u64)
    sig('mxb_rec_writer_close', None, c_vp)
    sig('mxb_rec_reader_open', c_vp, c_cp)
    sig('mxb_rec_reader_next', c_vp, c_vp, ctypes.POINTER(c_u64))
    sig('mxb_rec_reader_seek', None, c_vp, c_i64)
    sig('mxb_rec_reader_tell', c_i64, c_vp)
    sig('mxb_rec_reader_close', None, c_vp)
    sig('mxb_rec_prefetch_open', c_vp, c_cp, ctypes.POINTER(c_i64), c_i64, c_int)
    sig('mxb_rec_prefetch_next', c_vp, c_vp, ctypes.POINTER(c_u64))
    sig('mxb_rec_prefetch_close', None, c_vp)
    sig('mxb_csv_load', ctypes.POINTER(ctypes.c_float), c_cp, ctypes.POINTER(c_i64), ctypes.POINTER(c_i64))
    sig('mxb_libsvm_load', c_int, c_cp, ctypes.POINTER(ctypes.POINTER(ctypes.c_float)),
        ctypes.POINTER(ctypes.POINTER(ctypes.c_float)), ctypes.POINTER(ctypes.POINTER(c_i64)),
        ctypes.POINTER(ctypes.POINTER(c_i64)), ctypes.POINTER(c_i64), ctypes.POINTER(c_i64))
    sig('mxb_free', None, c_vp)
    sig('mxb_prof_now_us', c_i64)
    sig('mxb_prof_set_state', None, c_int)
    sig('mxb_prof_get_state', c_int)
    sig('mxb_prof_clear', None)
    sig('mxb_prof_name_process', None, c_int, c_cp)
    sig('mxb_prof_add', None, c_cp, c_cp, ctypes.c_char, c_i64, c_i64, c_int, c_int, ctypes.c_double)
    sig('mxb_prof_count', c_i64)
    sig('mxb_prof_dump', c_int, c_cp)
    sig('mxb_prof_aggregate', c_i64, ctypes.c_char_p, c_i64, c_int, c_int, c_int, c_int)


# ------------------------------------------------------------------------------------------------
# Engine wrapper
# ------------------------------------------------------------------------------------------------
class Var(object):
    __slots__ = ('handle', '_engine')

    def __init__(self, engine):
        self._engine = engine
        self.handle = lib().mxb_engine_new_var(engine._h)

    @property
    def version(self):
        return lib().mxb_engine_var_version(self.handle)


class Engine(object):
    """Python view of the native dependency engine.  ``push(fn, read_vars, write_vars, priority)``
    schedules ``fn()``; exceptions raised by ``fn`` are carried through the vars it mutates."""

    def __init__(self, naive=False, num_workers=2, num_priority_workers=2, kind=None):
        """``kind``: ``'NaiveEngine'`` (inline), ``'ThreadedEngine'`` (one pool of ``num_workers + num_priority_workers``
        workers on one queue) or ``'ThreadedEnginePerDevice'`` (the default: ``num_priority_workers`` workers are reserved
        for positive-priority operations)."""
        if kind is None:
            kind = 'NaiveEngine' if naive else 'ThreadedEnginePerDevice'
        naive = kind == 'NaiveEngine'
        if naive:
            self._h = lib().mxb_engine_create_ex(1, 1, 0)
        elif kind == 'ThreadedEngine':
            self._h = lib().mxb_engine_create_ex(0, int(num_workers + num_priority_workers), 0)
        else:
            self._h = lib().mxb_engine_create_ex(2, int(num_workers), int(num_priority_workers))
        self.kind = kind
        self.naive = naive
        self._tasks = {}
        self._errors = {}
        self._next = 1
        self._tlock = threading.Lock()

        def trampoline(arg, errbuf, errlen):
            tid = int(arg) if arg else 0
            with self._tlock:
                fn = self._tasks.pop(tid, None)
            if fn is None:
                return 0
            try:
                fn()
                return 0
            except BaseException as e:  # pylint: disable=broad-except
                with self._tlock:
                    self._errors[tid] = e
                msg = ('__pyexc__%d:%s: %s' % (tid, type(e).__name__, e)).encode('utf-8', 'replace')[:errlen - 1]
                ctypes.memmove(errbuf, msg + b'\0', len(msg) + 1)
                return 1
        self._trampoline = _RAW_TASK_FN(trampoline)

    def new_var(self):
        return Var(self)

    def delete_var(self, var):
        lib().mxb_engine_delete_var(self._h, var.handle)

    def push(self, fn, read_vars=(), write_vars=(), priority=0, name='task'):
        writes = list(dict.fromkeys(write_vars))
        wset = {id(v) for v in writes}
        reads = [v for v in dict.fromkeys(read_vars) if id(v) not in wset]
        with self._tlock:
            tid = self._next
            self._next += 1
            self._tasks[tid] = fn
        r = (c_vp * max(len(reads), 1))(*[v.handle for v in reads])
        w = (c_vp * max(len(writes), 1))(*[v.handle for v in writes])
        lib().mxb_engine_push(self._h, self._trampoline, c_vp(tid), r, len(reads), w, len(writes), int(priority),
                              name.encode())

    def _raise(self, buf):
        msg = buf.value.decode('utf-8', 'replace')
        if msg.startswith('__pyexc__'):
            tid = int(msg[9:].split(':', 1)[0])
            with self._tlock:
                e = self._errors.get(tid)
            if e is not None:
                raise e
            msg = msg.split(':', 1)[1]
        raise MXNetError(msg)

    def wait_for_var(self, var):
        buf = ctypes.create_string_buffer(2048)
        if lib().mxb_engine_wait_var(self._h, var.handle, buf, 2048):
            self._raise(buf)

    def wait_all(self):
        buf = ctypes.create_string_buffer(2048)
        if lib().mxb_engine_wait_all(self._h, buf, 2048):
            self._raise(buf)

    def rethrow(self):
        """Non-blocking check used by array sync points: nothing pending and an error stored."""
        if self.num_pending == 0 and self._errors:
            self.wait_all()

    @property
    def num_pending(self):
        return lib().mxb_engine_num_pending(self._h)

    def __del__(self):
        try:
            if self._h:
                lib().mxb_engine_destroy(self._h)
                self._h = None
        except Exception:  # pylint: disable=broad-except
            pass


# ------------------------------------------------------------------------------------------------
# Storage pools
# ------------------------------------------------------------------------------------------------
_STRATEGY = {'naive': 0, 'round': 1, 'unpooled': 2}


class Pool(object):
    """One pooled allocator (device type: 1 cpu, 2 gpu, 3 cpu_pinned)."""

    def __init__(self, dev_type, dev_id=0, strategy='Naive', page=4096, large_round=2 << 20, reserve=5, cutoff=24):
        self._h = lib().mxb_pool_create(dev_type, dev_id, _STRATEGY[strategy.lower()], page, large_round, reserve, cutoff)
        self.dev_type, self.dev_id = dev_type, dev_id

    def alloc(self, nbytes, failsafe=False):
        rounded = c_u64(0)
        p = lib().mxb_pool_alloc(self._h, int(nbytes), 1 if failsafe else 0, ctypes.byref(rounded))
        if not p:
            if failsafe:
                return None, 0
            raise MXNetError('out of memory allocating %d bytes on device type %d' % (nbytes, self.dev_type))
        return p, rounded.value

    def free(self, ptr, rounded):
        lib().mxb_pool_free(self._h, c_vp(ptr), rounded)

    def direct_free(self, ptr, rounded):
        lib().mxb_pool_direct_free(self._h, c_vp(ptr), rounded)

    def release_all(self):
        lib().mxb_pool_release_all(self._h)

    def round_size(self, n):
        return lib().mxb_pool_round(self._h, int(n))

    def stats(self):
        out = (c_i64 * 6)()
        lib().mxb_pool_stats(self._h, out)
        return dict(zip(('used', 'pooled', 'total', 'peak', 'hits', 'misses'), list(out)))

    def __del__(self):
        try:
            if self._h:
                lib().mxb_pool_destroy(self._h)
                self._h = None
        except Exception:  # pylint: disable=broad-except
            pass

"""Execution engine front end: streams, events, bulking scopes, async error surfacing.

Reference: ``include/mxnet/engine.h:213-437`` and ``src/engine/*`` (a thread-pool dependency
scheduler with per-device worker threads and per-variable read/write queues) plus
``python/mxnet/engine.py`` (``bulk``/``set_bulk_size``).

Design here: on a GPU the CUDA stream *is* the scheduler.  Every device owns a small set of
streams (compute = the tensor library's current stream, two communication streams with high/low
priority, copy-in, copy-out) and an event pool; ordering between streams is expressed with
events exactly like the reference's async-dependency mode (``SyncObject{reader_events,
writer_event}``, ``src/engine/threaded_engine.cc:627-747``).  Host-side tasks (data pipeline,
checkpoint writers, KVStore control messages) run on the native C++ dependency engine
(``csrc/engine.cc``) which keeps the var/read/write/priority/exception contract.  Failures of
asynchronous work are stored and rethrown at the next synchronisation point
(``wait_to_read``/``waitall``), as ``test_exc_handling.py`` requires.
"""
from __future__ import annotations

import contextlib
import threading
import weakref

import torch

from . import _state, env
from .base import MXNetError

__all__ = ['bulk', 'set_bulk_size', 'waitall', 'streams', 'is_naive', 'push_async_error', 'native', 'push', 'wait_for',
           'var_of', 'to_device_async', 'pinned_pool']

_pending = []
_pending_lock = threading.Lock()


def is_naive():
    """``MXNET_ENGINE_TYPE=NaiveEngine``: every operation completes before the call returns."""
    return env.get('MXNET_ENGINE_TYPE') == 'NaiveEngine'


def push_async_error(exc):
    """Record a failure raised by asynchronous work; rethrown at the next sync point."""
    with _pending_lock:
        _pending.append(exc)


def _rethrow_pending():
    if _pending:
        with _pending_lock:
            exc = _pending.pop(0) if _pending else None
        if exc is not None:
            raise exc
    n = _native_if_loaded()
    if n is not None:
        n.rethrow()


def _sync_device(device):
    try:
        torch.cuda.current_stream(device).synchronize()
        st = _streams.get(device.index if device.index is not None else torch.cuda.current_device())
        if st is not None:
            st.sync_side_streams()
    except RuntimeError as e:   # CUDA errors surface here as the reference's async exceptions do
        raise MXNetError(str(e))


def waitall():
    """Wait for all devices and host tasks; rethrow the first stored asynchronous failure."""
    n = _native_if_loaded()
    if n is not None:
        n.wait_all()
    if torch.cuda.is_available() and torch.cuda.is_initialized():
        for i in range(torch.cuda.device_count()):
            try:
                torch.cuda.synchronize(i)
            except RuntimeError as e:
                raise MXNetError(str(e))
    _check_fused_steps()
    _rethrow_pending()


def _check_fused_steps():
    """A fused optimizer step reports a device-side wait time-out through a status word; look at it here (and at exit), so
    that a failed LAST step is not silent."""
    import sys
    fused = sys.modules.get(__package__ + '.parallel.fused')
    if fused is not None:
        fused.check_all()


def _at_exit():
    try:
        _check_fused_steps()
    except MXNetError as e:          # no caller is left to catch it: say it on stderr
        import sys
        sys.stderr.write('mxnet_b200: %s\n' % e)


import atexit as _atexit  # noqa: E402
_atexit.register(_at_exit)


def set_bulk_size(size):
    """Maximum number of operators fused into one scheduling unit (kept for API parity: with
    stream execution there is no per-op scheduling cost to amortise; hybridize() captures CUDA
    graphs instead).  Returns the previous value."""
    prev = _state.state.bulk_size
    _state.state.bulk_size = int(size)
    return prev


@contextlib.contextmanager
def bulk(size):
    prev = set_bulk_size(size)
    try:
        yield
    finally:
        set_bulk_size(prev)


class DeviceStreams(object):
    """Streams and events of one GPU.

    compute    – the tensor library's current stream (forward/backward kernels)
    comm_high  – gradient reduce-scatter / all-gather of the earliest-needed buckets
    comm_low   – remaining communication
    copy_in    – host→device input staging
    copy_out   – device→host (metrics, checkpoints)
    """

    def __init__(self, index):
        self.index = index
        lo, hi = torch.cuda.Stream.priority_range() if hasattr(torch.cuda.Stream, 'priority_range') else (0, -1)
        with torch.cuda.device(index):
            self.comm_high = torch.cuda.Stream(device=index, priority=-1)
            self.comm_low = torch.cuda.Stream(device=index, priority=0)
            self.copy_in = torch.cuda.Stream(device=index, priority=0)
            self.copy_out = torch.cuda.Stream(device=index, priority=0)
        self._events = []
        self._lock = threading.Lock()

    @property
    def compute(self):
        return torch.cuda.current_stream(self.index)

    def event(self):
        """An event from the pool (the reference keeps a 64-entry ring per device)."""
        with self._lock:
            if self._events:
                return self._events.pop()
        return torch.cuda.Event(enable_timing=False)

    def recycle(self, ev):
        with self._lock:
            if len(self._events) < 64:
                self._events.append(ev)

    def order(self, producer, consumer):
        """Make ``consumer`` wait for everything queued so far on ``producer``."""
        ev = self.event()
        ev.record(producer)
        consumer.wait_event(ev)
        self.recycle(ev)

    def sync_side_streams(self):
        for s in (self.comm_high, self.comm_low, self.copy_in, self.copy_out):
            s.synchronize()


_streams = {}


def streams(device=None):
    """The :class:`DeviceStreams` of a GPU (index, torch.device or Device)."""
    if device is None:
        idx = torch.cuda.current_device()
    elif isinstance(device, int):
        idx = device
    elif isinstance(device, torch.device):
        idx = device.index if device.index is not None else torch.cuda.current_device()
    else:
        idx = device.device_id
    st = _streams.get(idx)
    if st is None:
        st = _streams[idx] = DeviceStreams(idx)
    return st


# ---- native host engine -----------------------------------------------------------------------
_native = None


def _native_if_loaded():
    return _native


def native():
    """The native dependency engine for host tasks (loaded on first use)."""
    global _native
    if _native is None:
        from .csrc import runtime
        kind = env.get('MXNET_ENGINE_TYPE')
        _native = runtime.Engine(kind=kind if kind in ('NaiveEngine', 'ThreadedEngine') else 'ThreadedEnginePerDevice',
                                 num_workers=max(1, int(env.get('MXNET_CPU_WORKER_NTHREADS'))),
                                 num_priority_workers=max(1, int(env.get('MXNET_CPU_PRIORITY_NTHREADS'))))
    return _native


# ---- host tasks with array dependencies --------------------------------------------------------------------------
# Arrays take part in the host engine's ordering through a variable that is created the first time a host task names
# the array (reference: every NDArray owns an engine variable, include/mxnet/ndarray.h `var()`).  Device work is ordered
# by streams and events; the variable orders HOST tasks (prefetching, file I/O, asynchronous loads) among themselves and
# against the sync points `wait_to_read`, `asnumpy` and `waitall`, and carries their exceptions there.
_vars = {}                      # id(array) -> (weak reference, variable): identity, not ==, decides (arrays compare elementwise)
_vars_lock = threading.Lock()


_tls = threading.local()


def in_task():
    """True on an engine worker thread while it runs a task (sync points must not wait on the engine from there: the
    task's dependencies are already satisfied, and a nested wait would occupy a second worker)."""
    return getattr(_tls, 'depth', 0) > 0


def _as_task(fn):
    def run():
        _tls.depth = getattr(_tls, 'depth', 0) + 1
        try:
            fn()
        finally:
            _tls.depth -= 1
    return run


def var_of(arr, create=True):
    """The engine variable of an array (or of any weak-referenceable object), created on first use."""
    key = id(arr)
    with _vars_lock:
        hit = _vars.get(key)
        if hit is not None and hit[0]() is arr:
            return hit[1]
        if not create:
            return None
        v = native().new_var()

        def forget(_ref, key=key):
            with _vars_lock:
                cur = _vars.get(key)
                if cur is not None and cur[0] is _ref:
                    del _vars[key]
        _vars[key] = (weakref.ref(arr, forget), v)
        return v


def _as_vars(items):
    from .csrc.runtime import Var
    return [x if isinstance(x, Var) else var_of(x) for x in items]


def push(fn, reads=(), writes=(), priority=0, name='task'):
    """Schedule the host function ``fn()`` after every earlier task that writes one of ``reads`` / ``writes`` and after
    every earlier reader of ``writes`` (``Engine::PushAsync``, include/mxnet/engine.h:213-300).  ``reads`` / ``writes``
    hold arrays or engine variables.  An exception raised by ``fn`` is stored in the variables it writes and raised by
    the next ``wait_to_read`` / ``asnumpy`` of such an array, or by ``waitall``; tasks that depend on a failed variable
    are not run and pass the failure on.  Under ``MXNET_ENGINE_TYPE=NaiveEngine`` the task runs before ``push``
    returns and its exception is raised here."""
    eng = native()
    r, w = _as_vars(reads), _as_vars(writes)
    if _state.naive_engine or eng.naive:
        for v in r + w:                 # earlier asynchronous tasks on these variables (and their failures) first
            eng.wait_for_var(v)
        fn()
        return
    eng.push(_as_task(fn), r, w, priority, name)


def wait_for(arr):
    """Block until the host tasks that write ``arr`` have finished; raise what they raised."""
    if _native is None or in_task():
        return
    v = var_of(arr, create=False)
    if v is not None:
        _native.wait_for_var(v)


# ---- pinned staging memory and asynchronous host -> device copies ----------------------------------------------------
_pinned = None


def pinned_pool():
    """The pool of page-locked host buffers (native storage manager, rounded size classes) that stages batches for
    host -> device copies; ``None`` without a CUDA runtime."""
    global _pinned
    if _pinned is None and torch.cuda.is_available():
        torch.cuda.init()            # the tensor library reports page-locked memory as such only once it has set CUDA up
        from .csrc import runtime
        _pinned = runtime.Pool(3, 0, 'Round')
    return _pinned


def pinned_like(t):
    """A page-locked tensor of the shape and dtype of the host tensor ``t``, from the pinned pool (handed back to the pool
    when the tensor is collected), filled with ``t``'s values."""
    pool = pinned_pool()
    if pool is None or t.is_cuda or t.numel() == 0:
        return t
    import ctypes
    nbytes = t.numel() * t.element_size()
    ptr, rounded = pool.alloc(nbytes)
    raw = (ctypes.c_uint8 * nbytes).from_address(ptr)
    out = torch.frombuffer(raw, dtype=torch.uint8).view(t.dtype).view(t.shape)
    weakref.finalize(raw, pool.free, ptr, rounded)        # `raw` lives as long as the tensor's storage refers to it
    out.copy_(t)
    return out


def to_device_async(t, device):
    """Copy a host tensor to ``device`` on the device's copy-in stream and make the compute stream wait for it with an
    event (no host block): compute that is already queued keeps running while the bytes travel.  Pageable memory falls
    back to an ordinary copy."""
    if t.is_cuda or not t.is_pinned():
        return t.to(device, non_blocking=True)
    st = streams(device)
    compute = torch.cuda.current_stream(device)
    with torch.cuda.stream(st.copy_in):
        out = t.to(device, non_blocking=True)
    st.order(st.copy_in, compute)
    out.record_stream(compute)
    return out

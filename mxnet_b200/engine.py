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

import torch

from . import _state, env
from .base import MXNetError

__all__ = ['bulk', 'set_bulk_size', 'waitall', 'streams', 'is_naive', 'push_async_error', 'native']

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
        _native = runtime.Engine(naive=is_naive(),
                                 num_workers=max(1, int(env.get('MXNET_CPU_WORKER_NTHREADS'))),
                                 num_priority_workers=max(1, int(env.get('MXNET_CPU_PRIORITY_NTHREADS'))))
    return _native

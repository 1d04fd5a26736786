"""Profiler front end (``python/mxnet/profiler.py:34-531``) over the native event store
(``csrc/profiler.cc``): ``set_config/set_state/dump/dumps/pause/resume``, user objects ``Domain``,
``Task``, ``Frame``, ``Event``, ``Counter``, ``Marker`` and ``scope``.  Operator events are emitted by
the invoke hook; device time of GPU operators is measured with CUDA events on the launching stream
and resolved when the profile is dumped, so profiling does not serialise the stream."""
import contextlib
import os
import threading

import torch

from . import _state

__all__ = ['set_config', 'set_state', 'dump', 'dumps', 'pause', 'resume', 'Domain', 'Task', 'Frame', 'Event',
           'Counter', 'Marker', 'scope', 'profiler_set_config', 'profiler_set_state', 'dump_profile']

_config = {'filename': 'profile.json', 'profile_all': False, 'profile_symbolic': False, 'profile_imperative': False,
           'profile_memory': False, 'profile_api': False, 'continuous_dump': False, 'dump_period': 1.0,
           'aggregate_stats': False, 'profile_process': 'worker', 'gpu_memory_profile_filename_prefix': 'gpu_memory_profile'}
_paused = False
_gpu_pending = []      # (name, start_event, end_event, host_ts, tid)


def _rt():
    from .csrc import runtime
    return runtime.lib()


def set_config(**kwargs):
    for k in kwargs:
        if k not in _config:
            raise ValueError('unknown profiler option %s' % k)
    _config.update(kwargs)


def profiler_set_config(mode='symbolic', filename='profile.json'):
    set_config(profile_symbolic=True, profile_imperative=mode == 'all', filename=filename)


class _OpScope(object):
    __slots__ = ('name', 't0', 'ev0')

    def __init__(self, name):
        self.name = name

    def __enter__(self):
        self.t0 = _rt().mxb_prof_now_us()
        self.ev0 = None
        if torch.cuda.is_available() and torch.cuda.is_initialized():
            self.ev0 = torch.cuda.Event(enable_timing=True)
            self.ev0.record()

    def __exit__(self, *a):
        L = _rt()
        t1 = L.mxb_prof_now_us()
        tid = threading.get_ident() % 100000
        name = (_state.state.profiler_scope + self.name) if _state.state.profiler_scope != '<unk>:' else self.name
        L.mxb_prof_add(name.encode(), b'operator', b'X', self.t0, max(t1 - self.t0, 1), os.getpid(), tid, 0.0)
        if self.ev0 is not None:
            ev1 = torch.cuda.Event(enable_timing=True)
            ev1.record()
            _gpu_pending.append((name, self.ev0, ev1, self.t0, tid))


def _op_hook(opname):
    if _paused:
        return None
    return _OpScope(opname)


def set_state(state='stop', profile_process='worker'):
    assert state in ('run', 'stop')
    run = state == 'run'
    _rt().mxb_prof_set_state(1 if run else 0)
    want_ops = _config['profile_all'] or _config['profile_imperative'] or _config['profile_symbolic']
    _state.profiler_hook = _op_hook if (run and want_ops) else None


def profiler_set_state(state='stop'):
    set_state(state)


def _flush_gpu():
    L = _rt()
    if not _gpu_pending:
        return
    torch.cuda.synchronize()
    was = L.mxb_prof_get_state()
    L.mxb_prof_set_state(1)
    for name, e0, e1, ts, tid in _gpu_pending:
        try:
            dur = int(e0.elapsed_time(e1) * 1000)
        except RuntimeError:
            continue
        L.mxb_prof_add(('[gpu] ' + name).encode(), b'operator', b'X', ts, max(dur, 1), os.getpid(), 100000 + tid % 100, 0.0)
    del _gpu_pending[:]
    L.mxb_prof_set_state(was)


def dump(finished=True, profile_process='worker'):
    """Write the Chrome trace-event file named by ``filename``."""
    _flush_gpu()
    L = _rt()
    L.mxb_prof_name_process(os.getpid(), b'mxnet_b200')
    if L.mxb_prof_dump(_config['filename'].encode()) != 0:
        raise IOError('cannot write %s' % _config['filename'])
    if finished:
        L.mxb_prof_clear()


def dump_profile():
    dump(True)


def dumps(reset=False, format='table', sort_by='total', ascending=False):  # pylint: disable=redefined-builtin
    """Aggregate statistics as a table or JSON string."""
    _flush_gpu()
    import ctypes
    sort_code = {'total': 0, 'avg': 1, 'min': 2, 'max': 3, 'count': 4}[sort_by]
    assert format in ('table', 'json')
    L = _rt()
    n = L.mxb_prof_aggregate(None, 0, 1 if format == 'json' else 0, sort_code, 1 if ascending else 0, 0)
    buf = ctypes.create_string_buffer(n + 16)
    L.mxb_prof_aggregate(buf, n + 16, 1 if format == 'json' else 0, sort_code, 1 if ascending else 0, 1 if reset else 0)
    return buf.value.decode()


def pause(profile_process='worker'):
    global _paused
    _paused = True
    _rt().mxb_prof_set_state(0)


def resume(profile_process='worker'):
    global _paused
    _paused = False
    _rt().mxb_prof_set_state(1)


class Domain(object):
    def __init__(self, name):
        self.name = name

    def __str__(self):
        return self.name

    def new_task(self, name): return Task(self, name)
    def new_frame(self, name): return Frame(self, name)
    def new_counter(self, name, value=None): return Counter(self, name, value)
    def new_marker(self, name): return Marker(self, name)


class _Span(object):
    _cat = 'task'

    def __init__(self, domain, name):
        self.domain, self.name = domain, name
        self._t0 = None

    def start(self):
        self._t0 = _rt().mxb_prof_now_us()

    def stop(self):
        if self._t0 is None:
            return
        L = _rt()
        t1 = L.mxb_prof_now_us()
        cat = str(self.domain) if self.domain is not None else self._cat
        L.mxb_prof_add(self.name.encode(), cat.encode(), b'X', self._t0, max(t1 - self._t0, 1), os.getpid(),
                       threading.get_ident() % 100000, 0.0)
        self._t0 = None

    def __enter__(self):
        self.start()
        return self

    def __exit__(self, *a):
        self.stop()

    def __str__(self):
        return self.name


class Task(_Span):
    _cat = 'task'


class Frame(_Span):
    _cat = 'frame'


class Event(_Span):
    _cat = 'event'

    def __init__(self, name):
        super().__init__(None, name)


class Counter(object):
    def __init__(self, domain, name, value=None):
        self.domain, self.name, self._value = domain, name, 0
        if value is not None:
            self.set_value(value)

    def _emit(self):
        _rt().mxb_prof_add(self.name.encode(), str(self.domain).encode(), b'C', _rt().mxb_prof_now_us(), 0, os.getpid(),
                           0, float(self._value))

    def set_value(self, value):
        self._value = value
        self._emit()

    def increment(self, delta=1):
        self._value += delta
        self._emit()

    def decrement(self, delta=1):
        self._value -= delta
        self._emit()

    def __iadd__(self, v):
        self.increment(v)
        return self

    def __isub__(self, v):
        self.decrement(v)
        return self

    def __str__(self):
        return self.name


class Marker(object):
    def __init__(self, domain, name):
        self.domain, self.name = domain, name

    def mark(self, scope='process'):  # pylint: disable=redefined-outer-name
        _rt().mxb_prof_add(self.name.encode(), str(self.domain).encode(), b'i', _rt().mxb_prof_now_us(), 0, os.getpid(),
                           threading.get_ident() % 100000, 0.0)


@contextlib.contextmanager
def scope(name='<unk>:', append_mode=False):
    """Name prefix attached to operators (and allocations) executed inside (``profiler.scope``)."""
    name = name if name.endswith(':') else name + ':'
    prev = _state.state.profiler_scope
    _state.state.profiler_scope = (prev + name) if (append_mode and prev != '<unk>:') else name
    try:
        yield
    finally:
        _state.state.profiler_scope = prev


if os.environ.get('MXNET_PROFILER_AUTOSTART', '0') == '1':
    set_config(profile_all=True)
    set_state('run')


_kvstore_handle = None


def set_kvstore_handle(handle):
    """Remember the kvstore whose servers ``profile_process='server'`` commands address.  Distributed stores here have
    no separate server processes (every rank is a worker over NCCL / gloo), so server-side calls profile this process."""
    global _kvstore_handle
    _kvstore_handle = handle

"""Process-wide set-up done once at import (reference: ``src/initialize.cc:73-220`` ``LibraryInitializer``).

* **fork**: worker threads do not survive ``fork()``.  Before a fork the host engine is drained, so no task is half done in
  the child's copy of memory; in the child the engine handle, the array variables and the pinned pool of the parent are
  dropped and fresh ones are created on first use (``pthread_atfork`` handlers of the reference stop and restart its
  engine the same way).  A child must not touch the parent's CUDA context; data-loader workers batchify on the host.
* **signals**: with ``MXNET_USE_SIGNAL_HANDLER`` (default on) a fatal signal (SIGSEGV, SIGFPE, SIGABRT, SIGBUS, SIGILL)
  prints the Python stack of every thread before the process dies, the counterpart of the reference's
  ``SegfaultLogger`` stack trace.
"""
import faulthandler
import os
import sys

from . import env

_installed = False


def _before_fork():
    from . import engine
    eng = engine._native_if_loaded()
    if eng is not None:
        try:
            eng.wait_all()
        except Exception:  # pylint: disable=broad-except
            pass                        # a stored failure stays with the parent; the child starts clean


def _after_fork_in_child():
    from . import engine
    # the parent's worker threads do not exist here: forget the engine and what refers to it, without running
    # destructors that would try to join those threads
    stale = engine._native
    engine._native = None
    engine._vars.clear()
    engine._pinned = None
    if stale is not None:
        stale._h = None
        _graveyard.append(stale)


_graveyard = []


def install():
    """Idempotent; called by the package ``__init__``."""
    global _installed
    if _installed:
        return
    _installed = True
    if hasattr(os, 'register_at_fork'):
        os.register_at_fork(before=_before_fork, after_in_child=_after_fork_in_child)
    if env.get('MXNET_USE_SIGNAL_HANDLER') and not faulthandler.is_enabled():
        try:
            faulthandler.enable(file=sys.stderr, all_threads=True)
        except (ValueError, OSError, AttributeError):      # stderr replaced by an object without a file descriptor
            pass

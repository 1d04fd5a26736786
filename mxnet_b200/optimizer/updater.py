"""``Updater``: the callable ``(index, grad, weight)`` that a kvstore or a Trainer hands gradients to (API of
``python/mxnet/optimizer/updater.py``).  It creates the optimizer state of an index on first sight, moves states to the
weight's device after ``set_states``, and feeds the optimizer either one tensor at a time or, for optimizers with
``aggregate_num > 1``, in same-dtype groups of at most that many tensors so the multi-tensor kernels see batches.
States travel as a pickle of ``states`` or of ``(states, optimizer)``.
"""
import math
import pickle

from ..ndarray.ndarray import NDArray

__all__ = ['Updater', 'get_updater']


def _as_lists(index, grad, weight):
    if isinstance(index, (list, tuple)):
        return list(index), list(grad), list(weight)
    return [index], [grad], [weight]


def _chunks(seq, size):
    for start in range(0, len(seq), size):
        yield seq[start:start + size]


class Updater(object):
    def __init__(self, optimizer):
        self.optimizer = optimizer
        self.states = {}
        self.states_synced = {}
        self.aggregate_updates = optimizer.aggregate_num > 1

    def _state_for(self, idx, weight):
        """State of ``idx``, created on first use and brought to ``weight``'s device after a ``set_states``."""
        if idx not in self.states:
            self.states[idx] = self.optimizer.create_state_multi_precision(idx, weight)
        elif not self.states_synced[idx]:
            self.states[idx] = self.sync_state_context(self.states[idx], weight.context)
        self.states_synced[idx] = True
        return self.states[idx]

    def __call__(self, index, grad, weight):
        indices, grads, weights = _as_lists(index, grad, weight)
        if not weights:
            return
        # update counts are kept per device, so the replicas of a parameter advance `t` in lock step
        self.optimizer._set_current_device(weights[0].context.device_id)
        indices = [i.decode('utf-8') if isinstance(i, bytes) else i for i in indices]
        triples = [(i, w, g, self._state_for(i, w)) for i, w, g in zip(indices, weights, grads)]
        if not self.aggregate_updates:
            for i, w, g, s in triples:
                self.optimizer.update_multi_precision([i], [w], [g], [s])
            return
        by_dtype = {}
        for t in triples:
            by_dtype.setdefault(str(t[1]._data.dtype), []).append(t)
        limit = self.optimizer.aggregate_num
        for group in by_dtype.values():
            size = len(group) if math.isinf(limit) else int(limit)
            for part in _chunks(group, size):
                i, w, g, s = (list(col) for col in zip(*part))
                self.optimizer.update_multi_precision(i, w, g, s)

    def sync_state_context(self, state, context):
        """``state`` (an array, or nested tuples / lists of arrays and other values) with every array on ``context``."""
        if isinstance(state, NDArray):
            return state.as_in_context(context)
        if isinstance(state, (tuple, list)):
            return type(state)(self.sync_state_context(s, context) for s in state)
        return state

    def set_states(self, states):
        loaded = pickle.loads(states)
        if isinstance(loaded, tuple) and len(loaded) == 2:
            self.states, self.optimizer = loaded
        else:
            self.states = loaded
        self.states_synced = {k: False for k in self.states}

    def get_states(self, dump_optimizer=False):
        return pickle.dumps((self.states, self.optimizer) if dump_optimizer else self.states)


def get_updater(optimizer):
    return Updater(optimizer)

"""Updater: applies an optimizer to (index, grad, weight) triples and owns the per-index states
(``python/mxnet/optimizer/updater.py``).  Calls are aggregated per dtype in groups of
``optimizer.aggregate_num`` tensors (``updater.py:61-90``) so the multi-tensor kernels see batches."""
import pickle

import numpy

from ..ndarray.ndarray import NDArray

__all__ = ['Updater', 'get_updater']


class Updater(object):
    def __init__(self, optimizer):
        self.optimizer = optimizer
        self.states = {}
        self.states_synced = {}
        self.aggregate_updates = optimizer.aggregate_num > 1

    def __call__(self, index, grad, weight):
        if not isinstance(index, (list, tuple)):
            indices, grads, weights = [index], [grad], [weight]
        else:
            indices, grads, weights = list(index), list(grad), list(weight)
        if weights:
            # update counts are kept per device (updater.py:51), so replicas advance `t` in lock step
            self.optimizer._set_current_device(weights[0].context.device_id)
        for i, idx in enumerate(indices):
            if isinstance(idx, bytes):
                indices[i] = idx = idx.decode('utf-8')
            if idx not in self.states:
                self.states[idx] = self.optimizer.create_state_multi_precision(idx, weights[i])
                self.states_synced[idx] = True
            elif not self.states_synced[idx]:
                self.states[idx] = self.sync_state_context(self.states[idx], weights[i].context)
                self.states_synced[idx] = True
        if self.aggregate_updates:
            type_map = {}
            for i, w, g in zip(indices, weights, grads):
                type_map.setdefault(str(w._data.dtype), []).append((i, w, g))
            for group in type_map.values():
                gi, gw, gg = zip(*group)
                agg = self.optimizer.aggregate_num
                step = len(gi) if agg is numpy.inf or agg == float('inf') else int(agg)
                cur = 0
                while cur < len(gi):
                    sl = slice(cur, cur + step)
                    self.optimizer.update_multi_precision(list(gi[sl]), list(gw[sl]), list(gg[sl]),
                                                          [self.states[i] for i in gi[sl]])
                    cur += step
        else:
            for i, w, g in zip(indices, weights, grads):
                self.optimizer.update_multi_precision([i], [w], [g], [self.states[i]])

    def sync_state_context(self, state, context):
        if isinstance(state, NDArray):
            return state.as_in_context(context)
        if isinstance(state, (tuple, list)):
            synced = (self.sync_state_context(i, context) for i in state)
            return tuple(synced) if isinstance(state, tuple) else list(synced)
        return state

    def set_states(self, states):
        states = pickle.loads(states)
        if isinstance(states, tuple) and len(states) == 2:
            self.states, self.optimizer = states
        else:
            self.states = states
        self.states_synced = dict.fromkeys(self.states.keys(), False)

    def get_states(self, dump_optimizer=False):
        return pickle.dumps((self.states, self.optimizer) if dump_optimizer else self.states)


def get_updater(optimizer):
    return Updater(optimizer)

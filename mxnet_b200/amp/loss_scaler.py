"""Dynamic loss scaling (``python/mxnet/amp/loss_scaler.py:34-74``): start at 2^16, double after 2000
clean steps, halve on overflow (and skip that step), cap at 2^24.

The reference checks overflow with ``multi_all_finite`` over chunks of 200 gradients followed by a
blocking ``asnumpy``.  Here the flag stays on the device when the fused optimizer step is active
(the kernels skip the update by predicate and adjust the scale themselves); the host-side check
below is the fallback for the generic Updater path."""
import torch


class LossScaler(object):
    def __init__(self, init_scale=2. ** 16, scale_seq_len=2000, max_scale=2. ** 24, min_scale=1.0):
        self._loss_scale = float(init_scale)
        self._next_loss_scale = self._loss_scale
        self._max_loss_scale = float(max_scale)
        self._min_loss_scale = float(min_scale)
        self._scale_seq_len = scale_seq_len
        self._unskipped = 0
        self._device_state = None       # float32[2] on device: [scale, clean steps], owned by the fused path
        self._device_states = {}        # the same state on every GPU of a single-process group, by torch device

    @property
    def loss_scale(self):
        if self._device_state is not None:
            self._loss_scale = float(self._device_state[0].item())
        return self._loss_scale

    def has_overflow(self, params):
        """True when any gradient holds inf/nan (one device reduction, one host read)."""
        grads = []
        for p in params:
            if p.grad_req != 'null' and p._grad is not None:
                grads.extend(g._data for g in p._grad.values())
        if not grads:
            return False
        from ..ops import registry as _reg
        ok = None
        for i in range(0, len(grads), 200):
            r = _reg.get('multi_all_finite').fn(*grads[i:i + 200], num_arrays=len(grads[i:i + 200]))
            ok = r if ok is None else ok * r.to(ok.device)
        return not bool(ok.item())

    def update_scale(self, overflow):
        if overflow:
            self._loss_scale = max(self._loss_scale / 2., self._min_loss_scale)
            self._unskipped = 0
        else:
            self._unskipped += 1
            if self._unskipped == self._scale_seq_len:
                self._unskipped = 0
                self._loss_scale = min(self._max_loss_scale, self._loss_scale * 2.)

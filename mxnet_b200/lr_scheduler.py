"""Learning-rate schedules (API of ``python/mxnet/lr_scheduler.py``: ``LRScheduler`` and the factor, multi-factor,
polynomial and cosine schedules, each with an optional warm-up ramp).

A schedule is a callable ``num_update -> lr``.  The base class owns the warm-up phase and validation; a subclass only
describes the post-warm-up curve in ``_after_warmup``.  The decaying schedules are stateful on purpose (``base_lr`` is
the current rate and may also be set from outside, which is what ``Optimizer.set_learning_rate`` does).
"""
import logging
import math

__all__ = ['LRScheduler', 'FactorScheduler', 'MultiFactorScheduler', 'PolyScheduler', 'CosineScheduler']

_log = logging.getLogger(__name__)
_WARMUP_MODES = ('linear', 'constant')


def _require(cond, message):
    if not cond:
        raise ValueError(message)


class LRScheduler(object):
    """Base class: ``base_lr`` after an optional warm-up of ``warmup_steps`` updates that starts at ``warmup_begin_lr``
    and either rises linearly to ``base_lr`` or stays constant."""

    def __init__(self, base_lr=0.01, warmup_steps=0, warmup_begin_lr=0, warmup_mode='linear'):
        if not isinstance(warmup_steps, int):
            raise AssertionError('warmup_steps must be an int')
        _require(warmup_steps >= 0, 'Warmup steps has to be positive or 0')
        _require(warmup_begin_lr <= base_lr, 'Base lr has to be higher than warmup_begin_lr')
        _require(warmup_mode in _WARMUP_MODES, 'Supports only linear and constant modes of warmup')
        self.base_lr = base_lr
        self.warmup_steps = warmup_steps
        self.warmup_begin_lr = warmup_begin_lr
        self.warmup_final_lr = base_lr
        self.warmup_mode = warmup_mode

    def get_warmup_lr(self, num_update):
        """Rate during warm-up (``num_update < warmup_steps``)."""
        if num_update >= self.warmup_steps:
            raise AssertionError('get_warmup_lr is only defined during the warm-up')
        if self.warmup_mode == 'constant':
            return self.warmup_begin_lr
        frac = float(num_update) / float(self.warmup_steps)
        return self.warmup_begin_lr + frac * (self.warmup_final_lr - self.warmup_begin_lr)

    def _after_warmup(self, num_update):
        raise NotImplementedError('must override this')

    def __call__(self, num_update):
        if type(self)._after_warmup is LRScheduler._after_warmup:
            raise NotImplementedError('must override this')
        if num_update < self.warmup_steps:
            return self.get_warmup_lr(num_update)
        return self._after_warmup(num_update)


class FactorScheduler(LRScheduler):
    """Multiply the rate by ``factor`` every ``step`` updates, never going below ``stop_factor_lr``."""

    def __init__(self, step, factor=1, stop_factor_lr=1e-8, base_lr=0.01, warmup_steps=0, warmup_begin_lr=0,
                 warmup_mode='linear'):
        super().__init__(base_lr, warmup_steps, warmup_begin_lr, warmup_mode)
        _require(step >= 1, 'Schedule step must be greater or equal than 1 round')
        _require(factor <= 1.0, 'Factor must be no more than 1 to make lr reduce')
        self.step = step
        self.factor = factor
        self.stop_factor_lr = stop_factor_lr
        self.count = 0          # last update at which the rate was lowered

    def _after_warmup(self, num_update):
        # catch up over every boundary passed since the last call
        while self.count + self.step < num_update:
            self.count += self.step
            lowered = self.base_lr * self.factor
            if lowered < self.stop_factor_lr:
                self.base_lr = self.stop_factor_lr
                _log.info('Update[%d]: learning rate reached its floor %0.5e and stays there', num_update, self.base_lr)
            else:
                self.base_lr = lowered
                _log.info('Update[%d]: learning rate is now %0.5e', num_update, self.base_lr)
        return self.base_lr


class MultiFactorScheduler(LRScheduler):
    """Multiply the rate by ``factor`` once at each update count listed in ``step`` (strictly increasing)."""

    def __init__(self, step, factor=1, base_lr=0.01, warmup_steps=0, warmup_begin_lr=0, warmup_mode='linear'):
        super().__init__(base_lr, warmup_steps, warmup_begin_lr, warmup_mode)
        if not (isinstance(step, list) and step):
            raise AssertionError('step must be a non-empty list')
        _require(all(b > a for a, b in zip(step, step[1:])), 'Schedule step must be an increasing integer list')
        _require(all(s >= 1 for s in step), 'Schedule step must be greater or equal than 1 round')
        _require(factor <= 1.0, 'Factor must be no more than 1 to make lr reduce')
        self.step = step
        self.factor = factor
        self.cur_step_ind = 0   # index of the next boundary
        self.count = 0          # the last boundary passed

    def _after_warmup(self, num_update):
        while self.cur_step_ind < len(self.step) and num_update > self.step[self.cur_step_ind]:
            self.count = self.step[self.cur_step_ind]
            self.cur_step_ind += 1
            self.base_lr *= self.factor
            _log.info('Update[%d]: learning rate is now %0.5e', num_update, self.base_lr)
        return self.base_lr


class _DecayToFinal(LRScheduler):
    """Shared part of the schedules that go from ``base_lr`` to ``final_lr`` over ``max_update`` updates along a curve
    ``shape(progress)`` with ``shape(0) = 1`` and ``shape(1) = 0``; afterwards the rate stays where it ended."""

    def __init__(self, max_update, base_lr, final_lr, warmup_steps, warmup_begin_lr, warmup_mode):
        super().__init__(base_lr, warmup_steps, warmup_begin_lr, warmup_mode)
        if not isinstance(max_update, int):
            raise AssertionError('max_update must be an int')
        _require(max_update >= 1, 'maximum number of updates must be strictly positive')
        self.base_lr_orig = self.base_lr
        self.max_update = max_update
        self.final_lr = final_lr
        self.max_steps = max_update - self.warmup_steps

    def _shape(self, progress):
        raise NotImplementedError

    def _after_warmup(self, num_update):
        if num_update <= self.max_update:
            progress = float(num_update - self.warmup_steps) / float(self.max_steps)
            self.base_lr = self.final_lr + (self.base_lr_orig - self.final_lr) * self._shape(progress)
        return self.base_lr


class PolyScheduler(_DecayToFinal):
    """``final_lr + (base_lr - final_lr) * (1 - progress) ** pwr``."""

    def __init__(self, max_update, base_lr=0.01, pwr=2, final_lr=0, warmup_steps=0, warmup_begin_lr=0, warmup_mode='linear'):
        super().__init__(max_update, base_lr, final_lr, warmup_steps, warmup_begin_lr, warmup_mode)
        self.power = pwr

    def _shape(self, progress):
        return pow(1.0 - progress, self.power)


class CosineScheduler(_DecayToFinal):
    """``final_lr + (base_lr - final_lr) * (1 + cos(pi * progress)) / 2``."""

    def __init__(self, max_update, base_lr=0.01, final_lr=0, warmup_steps=0, warmup_begin_lr=0, warmup_mode='linear'):
        super().__init__(max_update, base_lr, final_lr, warmup_steps, warmup_begin_lr, warmup_mode)

    def _shape(self, progress):
        return 0.5 * (1.0 + math.cos(math.pi * progress))

"""Event handlers of the Gluon ``Estimator`` (API of ``python/mxnet/gluon/contrib/estimator/event_handler.py``).

The estimator calls, in order of ``priority`` (lower first), the ``train_begin / epoch_begin / batch_begin / batch_end /
epoch_end / train_end`` methods of every handler that derives from the matching mix-in class.  ``batch_end`` and
``epoch_end`` may return ``True`` to ask for training to stop.  Handlers here: stopping after a number of epochs or
batches, metric updates, periodic validation, logging, checkpointing (periodic, best-so-far, pruning, resume), early
stopping, and the optimizer step itself.
"""
import logging
import os
import re
import time
import warnings

import numpy as np

from ...metric import EvalMetric, Loss as LossMetric, CompositeEvalMetric

__all__ = ['TrainBegin', 'TrainEnd', 'EpochBegin', 'EpochEnd', 'BatchBegin', 'BatchEnd', 'StoppingHandler',
           'MetricHandler', 'ValidationHandler', 'LoggingHandler', 'CheckpointHandler', 'EarlyStoppingHandler',
           'GradientUpdateHandler']


class EventHandler(object):
    """Marker base class of everything the estimator accepts as a handler."""


def _check_event_handlers(handlers):
    """``handlers`` as a list (``None`` -> ``[]``, a single handler -> ``[handler]``); anything else is refused."""
    if isinstance(handlers, EventHandler):
        return [handlers]
    handlers = list(handlers) if handlers else []
    for h in handlers:
        if not isinstance(h, EventHandler):
            raise ValueError('handlers must be an EventHandler or a list of EventHandler, got: {}'.format(handlers))
    return handlers


# ---- the six events: a handler opts in by deriving from the mix-in and overriding its method -------------------------
class TrainBegin(EventHandler):
    def train_begin(self, estimator, *args, **kwargs):
        pass


class TrainEnd(EventHandler):
    def train_end(self, estimator, *args, **kwargs):
        pass


class EpochBegin(EventHandler):
    def epoch_begin(self, estimator, *args, **kwargs):
        pass


class EpochEnd(EventHandler):
    def epoch_end(self, estimator, *args, **kwargs):
        return False


class BatchBegin(EventHandler):
    def batch_begin(self, estimator, *args, **kwargs):
        pass


class BatchEnd(EventHandler):
    def batch_end(self, estimator, *args, **kwargs):
        return False


def _as_list(x):
    if x is None:
        return []
    return list(x) if isinstance(x, (list, tuple)) else [x]


def _metric_summary(metrics):
    """``'name: value, name: value'`` for a list of metrics."""
    return ', '.join('%s: %.4f' % m.get() for m in metrics)


def _improvement_rule(mode, monitor, who):
    """``(is_better, worst_value)`` for a monitored metric: ``min`` / ``max`` as told, ``auto`` = larger is better for
    accuracy- and F1-like names and smaller is better otherwise."""
    if mode not in ('auto', 'min', 'max'):
        warnings.warn('%s mode %s is unknown, fallback to auto mode. ' % (who, mode), RuntimeWarning)
        mode = 'auto'
    if mode == 'auto':
        name = monitor.get()[0].lower()
        mode = 'max' if ('acc' in name or 'f1' in name) else 'min'
    return (np.greater, -np.inf) if mode == 'max' else (np.less, np.inf)


class _Counters(object):
    """Batches and epochs seen since ``train_begin`` (shared by the handlers that act every N-th batch or epoch)."""

    current_batch = 0
    current_epoch = 0

    def _restart(self):
        self.current_batch = 0
        self.current_epoch = 0

    @staticmethod
    def _due(count, period):
        return bool(period) and count % period == 0


class StoppingHandler(_Counters, TrainBegin, BatchEnd, EpochEnd):
    """Asks for a stop once ``max_epoch`` epochs or ``max_batch`` batches have run (the limits are taken from the
    estimator when training begins)."""

    def __init__(self, max_epoch=None, max_batch=None):
        self.max_epoch = max_epoch
        self.max_batch = max_batch
        self.stop_training = False
        self._restart()

    def train_begin(self, estimator, *args, **kwargs):
        self.max_epoch = estimator.max_epoch
        self.max_batch = estimator.max_batch
        self._restart()

    def batch_end(self, estimator, *args, **kwargs):
        self.current_batch += 1
        self.stop_training = self.stop_training or self.current_batch == self.max_batch
        return self.stop_training

    def epoch_end(self, estimator, *args, **kwargs):
        self.current_epoch += 1
        self.stop_training = self.stop_training or self.current_epoch == self.max_epoch
        return self.stop_training


class MetricHandler(EpochBegin, BatchEnd):
    """Resets the training metrics at every epoch and feeds them after every batch: loss metrics get the loss, the
    others ``(label, pred)``.  Runs early (priority -1000) so later handlers read fresh values."""

    def __init__(self, metrics, priority=-1000):
        self.metrics = _as_list(metrics)
        self.priority = priority

    def epoch_begin(self, estimator, *args, **kwargs):
        for m in self.metrics:
            m.reset()

    def batch_end(self, estimator, *args, **kwargs):
        for m in self.metrics:
            if isinstance(m, LossMetric):
                m.update(0, kwargs['loss'])
            else:
                m.update(kwargs['label'], kwargs['pred'])


class ValidationHandler(_Counters, TrainBegin, BatchEnd, EpochEnd):
    """Runs ``eval_fn`` on ``val_data`` every ``epoch_period`` epochs and / or every ``batch_period`` batches."""

    def __init__(self, val_data, eval_fn, epoch_period=1, batch_period=None, priority=-1000, event_handlers=None):
        self.val_data = val_data
        self.eval_fn = eval_fn
        self.epoch_period = epoch_period
        self.batch_period = batch_period
        self.priority = priority
        self.event_handlers = event_handlers
        self._restart()

    def _validate(self, estimator):
        self.eval_fn(val_data=self.val_data, batch_axis=estimator.batch_axis, event_handlers=self.event_handlers)

    def train_begin(self, estimator, *args, **kwargs):
        self._restart()

    def batch_end(self, estimator, *args, **kwargs):
        self.current_batch += 1
        if self._due(self.current_batch, self.batch_period):
            self._validate(estimator)

    def epoch_end(self, estimator, *args, **kwargs):
        self.current_epoch += 1
        if self._due(self.current_epoch, self.epoch_period):
            self._validate(estimator)


class LoggingHandler(TrainBegin, TrainEnd, EpochBegin, EpochEnd, BatchBegin, BatchEnd):
    """Writes progress to ``estimator.logger``: one line per epoch (``log_interval='epoch'``) or, with an integer
    ``log_interval``, also one line every that many batches with the time the interval took.  Runs last (priority
    +inf) so that the metrics it prints are up to date."""

    def __init__(self, log_interval='epoch', metrics=None, priority=np.inf):
        if log_interval != 'epoch' and not isinstance(log_interval, int):
            raise ValueError("log_interval must be either an integer or string 'epoch'")
        self.log_interval = log_interval
        self.metrics = _as_list(metrics)
        self.priority = priority
        self.batch_index = 0
        self.current_epoch = 0
        self.processed_samples = 0
        self.log_interval_time = 0

    @property
    def _per_batch(self):
        return isinstance(self.log_interval, int)

    def _line(self, estimator, head):
        tail = _metric_summary(self.metrics)
        estimator.logger.info((head + tail).rstrip(', '))

    def train_begin(self, estimator, *args, **kwargs):
        self.train_start = time.time()
        self.current_epoch = 0
        self.batch_index = 0
        trainer = estimator.trainer
        estimator.logger.info('Training begin: using optimizer %s with current learning rate %.4f ',
                              type(trainer.optimizer).__name__, trainer.learning_rate)
        if estimator.max_epoch:
            estimator.logger.info('Train for %d epochs.', estimator.max_epoch)
        else:
            estimator.logger.info('Train for %d batches.', estimator.max_batch)

    def train_end(self, estimator, *args, **kwargs):
        elapsed = time.time() - self.train_start
        self._line(estimator, 'Train finished using total %ds with %d epochs. ' % (elapsed, self.current_epoch))

    def epoch_begin(self, estimator, *args, **kwargs):
        self.epoch_start = time.time()
        estimator.logger.info('[Epoch %d] Begin, current learning rate: %.4f', self.current_epoch,
                              estimator.trainer.learning_rate)

    def epoch_end(self, estimator, *args, **kwargs):
        self._line(estimator, '[Epoch %d] Finished in %.3fs, ' % (self.current_epoch, time.time() - self.epoch_start))
        self.current_epoch += 1
        self.batch_index = 0

    def batch_begin(self, estimator, *args, **kwargs):
        if self._per_batch:
            self.batch_start = time.time()

    def batch_end(self, estimator, *args, **kwargs):
        if self._per_batch:
            self.log_interval_time += time.time() - self.batch_start
            self.processed_samples += kwargs['batch'][0].shape[0]
            if self.batch_index % self.log_interval == 0:
                head = '[Epoch %d][Batch %d][Samples %s] time/interval: %.3fs ' % (
                    self.current_epoch, self.batch_index, self.processed_samples, self.log_interval_time)
                self.log_interval_time = 0
                self._line(estimator, head)
        self.batch_index += 1


class CheckpointHandler(_Counters, TrainBegin, BatchEnd, EpochEnd):
    """Saves ``<prefix>-epoch<E>batch<B>.params`` (network) and ``.states`` (trainer) every ``epoch_period`` epochs and /
    or ``batch_period`` batches into ``model_dir``, keeps at most ``max_checkpoints`` of them, keeps the best model so far
    as ``<prefix>-best`` when ``save_best`` (judged on ``monitor`` by ``mode``), and can resume from the newest
    checkpoint found in ``model_dir``."""

    _NAME = re.compile(r'-epoch(\d+)batch(\d+)\.params$')

    def __init__(self, model_dir, model_prefix='model', monitor=None, verbose=0, save_best=False, mode='auto',
                 epoch_period=1, batch_period=None, max_checkpoints=5, resume_from_checkpoint=False):
        if save_best and not isinstance(monitor, EvalMetric):
            raise ValueError('To save best model only, please provide one of the metric objects from '
                             'estimator.train_metrics and estimator.val_metrics as monitor.')
        os.makedirs(model_dir, exist_ok=True)
        self.model_dir = model_dir
        self.model_prefix = model_prefix
        self.monitor = monitor
        self.verbose = verbose
        self.save_best = save_best
        self.epoch_period = epoch_period
        self.batch_period = batch_period
        self.max_checkpoints = max_checkpoints
        self.resume_from_checkpoint = resume_from_checkpoint
        self.saved_checkpoints = []
        self.trained_epoch = self.trained_batch = -1
        self._restart()
        if save_best:
            self.monitor_op, self.best = _improvement_rule(mode, monitor, 'ModelCheckpoint')

    # ---- events ---------------------------------------------------------------------------------------------
    def train_begin(self, estimator, *args, **kwargs):
        self._restart()
        if self.save_best:
            self.best = np.inf if self.monitor_op is np.less else -np.inf
        if not self.resume_from_checkpoint:
            return
        # a run limited by batches must checkpoint by batches only, one limited by epochs by epochs only: otherwise
        # the numbers in the file names could not be turned back into "how much is left"
        wrong = 'To use resume from checkpoint, you must only specify the same type of period you used for training.'
        if estimator.max_batch and (not self.batch_period or self.epoch_period):
            raise AssertionError(wrong)
        if estimator.max_epoch and (not self.epoch_period or self.batch_period):
            raise AssertionError(wrong)
        self._resume_from_checkpoint(estimator)

    def batch_end(self, estimator, *args, **kwargs):
        if self.current_batch == 0:
            self._save_symbol(estimator)
        if self._due(self.current_batch + 1, self.batch_period):
            self._save_checkpoint(estimator)
        self.current_batch += 1

    def epoch_end(self, estimator, *args, **kwargs):
        if self._due(self.current_epoch + 1, self.epoch_period):
            self._save_checkpoint(estimator)
        self.current_epoch += 1

    # ---- saving ---------------------------------------------------------------------------------------------
    def _numbers_for_name(self, estimator):
        """Epoch and batch numbers that go into the file name: counted from the checkpoint a resumed run started at."""
        if not self.resume_from_checkpoint:
            return self.current_epoch, self.current_batch
        epoch = self.current_epoch + self.trained_epoch + 1
        batch = self.current_batch + self.trained_batch + (1 if estimator.max_epoch else 0)
        return epoch, batch

    def _save_checkpoint(self, estimator):
        prefix = '%s-epoch%dbatch%d' % ((self.model_prefix,) + self._numbers_for_name(estimator))
        self._save_params_and_trainer(estimator, prefix)
        if self.verbose > 0:
            estimator.logger.info('[Epoch %d] CheckpointHandler: trained total %d batches, saving model at %s with '
                                  'prefix: %s', self.current_epoch, self.current_batch + 1, self.model_dir, prefix)
        if not self.save_best:
            return
        name, value = self.monitor.get()
        if np.isnan(value):
            warnings.warn(RuntimeWarning('Skipping save best because %s is not updated, make sure you pass one of the metric '
                                         'objects estimator.train_metrics and estimator.val_metrics as monitor' % name))
        elif self.monitor_op(value, self.best):
            self.best = value
            self._save_params_and_trainer(estimator, self.model_prefix + '-best')

    def _save_symbol(self, estimator):
        graph = getattr(estimator.net, '_cached_graph', None)
        if graph:
            graph[1].save(os.path.join(self.model_dir, self.model_prefix + '-symbol.json'))

    def _save_params_and_trainer(self, estimator, file_prefix):
        base = os.path.join(self.model_dir, file_prefix)
        estimator.net.save_parameters(base + '.params')
        estimator.trainer.save_states(base + '.states')
        if 'best' in file_prefix:
            return
        self.saved_checkpoints.append(file_prefix)
        while len(self.saved_checkpoints) > self.max_checkpoints:
            oldest = self.saved_checkpoints.pop(0)
            for ext in ('.params', '.states'):
                path = os.path.join(self.model_dir, oldest + ext)
                if os.path.exists(path):
                    os.remove(path)

    # ---- resuming -------------------------------------------------------------------------------------------
    def _scan(self):
        """``[(epoch, batch, prefix)]`` of the checkpoints of this model found in ``model_dir``."""
        found = []
        for fname in os.listdir(self.model_dir):
            if not fname.startswith(self.model_prefix + '-epoch') or '.params' not in fname:
                continue
            m = self._NAME.search(fname)
            if m is None:
                raise ValueError('Error parsing checkpoint file, please check your checkpoints have the format: '
                                 '{model_name}-epoch{epoch_number}batch{batch_number}.params, there should also be a '
                                 '.states file for each .params file ')
            found.append((int(m.group(1)), int(m.group(2)), fname[:-len('.params')]))
        return sorted(found)

    def _find_max_iteration(self, dir, prefix, start, end, saved_checkpoints=None):  # pylint: disable=redefined-builtin
        """Largest number between the markers ``start`` and ``end`` in the checkpoint names beginning with ``prefix``
        (-1 if there is none); kept for callers of the original interface."""
        best = -1
        for fname in os.listdir(dir):
            if fname.startswith(prefix) and '.params' in fname:
                if saved_checkpoints:
                    saved_checkpoints.append(fname[:fname.find('.params')])
                try:
                    best = max(best, int(fname[fname.find(start) + len(start):fname.find(end)]))
                except ValueError:
                    raise ValueError('Error parsing checkpoint file, please check your checkpoints have the format: '
                                     '{model_name}-epoch{epoch_number}batch{batch_number}.params, there should also be a '
                                     '.states file for each .params file ')
        return best

    def _resume_from_checkpoint(self, estimator):
        found = self._scan()
        if not found:
            self.trained_epoch = self.trained_batch = -1
            left = '%d batches' % estimator.max_batch if estimator.max_batch else '%d epochs' % estimator.max_epoch
            estimator.logger.info('CheckpointHandler: No checkpoint found, training from scratch for ' + left)
            return
        self.saved_checkpoints = [prefix for _, _, prefix in found]     # pruning goes on from what is on disk
        self.trained_epoch = found[-1][0]
        self.trained_batch = max(b for e, b, _ in found if e == self.trained_epoch)
        newest = '%s-epoch%dbatch%d' % (self.model_prefix, self.trained_epoch, self.trained_batch)
        msg = 'CheckpointHandler: Checkpoint resumed from epoch %d batch %d, continue to train for ' % (
            self.trained_epoch, self.trained_batch)
        done_msg = 'Found checkpoint with maximum number of %s %d reached, please specify resume_from_checkpoint=False ' \
                   '(default value) if you wan to train from scratch.'
        if estimator.max_epoch:
            if self.trained_epoch >= estimator.max_epoch - 1:
                raise ValueError(done_msg % ('epoch', estimator.max_epoch))
            estimator.max_epoch -= self.trained_epoch + 1
            msg += '%d epochs ' % estimator.max_epoch
        if estimator.max_batch:
            if self.trained_batch >= estimator.max_batch - 1:
                raise ValueError(done_msg % ('batch', self.trained_batch))
            estimator.max_batch -= self.trained_batch + 1
            msg += '%d batches ' % estimator.max_batch
        files = [os.path.join(self.model_dir, newest + ext) for ext in ('.params', '.states')]
        for path in files:
            if not os.path.exists(path):
                raise AssertionError('Failed to load checkpoint, %s does not exist' % path)
        estimator.net.load_parameters(files[0], ctx=estimator.device)
        estimator.trainer.load_states(files[1])
        estimator.logger.warning(msg)


class EarlyStoppingHandler(TrainBegin, EpochEnd, TrainEnd):
    """Stops training when ``monitor`` has not improved by more than ``min_delta`` for ``patience`` epochs in a row
    (``baseline``: the value to beat from the start)."""

    def __init__(self, monitor, min_delta=0, patience=0, mode='auto', baseline=None):
        if not isinstance(monitor, EvalMetric):
            raise ValueError('Please provide one of the metric objects from estimator.train_metrics and '
                             'estimator.val_metrics as monitor.')
        if isinstance(monitor, CompositeEvalMetric):
            raise ValueError('CompositeEvalMetric is not supported for EarlyStoppingHandler, please specify a simple '
                             'metric instead.')
        self.monitor = monitor
        self.baseline = baseline
        self.patience = patience
        self.monitor_op, self._worst = _improvement_rule(mode, monitor, 'EarlyStopping')
        # the margin always points in the direction of "better"
        self.min_delta = min_delta if self.monitor_op is np.greater else -min_delta
        self.train_begin(None)

    def train_begin(self, estimator, *args, **kwargs):
        self.wait = 0
        self.stopped_epoch = 0
        self.current_epoch = 0
        self.stop_training = False
        self.best = self._worst if self.baseline is None else self.baseline

    def epoch_end(self, estimator, *args, **kwargs):
        name, value = self.monitor.get()
        if np.isnan(value):
            warnings.warn(RuntimeWarning('%s is not updated, make sure you pass one of the metric objects from '
                                         'estimator.train_metrics and estimator.val_metrics as monitor.' % name))
        elif self.monitor_op(value - self.min_delta, self.best):
            self.best = value
            self.wait = 0
        else:
            self.wait += 1
            if self.wait >= self.patience:
                self.stopped_epoch = self.current_epoch
                self.stop_training = True
        self.current_epoch += 1
        return self.stop_training

    def train_end(self, estimator, *args, **kwargs):
        if self.stopped_epoch > 0:
            estimator.logger.info('[Epoch %d] EarlyStoppingHanlder: early stopping due to %s not improving',
                                  self.stopped_epoch, self.monitor.get()[0])


class GradientUpdateHandler(BatchEnd):
    """Calls ``trainer.step`` with the number of samples of the batch (summed over the per-device losses).  Runs before
    the metric handlers (priority -2000)."""

    def __init__(self, priority=-2000):
        self.priority = priority

    def batch_end(self, estimator, *args, **kwargs):
        losses = _as_list(kwargs['loss'])
        estimator.trainer.step(sum(l.shape[0] for l in losses))

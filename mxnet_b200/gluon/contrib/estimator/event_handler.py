"""Estimator event handlers (``event_handler.py``): stopping, metrics, validation, logging,
checkpointing (periodic, best-model tracking, resume, ``max_checkpoints``), early stopping, gradient update."""
import logging
import os
import time
import warnings

import numpy as np

from ...metric import EvalMetric, Loss as LossMetric, CompositeEvalMetric

__all__ = ['TrainBegin', 'TrainEnd', 'EpochBegin', 'EpochEnd', 'BatchBegin', 'BatchEnd', 'StoppingHandler',
           'MetricHandler', 'ValidationHandler', 'LoggingHandler', 'CheckpointHandler', 'EarlyStoppingHandler',
           'GradientUpdateHandler']


class EventHandler(object):
    pass


def _check_event_handlers(handlers):
    if isinstance(handlers, EventHandler):
        handlers = [handlers]
    else:
        handlers = handlers or []
        if not all(isinstance(h, EventHandler) for h in handlers):
            raise ValueError('handlers must be an EventHandler or a list of EventHandler, got: {}'.format(handlers))
    return handlers


class TrainBegin(EventHandler):
    def train_begin(self, estimator, *args, **kwargs): pass


class TrainEnd(EventHandler):
    def train_end(self, estimator, *args, **kwargs): pass


class EpochBegin(EventHandler):
    def epoch_begin(self, estimator, *args, **kwargs): pass


class EpochEnd(EventHandler):
    def epoch_end(self, estimator, *args, **kwargs): return False


class BatchBegin(EventHandler):
    def batch_begin(self, estimator, *args, **kwargs): pass


class BatchEnd(EventHandler):
    def batch_end(self, estimator, *args, **kwargs): return False


class StoppingHandler(TrainBegin, BatchEnd, EpochEnd):
    def __init__(self, max_epoch=None, max_batch=None):
        self.max_epoch, self.max_batch = max_epoch, max_batch
        self.current_batch = self.current_epoch = 0
        self.stop_training = False

    def train_begin(self, estimator, *args, **kwargs):
        self.max_epoch, self.max_batch = estimator.max_epoch, estimator.max_batch
        self.current_batch = self.current_epoch = 0

    def batch_end(self, estimator, *args, **kwargs):
        self.current_batch += 1
        if self.current_batch == self.max_batch:
            self.stop_training = True
        return self.stop_training

    def epoch_end(self, estimator, *args, **kwargs):
        self.current_epoch += 1
        if self.current_epoch == self.max_epoch:
            self.stop_training = True
        return self.stop_training


class MetricHandler(EpochBegin, BatchEnd):
    def __init__(self, metrics, priority=-1000):
        self.metrics = list(metrics) if isinstance(metrics, (list, tuple)) else [metrics]
        self.priority = priority

    def epoch_begin(self, estimator, *args, **kwargs):
        for metric in self.metrics:
            metric.reset()

    def batch_end(self, estimator, *args, **kwargs):
        pred, label, loss = kwargs['pred'], kwargs['label'], kwargs['loss']
        for metric in self.metrics:
            if isinstance(metric, LossMetric):
                metric.update(0, loss)
            else:
                metric.update(label, pred)


class ValidationHandler(TrainBegin, BatchEnd, EpochEnd):
    def __init__(self, val_data, eval_fn, epoch_period=1, batch_period=None, priority=-1000, event_handlers=None):
        self.val_data, self.eval_fn = val_data, eval_fn
        self.epoch_period, self.batch_period = epoch_period, batch_period
        self.current_batch = self.current_epoch = 0
        self.priority = priority
        self.event_handlers = event_handlers

    def train_begin(self, estimator, *args, **kwargs):
        self.current_batch = self.current_epoch = 0

    def batch_end(self, estimator, *args, **kwargs):
        self.current_batch += 1
        if self.batch_period and self.current_batch % self.batch_period == 0:
            self.eval_fn(val_data=self.val_data, batch_axis=estimator.batch_axis, event_handlers=self.event_handlers)

    def epoch_end(self, estimator, *args, **kwargs):
        self.current_epoch += 1
        if self.epoch_period and self.current_epoch % self.epoch_period == 0:
            self.eval_fn(val_data=self.val_data, batch_axis=estimator.batch_axis, event_handlers=self.event_handlers)


class LoggingHandler(TrainBegin, TrainEnd, EpochBegin, EpochEnd, BatchBegin, BatchEnd):
    def __init__(self, log_interval='epoch', metrics=None, priority=np.inf):
        if not isinstance(log_interval, int) and log_interval != 'epoch':
            raise ValueError("log_interval must be either an integer or string 'epoch'")
        self.metrics = list(metrics) if isinstance(metrics, (list, tuple)) else ([metrics] if metrics else [])
        self.batch_index = self.current_epoch = self.processed_samples = 0
        self.priority = priority
        self.log_interval = log_interval
        self.log_interval_time = 0

    def train_begin(self, estimator, *args, **kwargs):
        self.train_start = time.time()
        estimator.logger.info('Training begin: using optimizer %s with current learning rate %.4f ',
                              estimator.trainer.optimizer.__class__.__name__, estimator.trainer.learning_rate)
        if estimator.max_epoch:
            estimator.logger.info('Train for %d epochs.', estimator.max_epoch)
        else:
            estimator.logger.info('Train for %d batches.', estimator.max_batch)
        self.current_epoch = self.batch_index = 0

    def train_end(self, estimator, *args, **kwargs):
        train_time = time.time() - self.train_start
        msg = 'Train finished using total %ds with %d epochs. ' % (train_time, self.current_epoch)
        for metric in self.metrics:
            name, value = metric.get()
            msg += '%s: %.4f, ' % (name, value)
        estimator.logger.info(msg.rstrip(', '))

    def batch_begin(self, estimator, *args, **kwargs):
        if isinstance(self.log_interval, int):
            self.batch_start = time.time()

    def batch_end(self, estimator, *args, **kwargs):
        if isinstance(self.log_interval, int):
            batch_time = time.time() - self.batch_start
            msg = '[Epoch %d][Batch %d]' % (self.current_epoch, self.batch_index)
            self.processed_samples += kwargs['batch'][0].shape[0]
            msg += '[Samples %s] ' % (self.processed_samples)
            self.log_interval_time += batch_time
            if self.batch_index % self.log_interval == 0:
                msg += 'time/interval: %.3fs ' % self.log_interval_time
                self.log_interval_time = 0
                for metric in self.metrics:
                    name, value = metric.get()
                    msg += '%s: %.4f, ' % (name, value)
                estimator.logger.info(msg.rstrip(', '))
        self.batch_index += 1

    def epoch_begin(self, estimator, *args, **kwargs):
        if isinstance(self.log_interval, int) or self.log_interval == 'epoch':
            self.epoch_start = time.time()
            estimator.logger.info('[Epoch %d] Begin, current learning rate: %.4f', self.current_epoch, estimator.trainer.learning_rate)

    def epoch_end(self, estimator, *args, **kwargs):
        if isinstance(self.log_interval, int) or self.log_interval == 'epoch':
            epoch_time = time.time() - self.epoch_start
            msg = '[Epoch %d] Finished in %.3fs, ' % (self.current_epoch, epoch_time)
            for monitor in self.metrics:
                name, value = monitor.get()
                msg += '%s: %.4f, ' % (name, value)
            estimator.logger.info(msg.rstrip(', '))
        self.current_epoch += 1
        self.batch_index = 0


class CheckpointHandler(TrainBegin, BatchEnd, EpochEnd):
    """Save parameters and trainer states periodically; keep the best model according to ``monitor``;
    prune to ``max_checkpoints``; optionally resume from the latest checkpoint in ``model_dir``
    (``event_handler.py:336-620``)."""

    def __init__(self, model_dir, model_prefix='model', monitor=None, verbose=0, save_best=False, mode='auto',
                 epoch_period=1, batch_period=None, max_checkpoints=5, resume_from_checkpoint=False):
        self.monitor, self.verbose = monitor, verbose
        os.makedirs(model_dir, exist_ok=True)
        self.model_dir, self.model_prefix, self.save_best = model_dir, model_prefix, save_best
        if self.save_best and not isinstance(self.monitor, EvalMetric):
            raise ValueError('To save best model only, please provide one of the metric objects from estimator.train_metrics '
                             'and estimator.val_metrics as monitor.')
        self.epoch_period, self.batch_period = epoch_period, batch_period
        self.current_batch = self.current_epoch = 0
        self.max_checkpoints, self.resume_from_checkpoint = max_checkpoints, resume_from_checkpoint
        self.saved_checkpoints = []
        if self.save_best:
            if mode not in ['auto', 'min', 'max']:
                warnings.warn('ModelCheckpoint mode %s is unknown, fallback to auto mode. ' % mode, RuntimeWarning)
                mode = 'auto'
            if mode == 'min':
                self.monitor_op, self.best = np.less, np.inf
            elif mode == 'max':
                self.monitor_op, self.best = np.greater, -np.inf
            else:
                if 'acc' in self.monitor.get()[0].lower() or 'f1' in self.monitor.get()[0].lower():
                    self.monitor_op, self.best = np.greater, -np.inf
                else:
                    self.monitor_op, self.best = np.less, np.inf

    def train_begin(self, estimator, *args, **kwargs):
        self.current_epoch = self.current_batch = 0
        if self.save_best:
            self.best = np.inf if self.monitor_op == np.less else -np.inf
        if self.resume_from_checkpoint:
            error_msg = 'To use resume from checkpoint, you must only specify the same type of period you used for training.'
            if estimator.max_batch:
                assert self.batch_period, error_msg
                assert not self.epoch_period, error_msg
            if estimator.max_epoch:
                assert self.epoch_period, error_msg
                assert not self.batch_period, error_msg
            self._resume_from_checkpoint(estimator)

    def batch_end(self, estimator, *args, **kwargs):
        if self.current_batch == 0:
            self._save_symbol(estimator)
        if self.batch_period and (self.current_batch + 1) % self.batch_period == 0:
            self._save_checkpoint(estimator)
        self.current_batch += 1

    def epoch_end(self, estimator, *args, **kwargs):
        if self.epoch_period and (self.current_epoch + 1) % self.epoch_period == 0:
            self._save_checkpoint(estimator)
        self.current_epoch += 1

    def _save_checkpoint(self, estimator):
        if self.resume_from_checkpoint:
            save_epoch_number = self.current_epoch + self.trained_epoch + 1
            save_batch_number = self.current_batch + self.trained_batch + 1 if estimator.max_epoch else self.current_batch + self.trained_batch
        else:
            save_epoch_number, save_batch_number = self.current_epoch, self.current_batch
        prefix = '%s-epoch%dbatch%d' % (self.model_prefix, save_epoch_number, save_batch_number)
        self._save_params_and_trainer(estimator, prefix)
        if self.verbose > 0:
            estimator.logger.info('[Epoch %d] CheckpointHandler: trained total %d batches, saving model at %s with prefix: %s',
                                  self.current_epoch, self.current_batch + 1, self.model_dir, prefix)
        if self.save_best:
            monitor_name, monitor_value = self.monitor.get()
            if np.isnan(monitor_value):
                warnings.warn(RuntimeWarning('Skipping save best because %s is not updated, make sure you pass one of the '
                                             'metric objects estimator.train_metrics and estimator.val_metrics as monitor' % monitor_name))
            elif self.monitor_op(monitor_value, self.best):
                prefix = self.model_prefix + '-best'
                self._save_params_and_trainer(estimator, prefix)
                self.best = monitor_value

    def _save_symbol(self, estimator):
        symbol_file = os.path.join(self.model_dir, self.model_prefix + '-symbol.json')
        net = estimator.net
        if hasattr(net, '_cached_graph') and net._cached_graph:
            net._cached_graph[1].save(symbol_file)

    def _save_params_and_trainer(self, estimator, file_prefix):
        param_file = os.path.join(self.model_dir, file_prefix + '.params')
        trainer_file = os.path.join(self.model_dir, file_prefix + '.states')
        estimator.net.save_parameters(param_file)
        estimator.trainer.save_states(trainer_file)
        if 'best' not in file_prefix:
            self.saved_checkpoints.append(file_prefix)
        if len(self.saved_checkpoints) > self.max_checkpoints:
            prefix = self.saved_checkpoints.pop(0)
            for fname in os.listdir(self.model_dir):
                if fname.startswith(prefix + '.'):
                    os.remove(os.path.join(self.model_dir, fname))

    def _resume_from_checkpoint(self, estimator):
        prefix = self.model_prefix + '-epoch'
        self.trained_epoch = self._find_max_iteration(dir=self.model_dir, prefix=prefix, start='epoch', end='batch', saved_checkpoints=self.saved_checkpoints)
        prefix += str(self.trained_epoch)
        self.trained_batch = self._find_max_iteration(dir=self.model_dir, prefix=prefix, start='batch', end='.params')
        if self.trained_epoch == -1:
            msg = 'CheckpointHandler: No checkpoint found, training from scratch for '
            if estimator.max_batch:
                msg += '%d batches' % estimator.max_batch
            else:
                msg += '%d epochs' % estimator.max_epoch
            estimator.logger.info(msg)
        else:
            msg = 'CheckpointHandler: Checkpoint resumed from epoch %d batch %d, continue to train for ' % (self.trained_epoch, self.trained_batch)
            if estimator.max_epoch:
                if self.trained_epoch >= estimator.max_epoch - 1:
                    raise ValueError('Found checkpoint with maximum number of epoch %d reached, please specify resume_from_checkpoint=False '
                                     '(default value) if you wan to train from scratch.' % estimator.max_epoch)
                estimator.max_epoch = estimator.max_epoch - self.trained_epoch - 1
                msg += '%d epochs ' % estimator.max_epoch
            if estimator.max_batch:
                if self.trained_batch >= estimator.max_batch - 1:
                    raise ValueError('Found checkpoint with maximum number of batch %d reached, please specify resume_from_checkpoint=False '
                                     '(default value) if you wan to train from scratch.' % self.trained_batch)
                estimator.max_batch = estimator.max_batch - self.trained_batch - 1
                msg += '%d batches ' % estimator.max_batch
            param_file = '%s-epoch%dbatch%d.params' % (self.model_prefix, self.trained_epoch, self.trained_batch)
            param_file = os.path.join(self.model_dir, param_file)
            trainer_file = '%s-epoch%dbatch%d.states' % (self.model_prefix, self.trained_epoch, self.trained_batch)
            trainer_file = os.path.join(self.model_dir, trainer_file)
            assert os.path.exists(param_file), 'Failed to load checkpoint, %s does not exist' % param_file
            assert os.path.exists(trainer_file), 'Failed to load checkpoint, %s does not exist' % trainer_file
            estimator.net.load_parameters(param_file, ctx=estimator.device)
            estimator.trainer.load_states(trainer_file)
            estimator.logger.warning(msg)

    def _find_max_iteration(self, dir, prefix, start, end, saved_checkpoints=None):  # pylint: disable=redefined-builtin
        error_msg = 'Error parsing checkpoint file, please check your checkpoints have the format: ' \
                    '{model_name}-epoch{epoch_number}batch{batch_number}.params, there should also be a .states file for each .params file '
        max_iter = -1
        for fname in os.listdir(dir):
            if fname.startswith(prefix) and '.params' in fname:
                if saved_checkpoints:
                    saved_checkpoints.append(fname[:fname.find('.params')])
                try:
                    iter_num = int(fname[fname.find(start) + len(start):fname.find(end)])
                    if iter_num > max_iter:
                        max_iter = iter_num
                except ValueError:
                    raise ValueError(error_msg)
        return max_iter


class EarlyStoppingHandler(TrainBegin, EpochEnd, TrainEnd):
    def __init__(self, monitor, min_delta=0, patience=0, mode='auto', baseline=None):
        if not isinstance(monitor, EvalMetric):
            raise ValueError('Please provide one of the metric objects from estimator.train_metrics and estimator.val_metrics as monitor.')
        if isinstance(monitor, CompositeEvalMetric):
            raise ValueError('CompositeEvalMetric is not supported for EarlyStoppingHandler, please specify a simple metric instead.')
        self.monitor, self.baseline, self.patience, self.min_delta = monitor, baseline, patience, min_delta
        self.wait = self.stopped_epoch = self.current_epoch = 0
        self.stop_training = False
        if mode not in ['auto', 'min', 'max']:
            warnings.warn('EarlyStopping mode %s is unknown, fallback to auto mode. ' % mode, RuntimeWarning)
            mode = 'auto'
        if mode == 'min':
            self.monitor_op = np.less
        elif mode == 'max':
            self.monitor_op = np.greater
        else:
            self.monitor_op = np.greater if ('acc' in self.monitor.get()[0].lower() or 'f1' in self.monitor.get()[0].lower()) else np.less
        self.min_delta *= 1 if self.monitor_op == np.greater else -1

    def train_begin(self, estimator, *args, **kwargs):
        self.wait = self.stopped_epoch = self.current_epoch = 0
        self.stop_training = False
        self.best = self.baseline if self.baseline is not None else (np.inf if self.monitor_op == np.less else -np.inf)

    def epoch_end(self, estimator, *args, **kwargs):
        monitor_name, monitor_value = self.monitor.get()
        if np.isnan(monitor_value):
            warnings.warn(RuntimeWarning('%s is not updated, make sure you pass one of the metric objects from '
                                         'estimator.train_metrics and estimator.val_metrics as monitor.' % monitor_name))
        else:
            if self.monitor_op(monitor_value - self.min_delta, self.best):
                self.best = monitor_value
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
    def __init__(self, priority=-2000):
        self.priority = priority

    def batch_end(self, estimator, *args, **kwargs):
        loss = kwargs['loss']
        batch_size = 0
        if not isinstance(loss, list):
            loss = [loss]
        if isinstance(loss, list):
            for l in loss:
                batch_size += l.shape[0]
        estimator.trainer.step(batch_size)

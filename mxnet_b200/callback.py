"""Batch-end and epoch-end callbacks for the legacy training loops (API of ``python/mxnet/callback.py``).

A batch-end callback receives a ``BatchEndParam`` (``epoch``, ``nbatch``, ``eval_metric``, ``locals``); an epoch-end
callback receives ``(epoch, symbol, arg_params, aux_params)``.  The text of the log lines is part of the contract:
``tools/parse_log.py`` (and users' own scripts) read throughput and metric values back out of them.
"""
import logging
import math
import time

from .model import save_checkpoint   # noqa: F401  (re-exported as in python/mxnet/callback.py)

__all__ = ['do_checkpoint', 'module_checkpoint', 'log_train_metric', 'Speedometer', 'ProgressBar',
           'LogValidationMetricsCallback']


def _every(period):
    """Predicate "this is the last epoch of a period" over zero-based epoch numbers."""
    period = max(1, int(period))
    return lambda epoch: (epoch + 1) % period == 0


def _metric_pairs(metric):
    return list(metric.get_name_value()) if metric is not None else []


def do_checkpoint(prefix, period=1):
    """Epoch-end callback that writes ``prefix-symbol.json`` and ``prefix-NNNN.params`` every ``period`` epochs."""
    due = _every(period)

    def _callback(iter_no, sym, arg, aux):
        if due(iter_no):
            from .model import save_checkpoint
            save_checkpoint(prefix, iter_no + 1, sym, arg, aux)
    return _callback


def module_checkpoint(mod, prefix, period=1, save_optimizer_states=False):
    """The same through ``mod.save_checkpoint`` (which can also keep the optimizer states)."""
    due = _every(period)

    def _callback(iter_no, sym=None, arg=None, aux=None):
        if due(iter_no):
            mod.save_checkpoint(prefix, iter_no + 1, save_optimizer_states)
    return _callback


def log_train_metric(period, auto_reset=False):
    """Batch-end callback that logs the training metric every ``period`` batches."""
    def _callback(param):
        if param.eval_metric is None or param.nbatch % period:
            return
        for name, value in _metric_pairs(param.eval_metric):
            logging.info('Iter[%d] Batch[%d] Train-%s=%f', param.epoch, param.nbatch, name, value)
        if auto_reset:
            param.eval_metric.reset()
    return _callback


class Speedometer(object):
    """Logs samples per second, and the metric if there is one, every ``frequent`` batches.

    The clock starts at the first batch seen (and restarts when the batch counter goes backwards, i.e. a new epoch), so
    the first report covers ``frequent`` full batches.  With ``auto_reset`` the metric is cleared after each report and
    the line names the batch window it covers; without it the line covers the epoch so far."""

    def __init__(self, batch_size, frequent=50, auto_reset=True):
        self.batch_size = batch_size
        self.frequent = frequent
        self.auto_reset = auto_reset
        self.init = False
        self.tic = 0
        self.last_count = 0

    def _report(self, param, speed):
        count = param.nbatch
        pairs = _metric_pairs(param.eval_metric)
        if param.eval_metric is None:
            logging.info('Iter[%d] Batch [%d]\tSpeed: %.2f samples/sec', param.epoch, count, speed)
            return
        tail = ''.join('\t%s=%f' % (name, value) for name, value in pairs)
        if self.auto_reset:
            param.eval_metric.reset()
            window = '%d-%d' % (count - self.frequent, count)
        else:
            window = '0-%d' % count
        logging.info('Epoch[%d] Batch [%s]\tSpeed: %.2f samples/sec%s', param.epoch, window, speed, tail)

    def __call__(self, param):
        count = param.nbatch
        restarted = count < self.last_count
        self.last_count = count
        if restarted or not self.init:
            self.init = True
            self.tic = time.time()
            return
        if count % self.frequent:
            return
        elapsed = time.time() - self.tic
        speed = self.frequent * self.batch_size / elapsed if elapsed > 0 else float('inf')
        self._report(param, speed)
        self.tic = time.time()


class ProgressBar(object):
    """Logs a text progress bar of ``length`` characters for ``total`` batches."""

    def __init__(self, total, length=80):
        self.bar_len = length
        self.total = total

    def __call__(self, param):
        done = param.nbatch / float(self.total)
        filled = int(round(self.bar_len * done))
        bar = '=' * filled + '-' * (self.bar_len - filled)
        logging.info('[%s] %s%s\r', bar, math.ceil(100.0 * done), '%')


class LogValidationMetricsCallback(object):
    """Epoch-end evaluation callback: one line per validation metric."""

    def __call__(self, param):
        for name, value in _metric_pairs(param.eval_metric or None):
            logging.info('Epoch[%d] Validation-%s=%f', param.epoch, name, value)

"""``Estimator``: fit/evaluate driver with event handlers (``estimator.py``)."""
import copy
import logging
import sys
import warnings

from .... import device as _device
from ...loss import Loss as gluon_loss
from ...metric import Loss as metric_loss, EvalMetric
from ...trainer import Trainer
from .batch_processor import BatchProcessor
from .event_handler import (MetricHandler, ValidationHandler, LoggingHandler, StoppingHandler, GradientUpdateHandler,
                            TrainBegin, EpochBegin, BatchBegin, BatchEnd, EpochEnd, TrainEnd, _check_event_handlers)

__all__ = ['Estimator']


class Estimator(object):
    logger = None

    def __init__(self, net, loss, train_metrics=None, val_metrics=None, initializer=None, trainer=None, device=None,
                 val_net=None, val_loss=None, batch_processor=None, context=None):
        self.net = net
        self.loss = self._check_loss(loss)
        self._train_metrics = self._check_metrics(train_metrics)
        self._val_metrics = self._check_metrics(val_metrics)
        self._add_default_training_metrics()
        self._add_validation_metrics()
        self.val_loss = self.loss if val_loss is None else self._check_loss(val_loss)
        self.val_net = self.net if val_net is None else val_net
        self.logger = logging.Logger(name='Estimator', level=logging.INFO)
        self.logger.addHandler(logging.StreamHandler(sys.stdout))
        self.device = self._check_devices(device if device is not None else context)
        self._initialize(initializer)
        self.trainer = self._check_trainer(trainer)
        self.batch_processor = self._check_batch_processor(batch_processor)
        self.max_epoch = self.max_batch = None
        self.batch_axis = 0

    context = property(lambda self: self.device)

    def _check_loss(self, loss):
        if not isinstance(loss, gluon_loss):
            raise ValueError('loss must be a Loss, refer to gluon.loss.Loss:{}'.format(loss))
        return loss

    def _check_devices(self, device):
        if device is None:
            device = [_device.gpu(0)] if _device.num_gpus() > 0 else [_device.cpu()]
        elif isinstance(device, _device.Device):
            device = [device]
        return device

    def _check_batch_processor(self, batch_processor):
        if batch_processor is not None:
            model_fit = getattr(batch_processor, 'fit_batch', None)
            model_evaluate = getattr(batch_processor, 'evaluate_batch', None)
            if not callable(model_fit) or not callable(model_evaluate):
                raise ValueError('Customized Batch Processor must contain fit_batch() and evaluate_batch() methods')
            return batch_processor
        return BatchProcessor()

    def _check_metrics(self, metrics):
        if isinstance(metrics, EvalMetric):
            metrics = [metrics]
        else:
            metrics = metrics or []
            if not all(isinstance(m, EvalMetric) for m in metrics):
                raise ValueError('metrics must be a Metric or a list of Metric, refer to gluon.metric.EvalMetric: {}'.format(metrics))
        return metrics

    def _initialize(self, initializer):
        from .... import initializer as init_mod
        uninit = any(p._data is None and not p._deferred_init for p in self.net.collect_params().values())
        if uninit or initializer is not None:
            try:
                self.net.initialize(init=initializer or init_mod.Uniform(), device=self.device,
                                    force_reinit=initializer is not None)
            except Exception:  # pylint: disable=broad-except
                pass

    def _check_trainer(self, trainer):
        if not trainer:
            warnings.warn('No trainer specified, default SGD optimizer with learning rate 0.001 is used.')
            trainer = Trainer(self.net.collect_params(), 'sgd', {'learning_rate': 0.001})
        elif not isinstance(trainer, Trainer):
            raise ValueError('Trainer must be a Gluon Trainer instance, refer to gluon.Trainer:{}'.format(trainer))
        return trainer

    def _add_default_training_metrics(self):
        if not self._train_metrics:
            self._train_metrics = []
        for metric in self._train_metrics:
            metric.name = 'training ' + metric.name
        self._train_metrics.append(metric_loss('training ' + type(self.loss).__name__.lower()))

    def _add_validation_metrics(self):
        if not self._val_metrics:
            self._val_metrics = [copy.deepcopy(m) for m in self._train_metrics]
        for metric in self._val_metrics:
            metric.name = metric.name.replace('training', 'validation') if 'training' in metric.name else 'validation ' + metric.name

    @property
    def train_metrics(self):
        return self._train_metrics

    @property
    def val_metrics(self):
        return self._val_metrics

    def evaluate(self, val_data, batch_axis=0, event_handlers=None):
        for metric in self.val_metrics:
            metric.reset()
        for batch in val_data:
            _, label, pred, loss = self.batch_processor.evaluate_batch(self, batch, batch_axis)
            for metric in self.val_metrics:
                if isinstance(metric, metric_loss):
                    metric.update(0, loss)
                else:
                    metric.update(label, pred)

    def fit(self, train_data, val_data=None, epochs=None, event_handlers=None, batches=None, batch_axis=0):
        if not (epochs is None) ^ (batches is None):
            raise ValueError('Fit only supports exactly one type of limit; only one of epochs or batches can be specified.')
        self.max_epoch, self.max_batch, self.batch_axis = epochs, batches, batch_axis
        handlers = self._prepare_default_handlers(val_data, _check_event_handlers(event_handlers))
        train_begin, epoch_begin, batch_begin, batch_end, epoch_end, train_end = self._categorize_handlers(handlers)
        for h in train_begin:
            h.train_begin(self)
        stop = False
        while not stop:
            for h in epoch_begin:
                h.epoch_begin(self)
            for batch in train_data:
                for h in batch_begin:
                    h.batch_begin(self, batch=batch)
                _, label, pred, loss = self.batch_processor.fit_batch(self, batch, batch_axis)
                for h in batch_end:
                    if h.batch_end(self, batch=batch, pred=pred, label=label, loss=loss):
                        stop = True
                if stop:
                    break
            for h in epoch_end:
                if h.epoch_end(self):
                    stop = True
        for h in train_end:
            h.train_end(self)

    def _prepare_default_handlers(self, val_data, event_handlers):
        event_handlers = list(event_handlers)
        added = [StoppingHandler(self.max_epoch, self.max_batch)]
        if not any(isinstance(h, GradientUpdateHandler) for h in event_handlers):
            added.append(GradientUpdateHandler())
        if not any(isinstance(h, MetricHandler) for h in event_handlers):
            added.append(MetricHandler(metrics=self.train_metrics))
        if val_data is not None and not any(isinstance(h, ValidationHandler) for h in event_handlers):
            added.append(ValidationHandler(val_data=val_data, eval_fn=self.evaluate))
        if not any(isinstance(h, LoggingHandler) for h in event_handlers):
            added.append(LoggingHandler(metrics=self.train_metrics + (self.val_metrics if val_data is not None else [])))
        event_handlers.extend(added)
        event_handlers.sort(key=lambda h: getattr(h, 'priority', 0))
        return event_handlers

    def _categorize_handlers(self, event_handlers):
        cats = [[], [], [], [], [], []]
        for h in event_handlers:
            for i, cls in enumerate((TrainBegin, EpochBegin, BatchBegin, BatchEnd, EpochEnd, TrainEnd)):
                if isinstance(h, cls):
                    cats[i].append(h)
        return cats

"""Evaluation metrics (``python/mxnet/gluon/metric.py``): ``update(labels, preds)`` / ``get()`` /
``reset()`` with the registry/``create`` factory and ``CompositeEvalMetric``."""
import math
from collections import OrderedDict

import numpy

from .. import registry
from ..ndarray.ndarray import NDArray

__all__ = ['EvalMetric', 'CompositeEvalMetric', 'check_label_shapes', 'create', 'Accuracy', 'TopKAccuracy', 'F1',
           'Fbeta', 'BinaryAccuracy', 'MCC', 'Perplexity', 'MAE', 'MSE', 'RMSE', 'MeanPairwiseDistance',
           'MeanCosineSimilarity', 'CrossEntropy', 'PearsonCorrelation', 'PCC', 'Loss', 'CustomMetric', 'np',
           'register', 'alias']


def check_label_shapes(labels, preds, wrap=False, shape=False):
    if not shape:
        label_shape, pred_shape = len(labels), len(preds)
    else:
        label_shape, pred_shape = labels.shape, preds.shape
    if label_shape != pred_shape:
        raise ValueError('Shape of labels {} does not match shape of predictions {}'.format(label_shape, pred_shape))
    if wrap:
        if isinstance(labels, NDArray):
            labels = [labels]
        if isinstance(preds, NDArray):
            preds = [preds]
    return labels, preds


def _np(x):
    return x.asnumpy() if isinstance(x, NDArray) else numpy.asarray(x)


class EvalMetric(object):
    def __init__(self, name, output_names=None, label_names=None, **kwargs):
        self.name = str(name)
        self.output_names, self.label_names = output_names, label_names
        self._kwargs = kwargs
        self.reset()

    def __str__(self):
        return 'EvalMetric: {}'.format(dict(self.get_name_value()))

    def get_config(self):
        config = self._kwargs.copy()
        config.update({'metric': self.__class__.__name__, 'name': self.name, 'output_names': self.output_names,
                       'label_names': self.label_names})
        return config

    def update_dict(self, label, pred):
        pred = [pred[n] for n in self.output_names] if self.output_names is not None else list(pred.values())
        label = [label[n] for n in self.label_names] if self.label_names is not None else list(label.values())
        self.update(label, pred)

    def update(self, labels, preds):
        raise NotImplementedError()

    def reset(self):
        self.num_inst = 0
        self.sum_metric = 0.0

    def get(self):
        if self.num_inst == 0:
            return (self.name, float('nan'))
        return (self.name, self.sum_metric / self.num_inst)

    def get_name_value(self):
        name, value = self.get()
        if not isinstance(name, list):
            name = [name]
        if not isinstance(value, list):
            value = [value]
        return list(zip(name, value))


register = registry.get_register_func(EvalMetric, 'metric')
alias = registry.get_alias_func(EvalMetric, 'metric')
_create = registry.get_create_func(EvalMetric, 'metric')


def create(metric, *args, **kwargs):
    if callable(metric):
        return CustomMetric(metric, *args, **kwargs)
    if isinstance(metric, list):
        composite = CompositeEvalMetric()
        for child in metric:
            composite.add(create(child, *args, **kwargs))
        return composite
    return _create(metric, *args, **kwargs)


@register
@alias('composite')
class CompositeEvalMetric(EvalMetric):
    def __init__(self, metrics=None, name='composite', output_names=None, label_names=None):
        super().__init__(name, output_names=output_names, label_names=label_names)
        self.metrics = [create(i) for i in (metrics or [])]

    def add(self, metric):
        self.metrics.append(create(metric))

    def get_metric(self, index):
        try:
            return self.metrics[index]
        except IndexError:
            return ValueError('Metric index {} is out of range 0 and {}'.format(index, len(self.metrics)))

    def update_dict(self, labels, preds):
        if self.label_names is not None:
            labels = OrderedDict([i for i in labels.items() if i[0] in self.label_names])
        if self.output_names is not None:
            preds = OrderedDict([i for i in preds.items() if i[0] in self.output_names])
        for metric in self.metrics:
            metric.update_dict(labels, preds)

    def update(self, labels, preds):
        for metric in self.metrics:
            metric.update(labels, preds)

    def reset(self):
        for metric in getattr(self, 'metrics', []):
            metric.reset()

    def get(self):
        names, values = [], []
        for metric in self.metrics:
            name, value = metric.get()
            names.extend(name if isinstance(name, list) else [name])
            values.extend(value if isinstance(value, list) else [value])
        return (names, values)

    def get_config(self):
        config = super().get_config()
        config.update({'metrics': [i.get_config() for i in self.metrics]})
        return config


@register
@alias('acc')
class Accuracy(EvalMetric):
    def __init__(self, axis=1, name='accuracy', output_names=None, label_names=None):
        super().__init__(name, axis=axis, output_names=output_names, label_names=label_names)
        self.axis = axis

    def update(self, labels, preds):
        labels, preds = check_label_shapes(labels, preds, True)
        for label, pred_label in zip(labels, preds):
            pred_label, label = _np(pred_label), _np(label)
            if pred_label.shape != label.shape:
                pred_label = numpy.argmax(pred_label, axis=self.axis)
            pred_label = pred_label.astype('int32').reshape(-1)
            label = label.astype('int32').reshape(-1)
            check_label_shapes(label, pred_label)
            self.sum_metric += float((pred_label == label).sum())
            self.num_inst += len(pred_label)


@register
@alias('top_k_accuracy', 'top_k_acc')
class TopKAccuracy(EvalMetric):
    def __init__(self, top_k=1, name='top_k_accuracy', output_names=None, label_names=None):
        super().__init__(name, top_k=top_k, output_names=output_names, label_names=label_names)
        self.top_k = top_k
        assert self.top_k > 1, 'Please use Accuracy if top_k is no more than 1'
        self.name += '_%d' % self.top_k

    def update(self, labels, preds):
        labels, preds = check_label_shapes(labels, preds, True)
        for label, pred_label in zip(labels, preds):
            assert len(pred_label.shape) <= 2, 'Predictions should be no more than 2 dims'
            pred_label = numpy.argpartition(_np(pred_label).astype('float32'), -self.top_k)
            label = _np(label).astype('int32')
            check_label_shapes(label, pred_label)
            num_samples = pred_label.shape[0]
            num_dims = len(pred_label.shape)
            if num_dims == 1:
                self.sum_metric += float((pred_label.reshape(-1) == label.reshape(-1)).sum())
            elif num_dims == 2:
                num_classes = pred_label.shape[1]
                top_k = min(num_classes, self.top_k)
                for j in range(top_k):
                    self.sum_metric += float((pred_label[:, num_classes - 1 - j].reshape(-1) == label.reshape(-1)).sum())
            self.num_inst += num_samples


class _ClassificationMetrics(object):
    def __init__(self, class_type='binary', threshold=0.5, beta=1):
        self.class_type, self.threshold, self.beta = class_type, threshold, beta
        self.reset_stats()

    def _set(self, num):
        if self.num_classes is None:
            self.num_classes = num
            self.true_positives = numpy.zeros(num)
            self.false_negatives = numpy.zeros(num)
            self.false_positives = numpy.zeros(num)
            self.true_negatives = numpy.zeros(num)

    def update_stats(self, label, pred):
        pred, label = _np(pred).astype('float32'), _np(label).astype('int32')
        if self.class_type == 'binary':
            self._set(1)
            if label.max() > 1:
                raise ValueError('Wrong label for binary classification.')
            if pred.ndim == label.ndim + 1:
                pred = pred[..., 1] if pred.shape[-1] == 2 else pred.reshape(label.shape)
            pred_label = (pred.reshape(label.shape) > self.threshold).astype('int32')
            pred_true, pred_false = pred_label == 1, pred_label == 0
            label_true, label_false = label == 1, label == 0
            self.true_positives += (pred_true & label_true).sum()
            self.false_positives += (pred_true & label_false).sum()
            self.false_negatives += (pred_false & label_true).sum()
            self.true_negatives += (pred_false & label_false).sum()
        elif self.class_type == 'multiclass':
            num = pred.shape[-1]
            self._set(num)
            pred_label = pred.argmax(-1).reshape(-1)
            label = label.reshape(-1)
            for c in range(num):
                self.true_positives[c] += ((pred_label == c) & (label == c)).sum()
                self.false_positives[c] += ((pred_label == c) & (label != c)).sum()
                self.false_negatives[c] += ((pred_label != c) & (label == c)).sum()
                self.true_negatives[c] += ((pred_label != c) & (label != c)).sum()
        else:
            num = pred.shape[-1]
            self._set(num)
            pred_label = (pred > self.threshold).astype('int32')
            self.true_positives += ((pred_label == 1) & (label == 1)).sum(0)
            self.false_positives += ((pred_label == 1) & (label == 0)).sum(0)
            self.false_negatives += ((pred_label == 0) & (label == 1)).sum(0)
            self.true_negatives += ((pred_label == 0) & (label == 0)).sum(0)

    def _div(self, a, b):
        with numpy.errstate(divide='ignore', invalid='ignore'):
            r = numpy.where(b > 0, a / numpy.where(b > 0, b, 1), 0.0)
        return r

    def get_precision(self, average):
        if average == 'micro':
            return float(self._div(self.true_positives.sum(), (self.true_positives + self.false_positives).sum()))
        return float(self._div(self.true_positives, self.true_positives + self.false_positives).mean())

    def get_recall(self, average):
        if average == 'micro':
            return float(self._div(self.true_positives.sum(), (self.true_positives + self.false_negatives).sum()))
        return float(self._div(self.true_positives, self.true_positives + self.false_negatives).mean())

    def get_fscore(self, average):
        b2 = self.beta ** 2
        if average == 'micro':
            p, r = self.get_precision('micro'), self.get_recall('micro')
            return (1 + b2) * p * r / (b2 * p + r) if b2 * p + r > 0 else 0.
        p = self._div(self.true_positives, self.true_positives + self.false_positives)
        r = self._div(self.true_positives, self.true_positives + self.false_negatives)
        return float(self._div((1 + b2) * p * r, b2 * p + r).mean())

    def get_accuracy(self):
        tot = self.true_positives + self.true_negatives + self.false_positives + self.false_negatives
        return float(self._div((self.true_positives + self.true_negatives).sum(), tot.sum()))

    def matthewscc(self):
        tp, tn, fp, fn = (float(x.sum()) for x in (self.true_positives, self.true_negatives, self.false_positives,
                                                   self.false_negatives))
        terms = [(tp + fp), (tp + fn), (tn + fp), (tn + fn)]
        denom = 1.
        for t in terms:
            if t != 0.:
                denom *= t
        return ((tp * tn) - (fp * fn)) / math.sqrt(denom)

    @property
    def total_examples(self):
        if self.num_classes is None:
            return 0
        return int((self.false_negatives[0] + self.false_positives[0] + self.true_negatives[0] + self.true_positives[0]))

    def reset_stats(self):
        self.num_classes = None
        self.true_positives = self.false_negatives = self.false_positives = self.true_negatives = None


@register
class F1(EvalMetric):
    def __init__(self, name='f1', output_names=None, label_names=None, class_type='binary', threshold=0.5,
                 average='micro'):
        self.average = average
        self.metrics = _ClassificationMetrics(class_type=class_type, threshold=threshold, beta=getattr(self, '_beta', 1))
        super().__init__(name=name, output_names=output_names, label_names=label_names)

    def update(self, labels, preds):
        labels, preds = check_label_shapes(labels, preds, True)
        for label, pred in zip(labels, preds):
            self.metrics.update_stats(label, pred)
        # the running score weighted by the number of examples seen, so that sum_metric / num_inst is the score and
        # num_inst counts examples (python/mxnet/gluon/metric.py, F1.update)
        self.sum_metric = self.metrics.get_fscore(self.average) * self.metrics.total_examples
        self.num_inst = self.metrics.total_examples

    def get(self):
        if self.metrics.num_classes is None:
            return (self.name, float('nan'))
        return (self.name, self.metrics.get_fscore(self.average))

    def reset(self):
        self.sum_metric, self.num_inst = 0., 0
        self.metrics.reset_stats()


@register
class Fbeta(F1):
    def __init__(self, name='fbeta', output_names=None, label_names=None, class_type='binary', beta=1, threshold=0.5,
                 average='micro'):
        self._beta = beta
        super().__init__(name, output_names, label_names, class_type, threshold, average)


@register
class BinaryAccuracy(EvalMetric):
    def __init__(self, name='binary_accuracy', output_names=None, label_names=None, threshold=0.5):
        self.threshold = threshold
        super().__init__(name, output_names=output_names, label_names=label_names)

    def update(self, labels, preds):
        labels, preds = check_label_shapes(labels, preds, True)
        for label, pred in zip(labels, preds):
            pred, label = _np(pred), _np(label)
            pl = (pred.reshape(label.shape) > self.threshold).astype('int32')
            self.sum_metric += float((pl == label.astype('int32')).sum())
            self.num_inst += label.size


@register
class MCC(EvalMetric):
    def __init__(self, name='mcc', output_names=None, label_names=None):
        self._metrics = _ClassificationMetrics()
        super().__init__(name=name, output_names=output_names, label_names=label_names)

    def update(self, labels, preds):
        labels, preds = check_label_shapes(labels, preds, True)
        for label, pred in zip(labels, preds):
            self._metrics.update_stats(label, pred)
        self.sum_metric = self._metrics.matthewscc() * self._metrics.total_examples
        self.num_inst = self._metrics.total_examples

    def get(self):
        if self._metrics.num_classes is None:
            return (self.name, float('nan'))
        return (self.name, self._metrics.matthewscc())

    def reset(self):
        self.sum_metric, self.num_inst = 0., 0
        self._metrics.reset_stats()


@register
class Perplexity(EvalMetric):
    def __init__(self, eps=1e-12, ignore_label=None, axis=-1, from_logits=False, name='perplexity', output_names=None,
                 label_names=None):
        super().__init__(name, eps=eps, ignore_label=ignore_label, axis=axis, output_names=output_names,
                         label_names=label_names)
        self.eps, self.ignore_label, self.axis, self.from_logits = eps, ignore_label, axis, from_logits

    def update(self, labels, preds):
        assert len(labels) == len(preds)
        loss, num = 0., 0
        for label, pred in zip(labels, preds):
            label, pred = _np(label).astype('int64'), _np(pred).astype('float64')
            assert label.size == pred.size / pred.shape[-1], 'shape mismatch: %s vs. %s' % (label.shape, pred.shape)
            if self.from_logits:
                pred = pred - pred.max(-1, keepdims=True)
                pred = numpy.exp(pred) / numpy.exp(pred).sum(-1, keepdims=True)
            label = label.reshape(-1)
            pred = pred.reshape(label.size, -1)
            probs = pred[numpy.arange(label.size), label]
            if self.ignore_label is not None:
                ignore = (label == self.ignore_label)
                num -= int(ignore.sum())
                probs = probs * (1 - ignore) + ignore
            loss -= float(numpy.log(numpy.maximum(self.eps, probs)).sum())
            num += label.size
        self.sum_metric += loss
        self.num_inst += num

    def get(self):
        if self.num_inst == 0:
            return (self.name, float('nan'))
        return (self.name, math.exp(self.sum_metric / self.num_inst))


class _Regression(EvalMetric):
    def _pairs(self, labels, preds):
        labels, preds = check_label_shapes(labels, preds, True)
        for label, pred in zip(labels, preds):
            label, pred = _np(label), _np(pred)
            if len(label.shape) == 1:
                label = label.reshape(label.shape[0], 1)
            if len(pred.shape) == 1:
                pred = pred.reshape(pred.shape[0], 1)
            yield label, pred


@register
class MAE(_Regression):
    def __init__(self, name='mae', output_names=None, label_names=None):
        super().__init__(name, output_names=output_names, label_names=label_names)

    def update(self, labels, preds):
        for label, pred in self._pairs(labels, preds):
            self.sum_metric += float(numpy.abs(label - pred).reshape(label.shape[0], -1).mean(-1).sum())
            self.num_inst += label.shape[0]


@register
class MSE(_Regression):
    def __init__(self, name='mse', output_names=None, label_names=None):
        super().__init__(name, output_names=output_names, label_names=label_names)

    def update(self, labels, preds):
        for label, pred in self._pairs(labels, preds):
            self.sum_metric += float(((label - pred) ** 2.0).reshape(label.shape[0], -1).mean(-1).sum())
            self.num_inst += label.shape[0]


@register
class RMSE(MSE):
    def __init__(self, name='rmse', output_names=None, label_names=None):
        super().__init__(name, output_names=output_names, label_names=label_names)

    def get(self):
        if self.num_inst == 0:
            return (self.name, float('nan'))
        return (self.name, math.sqrt(self.sum_metric / self.num_inst))


@register
class MeanPairwiseDistance(_Regression):
    def __init__(self, name='mpd', output_names=None, label_names=None, p=2):
        super().__init__(name, output_names=output_names, label_names=label_names)
        self.p = p

    def update(self, labels, preds):
        for label, pred in self._pairs(labels, preds):
            label, pred = label.reshape(label.shape[0], -1), pred.reshape(pred.shape[0], -1)
            dis = ((numpy.abs(label - pred) ** self.p).sum(axis=-1)) ** (1. / self.p)
            self.sum_metric += float(dis.sum())
            self.num_inst += label.shape[0]


@register
class MeanCosineSimilarity(_Regression):
    def __init__(self, name='cos_sim', output_names=None, label_names=None, eps=1e-8):
        super().__init__(name, output_names=output_names, label_names=label_names)
        self.eps = eps

    def update(self, labels, preds):
        for label, pred in self._pairs(labels, preds):
            sim = (label * pred).sum(axis=-1)
            n1, n2 = numpy.linalg.norm(label, axis=-1), numpy.linalg.norm(pred, axis=-1)
            sim = sim / numpy.maximum(n1 * n2, self.eps)
            self.sum_metric += float(sim.sum())
            self.num_inst += sim.size


@register
@alias('ce')
class CrossEntropy(EvalMetric):
    def __init__(self, eps=1e-12, ignore_label=None, axis=-1, from_logits=False, name='cross-entropy',
                 output_names=None, label_names=None):
        super().__init__(name, eps=eps, output_names=output_names, label_names=label_names)
        self.eps, self.ignore_label, self.axis, self.from_logits = eps, ignore_label, axis, from_logits

    def update(self, labels, preds):
        labels, preds = check_label_shapes(labels, preds, True)
        for label, pred in zip(labels, preds):
            label, pred = _np(label).astype('int64').ravel(), _np(pred).astype('float64')
            pred = pred.reshape(label.shape[0], -1)
            if self.from_logits:
                pred = pred - pred.max(-1, keepdims=True)
                pred = numpy.exp(pred) / numpy.exp(pred).sum(-1, keepdims=True)
            prob = pred[numpy.arange(label.shape[0]), label]
            n = label.shape[0]
            if self.ignore_label is not None:
                ignore = (label == self.ignore_label)
                prob = prob * (1 - ignore) + ignore
                n -= int(ignore.sum())
            self.sum_metric += float((-numpy.log(prob + self.eps)).sum())
            self.num_inst += n


@register
@alias('pearsonr')
class PearsonCorrelation(EvalMetric):
    def __init__(self, name='pearsonr', output_names=None, label_names=None):
        super().__init__(name, output_names=output_names, label_names=label_names)

    def reset(self):
        self._sse_p = self._mean_p = self._sse_l = self._mean_l = self._pred_nums = self._label_nums = self._conv = 0
        self.num_inst = 0
        self.sum_metric = 0.0

    def update(self, labels, preds):
        labels, preds = check_label_shapes(labels, preds, True)
        for label, pred in zip(labels, preds):
            check_label_shapes(label, pred, False, True)
            label, pred = _np(label).ravel().astype(numpy.float64), _np(pred).ravel().astype(numpy.float64)
            self.num_inst += 1
            n = label.size
            mp, ml = pred.mean(), label.mean()
            tot = self._pred_nums + n
            dp, dl = mp - self._mean_p, ml - self._mean_l
            self._conv += ((pred - mp) * (label - ml)).sum() + dp * dl * self._pred_nums * n / tot
            self._sse_p += ((pred - mp) ** 2).sum() + dp * dp * self._pred_nums * n / tot
            self._sse_l += ((label - ml) ** 2).sum() + dl * dl * self._pred_nums * n / tot
            self._mean_p += dp * n / tot
            self._mean_l += dl * n / tot
            self._pred_nums = self._label_nums = tot

    def get(self):
        if self.num_inst == 0:
            return (self.name, float('nan'))
        n = self._label_nums
        pearsonr = self._conv / ((n - 1) * numpy.sqrt(self._sse_p / (n - 1)) * numpy.sqrt(self._sse_l / (n - 1)))
        return (self.name, float(pearsonr))


@register
class PCC(EvalMetric):
    """Multiclass Pearson correlation from the confusion matrix."""

    def __init__(self, name='pcc', output_names=None, label_names=None):
        self.k = 2
        super().__init__(name=name, output_names=output_names, label_names=label_names)

    def _grow(self, inc):
        self.lcm = numpy.pad(self.lcm, ((0, inc), (0, inc)), 'constant', constant_values=(0))
        self.k += inc

    def _calc_mcc(self, cmat):
        n = cmat.sum()
        x, y = cmat.sum(axis=1), cmat.sum(axis=0)
        cov_xx, cov_yy = numpy.sum(x * (n - x)), numpy.sum(y * (n - y))
        if cov_xx == 0 or cov_yy == 0:
            return float('nan')
        i = cmat.diagonal()
        cov_xy = numpy.sum(i * n - x * y)
        return cov_xy / (cov_xx * cov_yy) ** 0.5

    def update(self, labels, preds):
        labels, preds = check_label_shapes(labels, preds, True)
        for label, pred in zip(labels, preds):
            label = _np(label).astype('int32', copy=False).reshape(-1)
            pred = _np(pred)
            pred = pred.argmax(axis=1).astype('int32', copy=False) if pred.ndim > 1 else pred.astype('int32')
            n = int(max(pred.max(), label.max()))
            if n >= self.k:
                self._grow(n + 1 - self.k)
            bcm = numpy.zeros((self.k, self.k))
            for i, j in zip(pred, label):
                bcm[i, j] += 1
            self.lcm += bcm
        self.num_inst += 1

    @property
    def sum_metric(self):
        return self._calc_mcc(self.lcm) * self.num_inst

    @sum_metric.setter
    def sum_metric(self, v):
        pass

    def reset(self):
        self.num_inst = 0.
        self.lcm = numpy.zeros((self.k, self.k))


@register
class Loss(EvalMetric):
    def __init__(self, name='loss', output_names=None, label_names=None):
        super().__init__(name, output_names=output_names, label_names=label_names)

    def update(self, _, preds):
        if isinstance(preds, NDArray):
            preds = [preds]
        for pred in preds:
            loss = float(_np(pred).sum())
            self.sum_metric += loss
            self.num_inst += pred.size if hasattr(pred, 'size') else 1


@register
class Torch(Loss):
    def __init__(self, name='torch', output_names=None, label_names=None):
        super().__init__(name, output_names=output_names, label_names=label_names)


@register
class CustomMetric(EvalMetric):
    def __init__(self, feval, name=None, allow_extra_outputs=False, output_names=None, label_names=None):
        if name is None:
            name = feval.__name__
            if name.find('<') != -1:
                name = 'custom(%s)' % name
        super().__init__(name, feval=feval, allow_extra_outputs=allow_extra_outputs, output_names=output_names,
                         label_names=label_names)
        self._feval, self._allow_extra_outputs = feval, allow_extra_outputs

    def update(self, labels, preds):
        if not self._allow_extra_outputs:
            labels, preds = check_label_shapes(labels, preds, True)
        for pred, label in zip(preds, labels):
            reval = self._feval(_np(label), _np(pred))
            if isinstance(reval, tuple):
                (sum_metric, num_inst) = reval
                self.sum_metric += sum_metric
                self.num_inst += num_inst
            else:
                self.sum_metric += reval
                self.num_inst += 1

    def get_config(self):
        raise NotImplementedError('CustomMetric cannot be serialized')


def np(numpy_feval, name=None, allow_extra_outputs=False):
    def feval(label, pred):
        return numpy_feval(label, pred)
    feval.__name__ = numpy_feval.__name__
    return CustomMetric(feval, name, allow_extra_outputs)


def predict_with_threshold(pred, threshold=0.5):
    """Binary decisions of probabilities: ``pred > threshold`` with one threshold or one per class (last axis)."""
    import numpy as _onp
    if isinstance(threshold, float):
        return pred > threshold
    if hasattr(threshold, 'asnumpy'):
        threshold = threshold.asnumpy()
    threshold = _onp.asarray(threshold)
    num_classes = pred.shape[-1]
    assert threshold.shape[-1] == num_classes, 'shape mismatch: %s vs. %s' % (pred.shape[-1], threshold.shape[-1])
    return pred > threshold


def one_hot(idx, num):
    """(len(idx), num) int32 indicator matrix."""
    import numpy as _onp
    idx = _onp.asarray(idx)
    return (_onp.arange(num).astype(idx.dtype) == idx[:, None]).astype('int32')

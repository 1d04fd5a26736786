"""Loss blocks (``python/mxnet/gluon/loss.py``): 13 losses with ``weight`` / ``batch_axis`` /
``sample_weight`` semantics (loss is averaged over all axes except ``batch_axis``)."""
import math

import numpy as np

from .. import numpy as mnp, numpy_extension as npx
from ..ops import registry as _reg
from .block import HybridBlock

__all__ = ['Loss', 'L2Loss', 'L1Loss', 'SigmoidBinaryCrossEntropyLoss', 'SigmoidBCELoss', 'SoftmaxCrossEntropyLoss',
           'SoftmaxCELoss', 'KLDivLoss', 'CTCLoss', 'HuberLoss', 'HingeLoss', 'SquaredHingeLoss', 'LogisticLoss',
           'TripletLoss', 'PoissonNLLLoss', 'CosineEmbeddingLoss', 'SDMLLoss']


def _op(name, arrays, **attrs):
    return _reg.invoke(name, arrays, attrs)


def _apply_weighting(loss, weight=None, sample_weight=None):
    if sample_weight is not None:
        loss = loss * sample_weight
    if weight is not None:
        assert isinstance(weight, (int, float)), 'weight must be a number'
        loss = loss * weight
    return loss


def _reshape_like(x, y):
    return x.reshape(y.shape)


def _mean_except(loss, batch_axis):
    axes = tuple(i for i in range(loss.ndim) if i != batch_axis % max(loss.ndim, 1))
    if not axes:
        return loss
    return _op('mean', [loss], axis=axes)


class Loss(HybridBlock):
    def __init__(self, weight, batch_axis, **kwargs):
        super().__init__(**kwargs)
        self._weight = weight
        self._batch_axis = batch_axis

    def __repr__(self):
        return '{name}(batch_axis={_batch_axis}, w={_weight})'.format(name=self.__class__.__name__, **self.__dict__)

    def forward(self, x, *args, **kwargs):
        raise NotImplementedError


class L2Loss(Loss):
    def __init__(self, weight=1., batch_axis=0, **kwargs):
        super().__init__(weight, batch_axis, **kwargs)

    def forward(self, pred, label, sample_weight=None):
        label = _reshape_like(label, pred)
        loss = _op('square', [label - pred])
        loss = _apply_weighting(loss, self._weight / 2, sample_weight)
        return _mean_except(loss, self._batch_axis)


class L1Loss(Loss):
    def __init__(self, weight=None, batch_axis=0, **kwargs):
        super().__init__(weight, batch_axis, **kwargs)

    def forward(self, pred, label, sample_weight=None):
        label = _reshape_like(label, pred)
        loss = _op('abs', [label - pred])
        loss = _apply_weighting(loss, self._weight, sample_weight)
        return _mean_except(loss, self._batch_axis)


class SigmoidBinaryCrossEntropyLoss(Loss):
    def __init__(self, from_sigmoid=False, weight=None, batch_axis=0, **kwargs):
        super().__init__(weight, batch_axis, **kwargs)
        self._from_sigmoid = from_sigmoid

    def forward(self, pred, label, sample_weight=None, pos_weight=None):
        label = _reshape_like(label, pred)
        if not self._from_sigmoid:
            softplus = _op('Activation', [-_op('abs', [pred])], act_type='softrelu')
            if pos_weight is None:
                loss = _op('relu', [pred]) - pred * label + softplus
            else:
                log_weight = 1 + (pos_weight - 1) * label
                loss = pred - pred * label + log_weight * (softplus + _op('relu', [-pred]))
        else:
            eps = 1e-12
            if pos_weight is None:
                loss = -(_op('log', [pred + eps]) * label + _op('log', [1. - pred + eps]) * (1. - label))
            else:
                loss = -(_op('log', [pred + eps]) * label * pos_weight + _op('log', [1. - pred + eps]) * (1. - label))
        loss = _apply_weighting(loss, self._weight, sample_weight)
        return _mean_except(loss, self._batch_axis)


SigmoidBCELoss = SigmoidBinaryCrossEntropyLoss


class SoftmaxCrossEntropyLoss(Loss):
    """``-log softmax(pred)[label]``; with sparse labels on the last axis this is one fused kernel."""

    def __init__(self, axis=-1, sparse_label=True, from_logits=False, weight=None, batch_axis=0, **kwargs):
        super().__init__(weight, batch_axis, **kwargs)
        self._axis, self._sparse_label, self._from_logits = axis, sparse_label, from_logits

    def forward(self, pred, label, sample_weight=None):
        if self._sparse_label and not self._from_logits and self._axis in (-1, pred.ndim - 1):
            loss = _op('_npx_softmax_ce_loss', [pred, label], axis=-1)
            loss = _apply_weighting(loss, self._weight, sample_weight.reshape(loss.shape) if sample_weight is not None
                                    and sample_weight.shape != loss.shape and sample_weight.size == loss.size else sample_weight)
            return _mean_except(loss, self._batch_axis) if loss.ndim > 1 else loss
        if not self._from_logits:
            pred = _op('log_softmax', [pred], axis=self._axis)
        if self._sparse_label:
            loss = -_op('pick', [pred, label], axis=self._axis, keepdims=True)
        else:
            label = _reshape_like(label, pred)
            loss = -_op('sum', [pred * label], axis=self._axis, keepdims=True)
        loss = _apply_weighting(loss, self._weight, sample_weight)
        return _mean_except(loss, self._batch_axis)


SoftmaxCELoss = SoftmaxCrossEntropyLoss


class KLDivLoss(Loss):
    def __init__(self, from_logits=True, axis=-1, weight=None, batch_axis=0, **kwargs):
        super().__init__(weight, batch_axis, **kwargs)
        self._from_logits, self._axis = from_logits, axis

    def forward(self, pred, label, sample_weight=None):
        if not self._from_logits:
            pred = _op('log_softmax', [pred], axis=self._axis)
        loss = label * (_op('log', [label + 1e-12]) - pred)
        loss = _apply_weighting(loss, self._weight, sample_weight)
        return _mean_except(loss, self._batch_axis)


class CTCLoss(Loss):
    def __init__(self, layout='NTC', label_layout='NT', weight=None, **kwargs):
        assert layout in ['NTC', 'TNC'], 'Only "NTC" and "TNC" layouts are supported. Got: %s' % layout
        assert label_layout in ['NT', 'TN'], 'Only "NT" and "TN" label layouts are supported. Got: %s' % label_layout
        self._layout, self._label_layout = layout, label_layout
        super().__init__(weight, label_layout.find('N'), **kwargs)

    def forward(self, pred, label, pred_lengths=None, label_lengths=None, sample_weight=None):
        if self._layout == 'NTC':
            pred = _op('SwapAxis', [pred], dim1=0, dim2=1)
        if self._batch_axis == 1:
            label = _op('SwapAxis', [label], dim1=0, dim2=1)
        args = [pred, label]
        if pred_lengths is not None or label_lengths is not None:
            args += [pred_lengths, label_lengths]
        loss = _op('CTCLoss', args, use_data_lengths=pred_lengths is not None,
                   use_label_lengths=label_lengths is not None, blank_label='last')
        return _apply_weighting(loss, self._weight, sample_weight)


class HuberLoss(Loss):
    def __init__(self, rho=1, weight=None, batch_axis=0, **kwargs):
        super().__init__(weight, batch_axis, **kwargs)
        self._rho = rho

    def forward(self, pred, label, sample_weight=None):
        label = _reshape_like(label, pred)
        loss = _op('abs', [label - pred])
        loss = _op('where', [loss > self._rho, loss - 0.5 * self._rho, (0.5 / self._rho) * _op('square', [loss])])
        loss = _apply_weighting(loss, self._weight, sample_weight)
        return _mean_except(loss, self._batch_axis)


class HingeLoss(Loss):
    def __init__(self, margin=1, weight=None, batch_axis=0, **kwargs):
        super().__init__(weight, batch_axis, **kwargs)
        self._margin = margin

    def forward(self, pred, label, sample_weight=None):
        label = _reshape_like(label, pred)
        loss = _op('relu', [self._margin - pred * label])
        loss = _apply_weighting(loss, self._weight, sample_weight)
        return _mean_except(loss, self._batch_axis)


class SquaredHingeLoss(Loss):
    def __init__(self, margin=1, weight=None, batch_axis=0, **kwargs):
        super().__init__(weight, batch_axis, **kwargs)
        self._margin = margin

    def forward(self, pred, label, sample_weight=None):
        label = _reshape_like(label, pred)
        loss = _op('square', [_op('relu', [self._margin - pred * label])])
        loss = _apply_weighting(loss, self._weight, sample_weight)
        return _mean_except(loss, self._batch_axis)


class LogisticLoss(Loss):
    def __init__(self, weight=None, batch_axis=0, label_format='signed', **kwargs):
        super().__init__(weight, batch_axis, **kwargs)
        self._label_format = label_format
        if self._label_format not in ['signed', 'binary']:
            raise ValueError('label_format can only be signed or binary, received %s.' % label_format)

    def forward(self, pred, label, sample_weight=None):
        label = _reshape_like(label, pred)
        if self._label_format == 'signed':
            label = (label + 1.0) / 2.0
        loss = _op('relu', [pred]) - pred * label + _op('Activation', [-_op('abs', [pred])], act_type='softrelu')
        loss = _apply_weighting(loss, self._weight, sample_weight)
        return _mean_except(loss, self._batch_axis)


class TripletLoss(Loss):
    def __init__(self, margin=1, weight=None, batch_axis=0, **kwargs):
        super().__init__(weight, batch_axis, **kwargs)
        self._margin = margin

    def forward(self, pred, positive, negative, sample_weight=None):
        positive = _reshape_like(positive, pred)
        negative = _reshape_like(negative, pred)
        axes = tuple(i for i in range(pred.ndim) if i != self._batch_axis)
        loss = _op('sum', [_op('square', [positive - pred]) - _op('square', [negative - pred])], axis=axes)
        loss = _op('relu', [loss + self._margin])
        return _apply_weighting(loss, self._weight, sample_weight)


class PoissonNLLLoss(Loss):
    def __init__(self, weight=None, from_logits=True, batch_axis=0, compute_full=False, **kwargs):
        super().__init__(weight, batch_axis, **kwargs)
        self._from_logits, self._compute_full = from_logits, compute_full

    def forward(self, pred, target, sample_weight=None, epsilon=1e-08):
        target = _reshape_like(target, pred)
        if self._from_logits:
            loss = _op('exp', [pred]) - target * pred
        else:
            loss = pred - target * _op('log', [pred + epsilon])
        if self._compute_full:
            stirling = target * _op('log', [target]) - target + 0.5 * _op('log', [2 * target * np.pi])
            stirling = stirling * (target > 1)
            loss = loss + stirling
        loss = _apply_weighting(loss, self._weight, sample_weight)
        return _mean_except(loss, self._batch_axis)      # one value per sample, as the other losses


class CosineEmbeddingLoss(Loss):
    def __init__(self, weight=None, batch_axis=0, margin=0, **kwargs):
        super().__init__(weight, batch_axis, **kwargs)
        self._margin = margin

    def forward(self, input1, input2, label, sample_weight=None):
        input1 = _reshape_like(input1, input2)
        cos = self._cosine_similarity(input1, input2)
        label = _reshape_like(label, cos)
        # dissimilar pairs: the part of the similarity above the margin, at most 1 - margin
        loss = _op('where', [label == 1, 1 - cos, _op('clip', [cos - self._margin], a_min=0.0, a_max=1.0 - self._margin)])
        loss = _apply_weighting(loss, self._weight, sample_weight)
        return _mean_except(loss, self._batch_axis)      # one value per pair

    def _cosine_similarity(self, x, y, axis=-1):
        x_norm = _op('norm', [x], axis=axis).reshape(-1, 1)
        y_norm = _op('norm', [y], axis=axis).reshape(-1, 1)
        x_dot_y = _op('sum', [x * y], axis=axis).reshape(-1, 1)
        eps = 1e-12
        return x_dot_y / _op('broadcast_maximum' if x._kind == 'nd' else '_npi_maximum', [x_norm * y_norm, (x_norm * 0 + eps)])


class SDMLLoss(Loss):
    """Smoothed deep metric learning loss over a batch of paired embeddings."""

    def __init__(self, smoothing_parameter=0.3, weight=1., batch_axis=0, **kwargs):
        super().__init__(weight, batch_axis, **kwargs)
        self.kl_loss = KLDivLoss(from_logits=True)
        self.smoothing_parameter = smoothing_parameter

    def _compute_distances(self, x1, x2):
        x1_ = x1.reshape(x1.shape[0], 1, -1)
        x2_ = x2.reshape(1, x2.shape[0], -1)
        return _op('sum', [_op('square', [x1_ - x2_])], axis=2)

    def _compute_labels(self, batch_size, like):
        gold = np.eye(batch_size)
        labels = gold * (1 - self.smoothing_parameter) + (1 - gold) * self.smoothing_parameter / (batch_size - 1)
        return like.__class__(labels.astype('float32'), ctx=like.context)

    def forward(self, x1, x2):
        batch_size = x1.shape[0]
        labels = self._compute_labels(batch_size, x1)
        distances = self._compute_distances(x1, x2)
        log_probabilities = _op('log_softmax', [-distances], axis=1)
        return self.kl_loss(log_probabilities, labels) * batch_size

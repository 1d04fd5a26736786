"""Per-batch train/eval logic used by ``Estimator`` (``batch_processor.py``)."""
from .... import autograd
from ...utils import split_and_load


class BatchProcessor(object):
    def _get_data_and_label(self, batch, ctx, batch_axis=0):
        data, label = batch[0], batch[1]
        return split_and_load(data, ctx_list=ctx, batch_axis=batch_axis), split_and_load(label, ctx_list=ctx, batch_axis=batch_axis)

    def evaluate_batch(self, estimator, val_batch, batch_axis=0):
        data, label = self._get_data_and_label(val_batch, estimator.device, batch_axis)
        pred = [estimator.val_net(x) for x in data]
        loss = [estimator.val_loss(y_hat, y) for y_hat, y in zip(pred, label)]
        return data, label, pred, loss

    def fit_batch(self, estimator, train_batch, batch_axis=0):
        data, label = self._get_data_and_label(train_batch, estimator.device, batch_axis)
        with autograd.record():
            pred = [estimator.net(x) for x in data]
            loss = [estimator.loss(y_hat, y) for y_hat, y in zip(pred, label)]
        for l in loss:
            l.backward()
        return data, label, pred, loss

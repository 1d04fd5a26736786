"""TensorBoard bridge (``python/mxnet/contrib/tensorboard.py``): a batch-end callback logging metrics."""
import logging


class LogMetricsCallback(object):
    def __init__(self, logging_dir, prefix=None):
        self.prefix = prefix
        self.step = 0
        try:
            from torch.utils.tensorboard import SummaryWriter
            self.summary_writer = SummaryWriter(logging_dir)
        except Exception:  # pylint: disable=broad-except
            logging.error('tensorboard is not installed; metrics are not logged')
            self.summary_writer = None

    def __call__(self, param):
        if param.eval_metric is None or self.summary_writer is None:
            return
        self.step += 1
        for name, value in param.eval_metric.get_name_value():
            if self.prefix is not None:
                name = '%s-%s' % (self.prefix, name)
            self.summary_writer.add_scalar(name, value, self.step)

"""Logging helpers (``python/mxnet/log.py``)."""
import logging
import sys

CRITICAL, ERROR, WARNING, INFO, DEBUG, NOTSET = (logging.CRITICAL, logging.ERROR, logging.WARNING, logging.INFO,
                                                 logging.DEBUG, logging.NOTSET)
PY3 = True


class _Formatter(logging.Formatter):
    def __init__(self):
        super().__init__(datefmt='%m%d %H:%M:%S')

    def format(self, record):
        label = {logging.DEBUG: 'D', logging.INFO: 'I', logging.WARNING: 'W', logging.ERROR: 'E',
                 logging.CRITICAL: 'C'}.get(record.levelno, 'U')
        self._style._fmt = label + '%(asctime)s %(process)d %(pathname)s:%(funcName)s:%(lineno)d] %(message)s'
        return super().format(record)


def get_logger(name=None, filename=None, filemode=None, level=WARNING):
    logger = logging.getLogger(name)
    if name is not None and not getattr(logger, '_init_done', None):
        logger._init_done = True
        hdlr = logging.FileHandler(filename, filemode or 'a') if filename else logging.StreamHandler(sys.stderr)
        hdlr.setFormatter(_Formatter())
        logger.addHandler(hdlr)
        logger.setLevel(level)
    return logger


getLogger = get_logger

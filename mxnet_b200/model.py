"""Checkpoint files of the symbolic API and the kvstore choice of the legacy training loop (API of
``python/mxnet/model.py``: ``BatchEndParam``, ``save_checkpoint``, ``load_params``, ``load_checkpoint``,
``_create_kvstore``, ``_create_sparse_kvstore``).

A checkpoint is two files: ``<prefix>-symbol.json`` and ``<prefix>-<epoch:04d>.params``, the latter a name -> array
dictionary whose keys carry an ``arg:`` or ``aux:`` tag.
"""
import logging
import os
from collections import namedtuple

import numpy as np

from . import kvstore as kvs
from . import ndarray as nd
from . import symbol as sym

BatchEndParam = namedtuple('BatchEndParams', ['epoch', 'nbatch', 'eval_metric', 'locals'])

_BIG_PARAM = 16 * 1024 * 1024     # elements; above this a `local` store leaves the update to the workers


def _params_file(prefix, epoch):
    return '%s-%04d.params' % (prefix, epoch)


def _as_store(kvstore, what):
    if isinstance(kvstore, kvs.KVStoreBase):
        return kvstore
    if isinstance(kvstore, str):
        return kvs.create(kvstore)
    raise TypeError(what)


def _create_sparse_kvstore(kvstore):
    """Store for row-sparse parameters: always updates on the store, so it must be able to run an optimizer."""
    kv = _as_store(kvstore, "Cannot create '%s' KVStore with row_sparse parameters. The type must be KVStore or str."
                   % kvstore)
    if not kv.is_capable(kvs.KVStoreBase.OPTIMIZER):
        raise AssertionError('KVStore with sparse weight requires optimizer support.')
    return kv, True


def _create_kvstore(kvstore, num_device, arg_params):
    """``(store, update_on_kvstore)`` for a training run on ``num_device`` devices.

    No store at all for one device unless the name asks for a distributed one.  Updates run on the store when
    ``MXNET_UPDATE_ON_KVSTORE`` (default 1) says so and the store can run an optimizer, except for a ``local`` store with
    a parameter of more than 16M elements."""
    on_store = bool(int(os.environ.get('MXNET_UPDATE_ON_KVSTORE', '1')))
    kv = None
    if isinstance(kvstore, str):
        if num_device > 1 or 'dist' in kvstore:
            kv = kvs.create(kvstore)
            if kvstore == 'local' and max(int(np.prod(p.shape)) for p in arg_params.values()) > _BIG_PARAM:
                on_store = False
    elif kvstore is not None:
        kv = _as_store(kvstore, 'kvstore must be KVStore, str or None')
    if kv is None:
        return None, False
    return kv, on_store and kv.is_capable(kvs.KVStoreBase.OPTIMIZER)


def save_checkpoint(prefix, epoch, symbol, arg_params, aux_params, remove_amp_cast=True):
    """Write the graph (if given) and the tagged parameter dictionary of one epoch."""
    if symbol is not None:
        symbol.save(prefix + '-symbol.json', remove_amp_cast=remove_amp_cast)
    tagged = {}
    for tag, params in (('arg', arg_params), ('aux', aux_params)):
        for name, value in params.items():
            tagged['%s:%s' % (tag, name)] = value.as_nd_ndarray()
    fname = _params_file(prefix, epoch)
    nd.save(fname, tagged)
    logging.info('Saved checkpoint to "%s"', fname)


def load_params(prefix, epoch):
    """``(arg_params, aux_params)`` of one epoch; keys without an ``arg:`` / ``aux:`` tag are ignored."""
    fname = _params_file(prefix, epoch)
    loaded = nd.load(fname)
    out = {'arg': {}, 'aux': {}}
    if not loaded:
        logging.warning('Params file "%s" is empty', fname)
    for key, value in (loaded or {}).items():
        tag, _, name = key.partition(':')
        if tag in out:
            out[tag][name] = value
    return out['arg'], out['aux']


def load_checkpoint(prefix, epoch):
    """``(symbol, arg_params, aux_params)``."""
    return (sym.load(prefix + '-symbol.json'),) + load_params(prefix, epoch)

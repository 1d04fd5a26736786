"""Legacy checkpoint helpers and kvstore selection (``python/mxnet/model.py:74-113,189-264``)."""
import logging
from collections import namedtuple

from . import kvstore as kvs
from . import ndarray as nd
from . import symbol as sym

BatchEndParam = namedtuple('BatchEndParams', ['epoch', 'nbatch', 'eval_metric', 'locals'])


def _create_sparse_kvstore(kvstore):
    if isinstance(kvstore, kvs.KVStoreBase):
        kv = kvstore
    elif isinstance(kvstore, str):
        kv = kvs.create(kvstore)
    else:
        raise TypeError("Cannot create '%s' KVStore with row_sparse parameters. The type must be KVStore or str." % kvstore)
    assert kv.is_capable(kvs.KVStoreBase.OPTIMIZER), 'KVStore with sparse weight requires optimizer support.'
    return (kv, True)


def _create_kvstore(kvstore, num_device, arg_params):
    """Select a store and whether updates run on it: none for a single device unless ``dist`` is in
    the name; ``local`` stores update on the workers when a parameter is larger than 16M elements."""
    update_on_kvstore = bool(int(__import__('os').environ.get('MXNET_UPDATE_ON_KVSTORE', '1')))
    if kvstore is None:
        kv = None
    elif isinstance(kvstore, kvs.KVStoreBase):
        kv = kvstore
    elif isinstance(kvstore, str):
        if num_device == 1 and 'dist' not in kvstore:
            kv = None
        else:
            kv = kvs.create(kvstore)
            if kvstore == 'local':
                max_size = max(int(__import__('numpy').prod(param.shape)) for param in arg_params.values())
                if max_size > 1024 * 1024 * 16:
                    update_on_kvstore = False
    else:
        raise TypeError('kvstore must be KVStore, str or None')
    if kv is None:
        update_on_kvstore = False
    else:
        update_on_kvstore &= kv.is_capable(kvs.KVStoreBase.OPTIMIZER)
    return (kv, update_on_kvstore)


def save_checkpoint(prefix, epoch, symbol, arg_params, aux_params, remove_amp_cast=True):
    if symbol is not None:
        symbol.save('%s-symbol.json' % prefix, remove_amp_cast=remove_amp_cast)
    save_dict = {('arg:%s' % k): v.as_nd_ndarray() for k, v in arg_params.items()}
    save_dict.update({('aux:%s' % k): v.as_nd_ndarray() for k, v in aux_params.items()})
    param_name = '%s-%04d.params' % (prefix, epoch)
    nd.save(param_name, save_dict)
    logging.info('Saved checkpoint to "%s"', param_name)


def load_params(prefix, epoch):
    save_dict = nd.load('%s-%04d.params' % (prefix, epoch))
    arg_params, aux_params = {}, {}
    if not save_dict:
        logging.warning('Params file "%s" is empty', '%s-%04d.params' % (prefix, epoch))
        return (arg_params, aux_params)
    for k, v in save_dict.items():
        tp, name = k.split(':', 1)
        if tp == 'arg':
            arg_params[name] = v
        if tp == 'aux':
            aux_params[name] = v
    return (arg_params, aux_params)


def load_checkpoint(prefix, epoch):
    symbol = sym.load('%s-symbol.json' % prefix)
    arg_params, aux_params = load_params(prefix, epoch)
    return (symbol, arg_params, aux_params)

"""``mx.optimizer``."""
from .optimizer import *          # noqa: F401,F403
from .optimizer import Optimizer, Test, create, register
from .updater import Updater, get_updater
from . import optimizer, updater   # noqa: F401


def _submodules():
    """One module per optimizer as in ``python/mxnet/optimizer/`` (``mx.optimizer.sgd.SGD``, ``mx.optimizer.contrib.GroupAdaGrad``
    ...): the classes live in ``optimizer.py``; these modules give them their reference import paths."""
    import sys as _sys
    import types as _types
    reg = Optimizer.opt_registry
    layout = {'adabelief': ['adabelief'], 'adadelta': ['adadelta'], 'adagrad': ['adagrad'], 'adam': ['adam'], 'adamW': ['adamw'],
              'adamax': ['adamax'], 'dcasgd': ['dcasgd'], 'ftml': ['ftml'], 'ftrl': ['ftrl'], 'lamb': ['lamb'], 'lans': ['lans'],
              'lars': ['lars'], 'nadam': ['nadam'], 'nag': ['nag'], 'rmsprop': ['rmsprop'], 'sgd': ['sgd'], 'sgld': ['sgld'],
              'signum': ['signum'], 'contrib': ['groupadagrad']}
    here = _sys.modules[__name__]
    for mod_name, keys in layout.items():
        m = _types.ModuleType(__name__ + '.' + mod_name)
        names = []
        for k in keys:
            cls = reg.get(k)
            if cls is not None:
                setattr(m, cls.__name__, cls)
                names.append(cls.__name__)
        m.__all__ = names
        m.Optimizer, m.register = Optimizer, register
        _sys.modules[m.__name__] = m
        setattr(here, mod_name, m)
    utils = _types.ModuleType(__name__ + '.utils')

    def _flatten_list(nested_list):
        return [item for sublist in nested_list for item in sublist]
    utils._flatten_list = _flatten_list
    _sys.modules[utils.__name__] = utils
    here.utils = utils


_submodules()

"""``import mxnet`` compatibility name: every ``mxnet[.sub.module]`` resolves to ``mxnet_b200[.sub.module]``
(the same module objects, not copies), so reference user code runs unchanged:

    import mxnet as mx
    from mxnet import gluon, autograd
    from mxnet.gluon import nn
"""
import importlib
import importlib.abc
import importlib.util
import sys

_SRC, _DST = 'mxnet_b200', 'mxnet'


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target):
        self._target = target

    def create_module(self, spec):
        return importlib.import_module(self._target)

    def exec_module(self, module):
        pass


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if fullname != _DST and not fullname.startswith(_DST + '.'):
            return None
        real = _SRC + fullname[len(_DST):]
        try:
            found = importlib.util.find_spec(real)
        except (ImportError, ValueError):
            found = None
        if found is None:
            return None
        spec = importlib.util.spec_from_loader(fullname, _AliasLoader(real), is_package=found.submodule_search_locations is not None)
        return spec


sys.meta_path.insert(0, _AliasFinder())
_impl = importlib.import_module(_SRC)
# alias the modules that are already loaded, then replace this package object itself
for _name, _mod in list(sys.modules.items()):
    if _name == _SRC or _name.startswith(_SRC + '.'):
        sys.modules[_DST + _name[len(_SRC):]] = _mod
sys.modules[_DST] = _impl

"""Name -> class factories shared by optimizers, initializers, metrics and schedules (API of
``python/mxnet/registry.py``: ``get_register_func``, ``get_alias_func``, ``get_create_func``, ``get_registry``).

One ``_Factory`` per base class holds the table; the four public functions hand out bound views of it.  ``create``
accepts a registered name (case-insensitive) with constructor arguments, an existing instance, a dict of keyword
arguments that contains the name under the factory's nickname, or the JSON forms ``'["name", {kwargs}]'`` and
``'{"nickname": "name", ...}'`` that ``Initializer.dumps`` and friends produce.
"""
import json
import warnings


class _Factory(object):
    def __init__(self, base_class):
        self.base = base_class
        self.table = {}

    def add(self, klass, name, nickname):
        if not issubclass(klass, self.base):
            raise AssertionError('Can only register subclass of %s' % self.base.__name__)
        key = (name if name else klass.__name__).lower()
        old = self.table.get(key)
        if old is not None and old is not klass:
            warnings.warn('New %s %s.%s registered with name %s is overriding existing %s %s.%s'
                          % (nickname, klass.__module__, klass.__name__, key, nickname, old.__module__, old.__name__),
                          UserWarning, stacklevel=3)
        self.table[key] = klass
        return klass

    def build(self, nickname, args, kwargs):
        if args:
            spec, args = args[0], args[1:]
        else:
            spec = kwargs.pop(nickname)
        if isinstance(spec, self.base):
            if args or kwargs:
                raise AssertionError('%s is already an instance. Additional arguments are invalid' % nickname)
            return spec
        if isinstance(spec, dict):
            return self.build(nickname, (), dict(spec))
        if not isinstance(spec, str):
            raise AssertionError('%s must be of string type' % nickname)
        if spec[:1] in ('[', '{'):
            if args or kwargs:
                raise AssertionError('a JSON description of a %s takes no further arguments' % nickname)
            decoded = json.loads(spec)
            if isinstance(decoded, list):
                name, kw = decoded
                return self.build(nickname, (name,), dict(kw))
            return self.build(nickname, (), decoded)
        klass = self.table.get(spec.lower())
        if klass is None:
            raise AssertionError('%s is not registered. Please register with %s.register first' % (spec.lower(), nickname))
        return klass(*args, **kwargs)


_FACTORIES = {}


def _factory(base_class):
    f = _FACTORIES.get(base_class)
    if f is None:
        f = _FACTORIES[base_class] = _Factory(base_class)
    return f


def get_registry(base_class):
    """A copy of the name -> class table of ``base_class``."""
    return dict(_factory(base_class).table)


def get_register_func(base_class, nickname):
    """``register(klass, name=None)``: decorator-friendly, registers under the lower-cased class name by default."""
    f = _factory(base_class)

    def register(klass, name=None):
        return f.add(klass, name, nickname)
    register.__doc__ = 'Register %s to the %s factory' % (nickname, nickname)
    return register


def get_alias_func(base_class, nickname):
    """``alias(*names)``: class decorator that registers the class under extra names."""
    f = _factory(base_class)

    def alias(*aliases):
        def decorate(klass):
            for name in aliases:
                f.add(klass, name, nickname)
            return klass
        return decorate
    return alias


def get_create_func(base_class, nickname):
    """``create(name_or_spec, *args, **kwargs)`` as described in the module docstring."""
    f = _factory(base_class)

    def create(*args, **kwargs):
        return f.build(nickname, args, kwargs)
    create.__doc__ = 'Create a %s instance from config.' % nickname
    return create

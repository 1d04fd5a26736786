"""Weight initializers (``python/mxnet/initializer.py``).

Dispatch on the parameter-name suffix: ``*weight`` → ``_init_weight``, ``*bias`` → 0, ``*gamma`` → 1,
``*beta`` → 0, ``*running_mean``/``*moving_mean`` → 0, ``*running_var``/``*moving_var`` → 1
(``initializer.py:140-210``).  Random streams differ from the reference's; distributions match.
"""
import json
import math
import re

import numpy as np
import torch

from . import registry
from .ndarray.ndarray import NDArray

__all__ = ['InitDesc', 'Initializer', 'register', 'alias', 'create', 'Load', 'Mixed', 'Zero', 'One', 'Constant',
           'Uniform', 'Normal', 'Orthogonal', 'Xavier', 'MSRAPrelu', 'Bilinear', 'LSTMBias', 'RNNFused', 'FusedRNN']


class InitDesc(str):
    """Name of the parameter to initialise, carrying attributes and a global fallback initializer."""

    def __new__(cls, name, attrs=None, global_init=None):
        ret = super(InitDesc, cls).__new__(cls, name)
        ret.attrs = attrs or {}
        ret.global_init = global_init
        return ret


class Initializer(object):
    def __init__(self, **kwargs):
        self._kwargs = kwargs
        self._verbose = False
        self._print_func = None

    def set_verbosity(self, verbose=False, print_func=None):
        self._verbose = verbose
        self._print_func = print_func or (lambda x: str((np.abs(x.asnumpy()).mean())))
        return self

    def dumps(self):
        return json.dumps([self.__class__.__name__.lower(), self._kwargs])

    def __call__(self, desc, arr):
        if not isinstance(desc, InitDesc):
            desc = InitDesc(str(desc))
        if desc.global_init is None:
            desc.global_init = self
        init = desc.attrs.get('__init__', '')
        if init:
            create(init)._init_weight(desc, arr)
            return
        name = str(desc)
        if name.endswith('weight'):
            self._init_weight(desc, arr)
        elif name.endswith('bias'):
            self._init_bias(desc, arr)
        elif name.endswith('gamma'):
            self._init_gamma(desc, arr)
        elif name.endswith('beta'):
            self._init_beta(desc, arr)
        elif name.endswith('running_mean') or name.endswith('moving_mean'):
            self._init_zero(desc, arr)
        elif name.endswith('running_var') or name.endswith('moving_var'):
            self._init_one(desc, arr)
        elif name.endswith('moving_inv_var') or name.endswith('moving_avg'):
            self._init_zero(desc, arr)
        elif name.endswith('min') or name.endswith('max'):
            self._init_zero(desc, arr)
        else:
            self._init_default(desc, arr)

    def _init_bias(self, _, arr): arr._data.zero_()
    def _init_gamma(self, _, arr): arr._data.fill_(1.0)
    def _init_beta(self, _, arr): arr._data.zero_()
    def _init_zero(self, _, arr): arr._data.zero_()
    def _init_one(self, _, arr): arr._data.fill_(1.0)

    def _init_weight(self, name, arr):
        raise NotImplementedError('Must override it')

    def _init_default(self, name, _):
        raise ValueError('Unknown initialization pattern for %s. Default initialization is now limited to '
                         '"weight", "bias", "gamma" (1.0), and "beta" (0.0). Please use mx.sym.Variable(init=...) '
                         'to set initialization pattern' % name)

    def __eq__(self, other):
        return isinstance(other, Initializer) and self.__class__ is other.__class__ and self._kwargs == other._kwargs

    __hash__ = object.__hash__


register = registry.get_register_func(Initializer, 'initializer')
alias = registry.get_alias_func(Initializer, 'initializer')
_create = registry.get_create_func(Initializer, 'initializer')


def create(*args, **kwargs):
    if args and args[0] is None:
        return Uniform()
    return _create(*args, **kwargs)


def _fill(arr, t):
    with torch.no_grad():
        arr._data.copy_(t.to(arr._data.dtype))


class Load(object):
    """Initialise from a dict or file of saved arrays, falling back to ``default_init``."""

    def __init__(self, param, default_init=None, verbose=False):
        if isinstance(param, str):
            from .ndarray.utils import load
            param = load(param)
        self.param = {}
        for name, arr in param.items():
            self.param[name[4:] if name.startswith('arg:') or name.startswith('aux:') else name] = arr
        self.default_init = default_init
        self.verbose = verbose

    def __call__(self, name, arr):
        if name in self.param:
            assert arr.shape == self.param[name].shape, \
                'Parameter %s cannot be initialized from loading. Shape mismatch, target %s vs loaded %s' % (
                    name, str(arr.shape), self.param[name].shape)
            _fill(arr, self.param[name]._data)
        else:
            assert self.default_init is not None, \
                'Cannot Initialize %s. Not found in loaded param and no default Initializer is provided.' % name
            self.default_init(name, arr)


class Mixed(object):
    """Pattern-matched list of initializers."""

    def __init__(self, patterns, initializers):
        assert len(patterns) == len(initializers)
        self.map = list(zip([re.compile(p) for p in patterns], initializers))

    def __call__(self, name, arr):
        for prog, init in self.map:
            if prog.match(name):
                init(name, arr)
                return
        raise ValueError('Parameter name %s did not match any pattern. Consider adding a ".*" pattern at the '
                         'and with default Initializer.' % name)


@register
@alias('zeros')
class Zero(Initializer):
    def _init_weight(self, _, arr): arr._data.zero_()


@register
@alias('ones')
class One(Initializer):
    def _init_weight(self, _, arr): arr._data.fill_(1.0)


@register
class Constant(Initializer):
    def __init__(self, value=0.0):
        super().__init__(value=value if not isinstance(value, NDArray) else value.asnumpy().tolist())
        self.value = value

    def _init_weight(self, _, arr):
        v = self.value
        if isinstance(v, NDArray):
            _fill(arr, v._data.to(arr._data.device).expand_as(arr._data))
        elif isinstance(v, (list, tuple, np.ndarray)):
            _fill(arr, torch.as_tensor(np.asarray(v)).to(arr._data.device).expand_as(arr._data))
        else:
            arr._data.fill_(v)

    _init_default = _init_weight
    _init_bias = _init_gamma = _init_beta = _init_weight


@register
class Uniform(Initializer):
    def __init__(self, scale=0.07):
        super().__init__(scale=scale)
        self.scale = scale

    def _init_weight(self, _, arr):
        with torch.no_grad():
            arr._data.uniform_(-self.scale, self.scale) if arr._data.dtype != torch.float16 or arr._data.is_cuda else \
                arr._data.copy_(torch.empty(arr.shape).uniform_(-self.scale, self.scale))


@register
class Normal(Initializer):
    def __init__(self, sigma=0.01):
        super().__init__(sigma=sigma)
        self.sigma = sigma

    def _init_weight(self, _, arr):
        with torch.no_grad():
            arr._data.copy_(torch.empty(arr.shape, device=arr._data.device).normal_(0, self.sigma))


@register
class Orthogonal(Initializer):
    def __init__(self, scale=1.414, rand_type='uniform'):
        super().__init__(scale=scale, rand_type=rand_type)
        self.scale, self.rand_type = scale, rand_type

    def _init_weight(self, _, arr):
        nout = arr.shape[0]
        nin = int(np.prod(arr.shape[1:]))
        tmp = np.random.uniform(-1.0, 1.0, (nout, nin)) if self.rand_type == 'uniform' else np.random.normal(0.0, 1.0, (nout, nin))
        u, _, v = np.linalg.svd(tmp, full_matrices=False)
        res = u if u.shape == tmp.shape else v
        _fill(arr, torch.from_numpy(self.scale * res.reshape(arr.shape)).to(arr._data.device))


@register
class Xavier(Initializer):
    """``scale = sqrt(magnitude / factor)``, factor from fan-in/out (``initializer.py:583-648``)."""

    def __init__(self, rnd_type='uniform', factor_type='avg', magnitude=3):
        super().__init__(rnd_type=rnd_type, factor_type=factor_type, magnitude=magnitude)
        self.rnd_type, self.factor_type, self.magnitude = rnd_type, factor_type, float(magnitude)

    def _init_weight(self, name, arr):
        shape = arr.shape
        hw_scale = 1.
        if len(shape) < 2:
            raise ValueError('Xavier initializer cannot be applied to vector {0}. It requires at least 2D.'.format(name))
        if len(shape) > 2:
            hw_scale = np.prod(shape[2:])
        fan_in, fan_out = shape[1] * hw_scale, shape[0] * hw_scale
        if self.factor_type == 'avg':
            factor = (fan_in + fan_out) / 2.0
        elif self.factor_type == 'in':
            factor = fan_in
        elif self.factor_type == 'out':
            factor = fan_out
        else:
            raise ValueError('Incorrect factor type')
        scale = math.sqrt(self.magnitude / factor)
        with torch.no_grad():
            tmp = torch.empty(shape, device=arr._data.device, dtype=torch.float32)
            if self.rnd_type == 'uniform':
                tmp.uniform_(-scale, scale)
            elif self.rnd_type == 'gaussian':
                tmp.normal_(0, scale)
            else:
                raise ValueError('Unknown random type')
            arr._data.copy_(tmp)


@register
class MSRAPrelu(Xavier):
    def __init__(self, factor_type='avg', slope=0.25):
        magnitude = 2. / (1 + slope ** 2)
        super().__init__('gaussian', factor_type, magnitude)
        self._kwargs = {'factor_type': factor_type, 'slope': slope}


@register
class Bilinear(Initializer):
    def _init_weight(self, _, arr):
        weight = np.zeros(int(np.prod(arr.shape)), dtype='float32')
        shape = arr.shape
        f = np.ceil(shape[3] / 2.)
        c = (2 * f - 1 - f % 2) / (2. * f)
        for i in range(weight.size):
            x = i % shape[3]
            y = (i // shape[3]) % shape[2]
            weight[i] = (1 - abs(x / f - c)) * (1 - abs(y / f - c))
        _fill(arr, torch.from_numpy(weight.reshape(shape)).to(arr._data.device))


@register
class LSTMBias(Initializer):
    """Forget-gate bias set to ``forget_bias``, the rest zero (gate order i, f, g, o)."""

    def __init__(self, forget_bias=1.0):
        super().__init__(forget_bias=forget_bias)
        self.forget_bias = forget_bias

    def _init_weight(self, name, arr):
        arr._data.zero_()
        num_hidden = int(arr.shape[0] / 4)
        arr._data[num_hidden:2 * num_hidden] = self.forget_bias

    _init_bias = _init_weight


@register
class RNNFused(Initializer):
    """Initialise the flat parameter vector of the fused RNN operator piece by piece."""

    def __init__(self, mode, num_layers, state_size, bidirectional=False, projection_size=None, i2h_weight_initializer=None,
                 h2h_weight_initializer=None, i2h_bias_initializer=None, h2h_bias_initializer=None,
                 h2r_weight_initializer=None):
        super().__init__(mode=mode, num_layers=num_layers, state_size=state_size, bidirectional=bidirectional,
                         projection_size=projection_size)
        self._mode, self._num_layers, self._state_size = mode, num_layers, state_size
        self._bidirectional, self._projection_size = bidirectional, projection_size
        self._inits = {'i2h_weight': i2h_weight_initializer, 'h2h_weight': h2h_weight_initializer,
                       'i2h_bias': i2h_bias_initializer or 'zeros', 'h2h_bias': h2h_bias_initializer or 'zeros',
                       'h2r_weight': h2r_weight_initializer}

    def _init_weight(self, desc, arr):
        from .ops.nn import rnn_unpack, _GATES
        g, d = _GATES[self._mode], 2 if self._bidirectional else 1
        h = self._state_size
        p = self._projection_size or h
        total = arr.shape[0]
        # solve the input size from the total length
        rest = total - d * (g * h * p + 2 * g * h + (p * h if self._projection_size else 0))
        for l in range(1, self._num_layers):
            rest -= d * (g * h * p * d + g * h * p + 2 * g * h + (p * h if self._projection_size else 0))
        ni = rest // (d * g * h)
        pieces = rnn_unpack(arr._data, self._mode, self._num_layers, ni, h, self._bidirectional, self._projection_size)
        glob = desc.global_init if isinstance(desc, InitDesc) else None
        for w_ih, w_hh, w_hr, b_ih, b_hh in pieces:
            for nm, t in (('i2h_weight', w_ih), ('h2h_weight', w_hh), ('h2r_weight', w_hr), ('i2h_bias', b_ih), ('h2h_bias', b_hh)):
                if t is None:
                    continue
                init = self._inits[nm]
                init = create(init) if init is not None else (glob or Uniform())
                tmp = NDArray._from_tensor(torch.zeros(t.shape, dtype=torch.float32, device=t.device))
                init(InitDesc(nm), tmp)
                with torch.no_grad():
                    t.copy_(tmp._data)


FusedRNN = RNNFused

"""Activation layers (``python/mxnet/gluon/nn/activations.py``)."""
from ...ops import registry as _reg
from ..block import HybridBlock
from ..parameter import Parameter

__all__ = ['Activation', 'LeakyReLU', 'PReLU', 'ELU', 'SELU', 'Swish', 'GELU', 'SiLU']


def _op(name, arrays, **attrs):
    return _reg.invoke(name, arrays, attrs)


class Activation(HybridBlock):
    def __init__(self, activation):
        self._act_type = activation
        super().__init__()

    def _alias(self):
        return self._act_type

    def forward(self, x):
        return _op('Activation', [x], act_type=self._act_type)

    def __repr__(self):
        return '{name}({_act_type})'.format(name=self.__class__.__name__, **self.__dict__)


class LeakyReLU(HybridBlock):
    def __init__(self, alpha):
        assert alpha >= 0, 'Slope coefficient for LeakyReLU must be no less than 0.'
        super().__init__()
        self._alpha = alpha

    def forward(self, x):
        return _op('LeakyReLU', [x], act_type='leaky', slope=self._alpha)

    def __repr__(self):
        return '{name}({alpha})'.format(name=self.__class__.__name__, alpha=self._alpha)


class PReLU(HybridBlock):
    def __init__(self, alpha_initializer=None, in_channels=1):
        super().__init__()
        from ... import initializer
        self.alpha = Parameter('alpha', shape=(in_channels,), init=alpha_initializer or initializer.Constant(0.25))

    def forward(self, x):
        return _op('LeakyReLU', [x, self.alpha.data(x.context)], act_type='prelu')


class ELU(HybridBlock):
    def __init__(self, alpha=1.0):
        super().__init__()
        self._alpha = alpha

    def forward(self, x):
        return _op('LeakyReLU', [x], act_type='elu', slope=self._alpha)


class SELU(HybridBlock):
    def forward(self, x):
        return _op('LeakyReLU', [x], act_type='selu')


class GELU(HybridBlock):
    def __init__(self, approximation='erf'):
        super().__init__()
        self._act = 'gelu' if approximation == 'erf' else 'gelu_tanh'

    def forward(self, x):
        return _op('LeakyReLU', [x], act_type=self._act)


class Swish(HybridBlock):
    def __init__(self, beta=1.0):
        super().__init__()
        self._beta = beta

    def forward(self, x):
        return x * _op('sigmoid', [x * self._beta])


class SiLU(HybridBlock):
    def forward(self, x):
        return x * _op('sigmoid', [x])

"""Basic neural-network layers (``python/mxnet/gluon/nn/basic_layers.py``)."""
import warnings

import numpy as np

from ... import _state
from ...ops import registry as _reg
from ...util import is_np_array
from ..block import Block, HybridBlock
from ..parameter import Parameter
from .activations import Activation

__all__ = ['Sequential', 'HybridSequential', 'Dense', 'Dropout', 'Embedding', 'BatchNorm', 'SyncBatchNorm',
           'BatchNormReLU', 'InstanceNorm', 'LayerNorm', 'GroupNorm', 'Flatten', 'Lambda', 'HybridLambda',
           'Concatenate', 'HybridConcatenate', 'Identity']


def _op(name, arrays, **attrs):
    return _reg.invoke(name, arrays, attrs)


class Sequential(Block):
    def __init__(self):
        super().__init__()
        self._layers = []

    def add(self, *blocks):
        for block in blocks:
            self._layers.append(block)
            self.register_child(block)

    def forward(self, x, *args):
        for block in self._children.values():
            x = block(x, *args)
            args = []
            if isinstance(x, (tuple, list)):
                args = x[1:]
                x = x[0]
        if args:
            x = tuple([x] + list(args))
        return x

    def __repr__(self):
        modstr = '\n'.join(['  ({key}): {block}'.format(key=key, block=repr(block).replace('\n', '\n  '))
                            for key, block in self._children.items()])
        return '{name}(\n{modstr}\n)'.format(name=self.__class__.__name__, modstr=modstr)

    def __getitem__(self, key):
        layers = list(self._children.values())[key]
        if isinstance(layers, list):
            net = type(self)()
            net.add(*layers)
            return net
        return layers

    def __len__(self):
        return len(self._children)

    def hybridize(self, active=True, **kwargs):
        if self._children and all(isinstance(c, HybridBlock) for c in self._children.values()):
            warnings.warn('All children of this Sequential layer \'%s\' are HybridBlocks. Consider using '
                          'HybridSequential for the best performance.' % type(self).__name__, stacklevel=2)
        super().hybridize(active, **kwargs)


class HybridSequential(HybridBlock):
    def __init__(self):
        super().__init__()
        self._layers = []

    def add(self, *blocks):
        for block in blocks:
            self._layers.append(block)
            self.register_child(block)

    def forward(self, x, *args):
        for block in self._children.values():
            x = block(x, *args)
            args = []
            if isinstance(x, (tuple, list)):
                args = x[1:]
                x = x[0]
        if args:
            x = tuple([x] + list(args))
        return x

    def infer_shape(self, *args):
        pass

    __repr__ = Sequential.__repr__

    def __getitem__(self, key):
        layers = list(self._children.values())[key]
        if isinstance(layers, list):
            net = type(self)()
            net.add(*layers)
            return net
        return layers

    def __len__(self):
        return len(self._children)


class Dense(HybridBlock):
    """``y = act(x · Wᵀ + b)``; weight ``(units, in_units)``.  On the GPU bias and activation are
    epilogues of the tensor-core GEMM."""

    def __init__(self, units, activation=None, use_bias=True, flatten=True, dtype='float32', weight_initializer=None,
                 bias_initializer='zeros', in_units=0):
        super().__init__()
        self._flatten = flatten
        self._units = units
        self._in_units = in_units
        self.weight = Parameter('weight', shape=(units, in_units), init=weight_initializer, dtype=dtype,
                                allow_deferred_init=True)
        self.bias = Parameter('bias', shape=(units,), init=bias_initializer, dtype=dtype,
                              allow_deferred_init=True) if use_bias else None
        self.act = Activation(activation) if activation is not None else None

    def forward(self, x):
        ctx = x.context
        args = [x, self.weight.data(ctx)]
        if self.bias is not None:
            args.append(self.bias.data(ctx))
        act = _op('FullyConnected', args, num_hidden=self._units, no_bias=self.bias is None, flatten=self._flatten)
        if self.act is not None:
            act = self.act(act)
        return act

    def infer_shape(self, x, *args):
        if self._flatten:
            num_input = 1
            for i in range(1, x.ndim):
                num_input *= x.shape[i]
            self.weight.shape = (self.weight.shape[0], num_input)
        else:
            self.weight.shape = (self.weight.shape[0], x.shape[x.ndim - 1])

    def __repr__(self):
        shape = self.weight.shape
        return '{name}({layout}, {act})'.format(name=self.__class__.__name__, act=self.act if self.act else 'linear',
                                                layout='{0} -> {1}'.format(shape[1] if shape[1] else None, shape[0]))


class Dropout(HybridBlock):
    def __init__(self, rate, axes=()):
        super().__init__()
        self._rate, self._axes = rate, axes

    def forward(self, x):
        if self._rate > 0:
            return _op('Dropout', [x], p=self._rate, axes=self._axes)
        return x

    def __repr__(self):
        return '{name}(p = {_rate}, axes={_axes})'.format(name=self.__class__.__name__, **self.__dict__)


class _BatchNorm(HybridBlock):
    def __init__(self, axis=1, momentum=0.9, epsilon=1e-5, center=True, scale=True, use_global_stats=False,
                 fuse_relu=False, beta_initializer='zeros', gamma_initializer='ones',
                 running_mean_initializer='zeros', running_variance_initializer='ones', in_channels=0):
        super().__init__()
        self._kwargs = {'axis': axis, 'eps': epsilon, 'momentum': momentum, 'fix_gamma': not scale,
                        'use_global_stats': use_global_stats}
        self.fuse_relu = fuse_relu
        self._axis = axis
        if in_channels != 0:
            self.in_channels = in_channels
        self.gamma = Parameter('gamma', grad_req='write' if scale else 'null', shape=(in_channels,),
                               init=gamma_initializer, allow_deferred_init=True, differentiable=scale)
        self.beta = Parameter('beta', grad_req='write' if center else 'null', shape=(in_channels,),
                              init=beta_initializer, allow_deferred_init=True, differentiable=center)
        self.running_mean = Parameter('running_mean', grad_req='null', shape=(in_channels,),
                                      init=running_mean_initializer, allow_deferred_init=True, differentiable=False)
        self.running_var = Parameter('running_var', grad_req='null', shape=(in_channels,),
                                     init=running_variance_initializer, allow_deferred_init=True, differentiable=False)

    def cast(self, dtype):
        import numpy as _np
        if str(dtype) in ('float16', "<class 'numpy.float16'>") or dtype == _np.float16 or str(dtype) == 'bfloat16':
            dtype = 'float32'
        super().cast(dtype)

    def forward(self, x, residual=None):
        ctx = x.context
        args = [x, self.gamma.data(ctx), self.beta.data(ctx), self.running_mean.data(ctx), self.running_var.data(ctx)]
        kw = dict(self._kwargs)
        if self.fuse_relu:
            kw['act_type'] = 'relu'
        if residual is not None:
            args.append(residual)
        return _op('BatchNorm', args, **kw)

    def infer_shape(self, x, *args):
        channel_count = x.shape[self._axis]
        for p in (self.gamma, self.beta, self.running_mean, self.running_var):
            p.shape = (channel_count,)

    def __repr__(self):
        in_channels = self.gamma.shape[0]
        return '{name}({content}, in_channels={in_channels})'.format(
            name=self.__class__.__name__, in_channels=in_channels if in_channels else None,
            content=', '.join(['='.join([k, v.__repr__()]) for k, v in self._kwargs.items()]))


class BatchNorm(_BatchNorm):
    """Batch normalisation (``basic_layers.py:345-375``): ``axis=1, momentum=0.9, epsilon=1e-5``."""

    def __init__(self, axis=1, momentum=0.9, epsilon=1e-5, center=True, scale=True, use_global_stats=False,
                 beta_initializer='zeros', gamma_initializer='ones', running_mean_initializer='zeros',
                 running_variance_initializer='ones', in_channels=0, **kwargs):
        super().__init__(axis, momentum, epsilon, center, scale, use_global_stats, False, beta_initializer,
                         gamma_initializer, running_mean_initializer, running_variance_initializer, in_channels)


class BatchNormReLU(_BatchNorm):
    """BatchNorm with the ReLU (and optionally a residual add before it) fused into the same kernel."""

    def __init__(self, axis=1, momentum=0.9, epsilon=1e-5, center=True, scale=True, use_global_stats=False,
                 beta_initializer='zeros', gamma_initializer='ones', running_mean_initializer='zeros',
                 running_variance_initializer='ones', in_channels=0, **kwargs):
        super().__init__(axis, momentum, epsilon, center, scale, use_global_stats, True, beta_initializer,
                         gamma_initializer, running_mean_initializer, running_variance_initializer, in_channels)


class SyncBatchNorm(BatchNorm):
    """Cross-device BatchNorm (``src/operator/contrib/sync_batch_norm-inl.h``)."""

    def __init__(self, in_channels=0, num_devices=None, momentum=0.9, epsilon=1e-5, center=True, scale=True,
                 use_global_stats=False, beta_initializer='zeros', gamma_initializer='ones',
                 running_mean_initializer='zeros', running_variance_initializer='ones', **kwargs):
        super().__init__(1, momentum, epsilon, center, scale, use_global_stats, beta_initializer, gamma_initializer,
                         running_mean_initializer, running_variance_initializer, in_channels)
        self._ndev = num_devices or 1

    def forward(self, x, residual=None):
        ctx = x.context
        args = [x, self.gamma.data(ctx), self.beta.data(ctx), self.running_mean.data(ctx), self.running_var.data(ctx)]
        kw = {k: v for k, v in self._kwargs.items() if k != 'axis'}
        return _op('SyncBatchNorm', args, ndev=self._ndev, key=str(id(self)), **kw)


class Embedding(HybridBlock):
    def __init__(self, input_dim, output_dim, dtype='float32', weight_initializer=None, sparse_grad=False):
        super().__init__()
        self._kwargs = {'input_dim': input_dim, 'output_dim': output_dim, 'dtype': dtype, 'sparse_grad': sparse_grad}
        self.weight = Parameter('weight', shape=(input_dim, output_dim), init=weight_initializer, dtype=dtype,
                                allow_deferred_init=True, grad_stype='default')

    def forward(self, x):
        return _op('Embedding', [x, self.weight.data(x.context)], **self._kwargs)

    def __repr__(self):
        return '{name}({input_dim} -> {output_dim}, {dtype})'.format(name=self.__class__.__name__, **self._kwargs)


class Flatten(HybridBlock):
    def forward(self, x):
        return _op('Flatten', [x])

    def __repr__(self):
        return self.__class__.__name__


class InstanceNorm(HybridBlock):
    def __init__(self, axis=1, epsilon=1e-5, center=True, scale=False, beta_initializer='zeros',
                 gamma_initializer='ones', in_channels=0):
        super().__init__()
        self._kwargs = {'eps': epsilon, 'axis': axis, 'center': center, 'scale': scale}
        self._axis, self._epsilon = axis, epsilon
        self.gamma = Parameter('gamma', grad_req='write' if scale else 'null', shape=(in_channels,),
                               init=gamma_initializer, allow_deferred_init=True)
        self.beta = Parameter('beta', grad_req='write' if center else 'null', shape=(in_channels,),
                              init=beta_initializer, allow_deferred_init=True)

    def forward(self, x):
        ctx = x.context
        if self._axis == 1:
            return _op('InstanceNorm', [x, self.gamma.data(ctx), self.beta.data(ctx)], eps=self._epsilon)
        x = _op('SwapAxis', [x], dim1=1, dim2=self._axis)
        y = _op('InstanceNorm', [x, self.gamma.data(ctx), self.beta.data(ctx)], eps=self._epsilon)
        return _op('SwapAxis', [y], dim1=1, dim2=self._axis)

    def infer_shape(self, x, *args):
        self.gamma.shape = (x.shape[self._axis],)
        self.beta.shape = (x.shape[self._axis],)


class LayerNorm(HybridBlock):
    def __init__(self, axis=-1, epsilon=1e-5, center=True, scale=True, beta_initializer='zeros',
                 gamma_initializer='ones', in_channels=0):
        super().__init__()
        self._kwargs = {'eps': epsilon, 'axis': axis, 'center': center, 'scale': scale}
        self._axis, self._epsilon, self._center, self._scale = axis, epsilon, center, scale
        self.gamma = Parameter('gamma', grad_req='write' if scale else 'null', shape=(in_channels,),
                               init=gamma_initializer, allow_deferred_init=True)
        self.beta = Parameter('beta', grad_req='write' if center else 'null', shape=(in_channels,),
                              init=beta_initializer, allow_deferred_init=True)

    def forward(self, data):
        ctx = data.context
        known = self.gamma.shape[0] if self.gamma.shape else 0
        assert known <= 0 or known == data.shape[self._axis], \
            'LayerNorm was built for %d channels along axis %d but the input has %d' % (known, self._axis, data.shape[self._axis])
        return _op('LayerNorm', [data, self.gamma.data(ctx), self.beta.data(ctx)], axis=self._axis, eps=self._epsilon)

    def infer_shape(self, data, *args):
        self.gamma.shape = (data.shape[self._axis],)
        self.beta.shape = (data.shape[self._axis],)

    def __repr__(self):
        in_channels = self.gamma.shape[0]
        return '{name}({content}, in_channels={in_channels})'.format(
            name=self.__class__.__name__, in_channels=in_channels,
            content=', '.join(['='.join([k, v.__repr__()]) for k, v in self._kwargs.items()]))


class GroupNorm(HybridBlock):
    def __init__(self, num_groups=1, epsilon=1e-5, center=True, scale=True, beta_initializer='zeros',
                 gamma_initializer='ones', in_channels=0):
        super().__init__()
        self._kwargs = {'eps': epsilon, 'num_groups': num_groups, 'center': center, 'scale': scale}
        self._num_groups, self._epsilon = num_groups, epsilon
        self.gamma = Parameter('gamma', grad_req='write' if scale else 'null', shape=(in_channels,),
                               init=gamma_initializer, allow_deferred_init=True)
        self.beta = Parameter('beta', grad_req='write' if center else 'null', shape=(in_channels,),
                              init=beta_initializer, allow_deferred_init=True)

    def forward(self, data):
        ctx = data.context
        return _op('GroupNorm', [data, self.gamma.data(ctx), self.beta.data(ctx)], num_groups=self._num_groups,
                   eps=self._epsilon)

    def infer_shape(self, data, *args):
        self.gamma.shape = (data.shape[1],)
        self.beta.shape = (data.shape[1],)


class Lambda(Block):
    def __init__(self, function):
        super().__init__()
        if isinstance(function, str):
            from ... import ndarray as nd, numpy as mnp, numpy_extension as npx
            for mod in (mnp, npx, nd):
                if hasattr(mod, function):
                    self._func_impl = getattr(mod, function)
                    break
            else:
                raise AssertionError('Function name %s is not found in ndarray.' % function)
        elif callable(function):
            self._func_impl = function
        else:
            raise ValueError('Unrecognized function in lambda: {} of type {}'.format(function, type(function)))

    def forward(self, *args):
        return self._func_impl(*args)


class HybridLambda(HybridBlock):
    def __init__(self, function):
        super().__init__()
        if isinstance(function, str):
            from ... import ndarray as nd, numpy as mnp, numpy_extension as npx
            for mod in (mnp, npx, nd):
                if hasattr(mod, function):
                    self._func = getattr(mod, function)
                    break
            else:
                raise AssertionError('Function name %s is not found in ndarray.' % function)
            self._func_name = function
        elif callable(function):
            self._func = function
            self._func_name = getattr(function, '__name__', 'lambda')
        else:
            raise ValueError('Unrecognized function in lambda: {} of type {}'.format(function, type(function)))

    def forward(self, x, *args):
        return self._func(x, *args)

    def infer_shape(self, *args):
        pass


class Concatenate(Sequential):
    def __init__(self, axis=-1):
        super().__init__()
        self.axis = axis

    def forward(self, x):
        out = [block(x) for block in self._children.values()]
        return _op('Concat', out, dim=self.axis)


class HybridConcatenate(HybridSequential):
    def __init__(self, axis=-1):
        super().__init__()
        self.axis = axis

    def forward(self, x):
        out = [block(x) for block in self._children.values()]
        return _op('Concat', out, dim=self.axis)


class Identity(HybridBlock):
    def forward(self, x):
        return x

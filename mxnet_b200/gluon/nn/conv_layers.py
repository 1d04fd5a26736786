"""Convolution, transposed convolution, pooling and padding layers
(``python/mxnet/gluon/nn/conv_layers.py``)."""
from ...ops import registry as _reg
from ..block import HybridBlock
from ..parameter import Parameter
from .activations import Activation

__all__ = ['Conv1D', 'Conv2D', 'Conv3D', 'Conv1DTranspose', 'Conv2DTranspose', 'Conv3DTranspose', 'MaxPool1D',
           'MaxPool2D', 'MaxPool3D', 'AvgPool1D', 'AvgPool2D', 'AvgPool3D', 'GlobalMaxPool1D', 'GlobalMaxPool2D',
           'GlobalMaxPool3D', 'GlobalAvgPool1D', 'GlobalAvgPool2D', 'GlobalAvgPool3D', 'ReflectionPad2D',
           'DeformableConvolution', 'ModulatedDeformableConvolution', 'PixelShuffle1D', 'PixelShuffle2D', 'PixelShuffle3D']


def _op(name, arrays, **attrs):
    return _reg.invoke(name, arrays, attrs)


def _tup(v, n):
    return (v,) * n if isinstance(v, int) else tuple(v)


class _Conv(HybridBlock):
    def __init__(self, channels, kernel_size, strides, padding, dilation, groups, layout, in_channels=0,
                 activation=None, use_bias=True, weight_initializer=None, bias_initializer='zeros',
                 op_name='Convolution', adj=None, dtype='float32'):
        super().__init__()
        self._channels, self._in_channels = channels, in_channels
        nd = len(kernel_size)
        self._kwargs = {'kernel': kernel_size, 'stride': _tup(strides, nd), 'dilate': _tup(dilation, nd),
                        'pad': _tup(padding, nd), 'num_filter': channels, 'num_group': groups,
                        'no_bias': not use_bias, 'layout': layout}
        if adj is not None:
            self._kwargs['adj'] = _tup(adj, nd)
        self._op_name = op_name
        self._layout = layout
        self._groups = groups
        channel_last = layout[-1] == 'C'
        if op_name == 'Convolution':
            wshape = (channels,) + tuple(kernel_size) + (in_channels // groups,) if channel_last else \
                (channels, in_channels // groups) + tuple(kernel_size)
        else:
            wshape = (in_channels,) + tuple(kernel_size) + (channels // groups,) if channel_last else \
                (in_channels, channels // groups) + tuple(kernel_size)
        self.weight = Parameter('weight', shape=wshape, init=weight_initializer, allow_deferred_init=True, dtype=dtype)
        self.bias = Parameter('bias', shape=(channels,), init=bias_initializer, allow_deferred_init=True,
                              dtype=dtype) if use_bias else None
        self.act = Activation(activation) if activation is not None else None

    def forward(self, x):
        ctx = x.context
        args = [x, self.weight.data(ctx)]
        if self.bias is not None:
            args.append(self.bias.data(ctx))
        act = _op(self._op_name, args, **self._kwargs)
        if self.act is not None:
            act = self.act(act)
        return act

    def infer_shape(self, x, *args):
        channel_last = self._layout[-1] == 'C'
        in_c = x.shape[-1] if channel_last else x.shape[1]
        shape = list(self.weight.shape)
        if self._op_name == 'Convolution':
            shape[-1 if channel_last else 1] = in_c // self._groups
        else:
            shape[0] = in_c
        self.weight.shape = tuple(shape)

    def _alias(self):
        return 'conv'

    def __repr__(self):
        s = '{name}({mapping}, kernel_size={kernel}, stride={stride}'
        len_kernel_size = len(self._kwargs['kernel'])
        if self._kwargs['pad'] != (0,) * len_kernel_size:
            s += ', padding={pad}'
        if self._kwargs['dilate'] != (1,) * len_kernel_size:
            s += ', dilation={dilate}'
        if self._kwargs['num_group'] != 1:
            s += ', groups={num_group}'
        if self.bias is None:
            s += ', bias=False'
        if self.act:
            s += ', {}'.format(self.act)
        s += ')'
        shape = self.weight.shape
        return s.format(name=self.__class__.__name__,
                        mapping='{0} -> {1}'.format(self._in_channels or None, self._channels), **self._kwargs)


class Conv1D(_Conv):
    def __init__(self, channels, kernel_size, strides=1, padding=0, dilation=1, groups=1, layout='NCW', activation=None,
                 use_bias=True, weight_initializer=None, bias_initializer='zeros', in_channels=0, dtype='float32'):
        assert layout in ('NCW', 'NWC'), 'Only supports NCW and NWC layout for now'
        super().__init__(channels, _tup(kernel_size, 1), strides, padding, dilation, groups, layout, in_channels,
                         activation, use_bias, weight_initializer, bias_initializer, dtype=dtype)


class Conv2D(_Conv):
    def __init__(self, channels, kernel_size, strides=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1, layout='NCHW',
                 activation=None, use_bias=True, weight_initializer=None, bias_initializer='zeros', in_channels=0,
                 dtype='float32'):
        assert layout in ('NCHW', 'NHWC'), 'Only supports NCHW and NHWC layout for now'
        super().__init__(channels, _tup(kernel_size, 2), strides, padding, dilation, groups, layout, in_channels,
                         activation, use_bias, weight_initializer, bias_initializer, dtype=dtype)


class Conv3D(_Conv):
    def __init__(self, channels, kernel_size, strides=(1, 1, 1), padding=(0, 0, 0), dilation=(1, 1, 1), groups=1,
                 layout='NCDHW', activation=None, use_bias=True, weight_initializer=None, bias_initializer='zeros',
                 in_channels=0, dtype='float32'):
        assert layout in ('NCDHW', 'NDHWC'), 'Only supports NCDHW and NDHWC layout for now'
        super().__init__(channels, _tup(kernel_size, 3), strides, padding, dilation, groups, layout, in_channels,
                         activation, use_bias, weight_initializer, bias_initializer, dtype=dtype)


class Conv1DTranspose(_Conv):
    def __init__(self, channels, kernel_size, strides=1, padding=0, output_padding=0, dilation=1, groups=1, layout='NCW',
                 activation=None, use_bias=True, weight_initializer=None, bias_initializer='zeros', in_channels=0,
                 dtype='float32'):
        super().__init__(channels, _tup(kernel_size, 1), strides, padding, dilation, groups, layout, in_channels,
                         activation, use_bias, weight_initializer, bias_initializer, 'Deconvolution', output_padding, dtype)
        self.outpad = output_padding


class Conv2DTranspose(_Conv):
    def __init__(self, channels, kernel_size, strides=(1, 1), padding=(0, 0), output_padding=(0, 0), dilation=(1, 1),
                 groups=1, layout='NCHW', activation=None, use_bias=True, weight_initializer=None,
                 bias_initializer='zeros', in_channels=0, dtype='float32'):
        super().__init__(channels, _tup(kernel_size, 2), strides, padding, dilation, groups, layout, in_channels,
                         activation, use_bias, weight_initializer, bias_initializer, 'Deconvolution', output_padding, dtype)
        self.outpad = output_padding


class Conv3DTranspose(_Conv):
    def __init__(self, channels, kernel_size, strides=(1, 1, 1), padding=(0, 0, 0), output_padding=(0, 0, 0),
                 dilation=(1, 1, 1), groups=1, layout='NCDHW', activation=None, use_bias=True, weight_initializer=None,
                 bias_initializer='zeros', in_channels=0, dtype='float32'):
        super().__init__(channels, _tup(kernel_size, 3), strides, padding, dilation, groups, layout, in_channels,
                         activation, use_bias, weight_initializer, bias_initializer, 'Deconvolution', output_padding, dtype)
        self.outpad = output_padding


class _Pooling(HybridBlock):
    def __init__(self, pool_size, strides, padding, ceil_mode, global_pool, pool_type, layout, count_include_pad=None):
        super().__init__()
        if strides is None:
            strides = pool_size
        nd = len(pool_size)
        self._kwargs = {'kernel': pool_size, 'stride': _tup(strides, nd), 'pad': _tup(padding, nd),
                        'global_pool': global_pool, 'pool_type': pool_type, 'layout': layout,
                        'pooling_convention': 'full' if ceil_mode else 'valid'}
        if count_include_pad is not None:
            self._kwargs['count_include_pad'] = count_include_pad

    def _alias(self):
        return 'pool'

    def forward(self, x):
        return _op('Pooling', [x], **self._kwargs)

    def __repr__(self):
        s = '{name}(size={kernel}, stride={stride}, padding={pad}, ceil_mode={ceil_mode}, global_pool={global_pool}, ' \
            'pool_type={pool_type}, layout={layout})'
        return s.format(name=self.__class__.__name__, ceil_mode=self._kwargs['pooling_convention'] == 'full', **self._kwargs)


def _make_pool(name, nd, pool_type, global_pool, default_layout):
    if global_pool:
        def __init__(self, layout=default_layout):
            _Pooling.__init__(self, (1,) * nd, None, 0, True, True, pool_type, layout)
    elif pool_type == 'max':
        def __init__(self, pool_size=(2,) * nd if nd > 1 else 2, strides=None, padding=0, layout=default_layout, ceil_mode=False):
            _Pooling.__init__(self, _tup(pool_size, nd), strides, padding, ceil_mode, False, 'max', layout)
    else:
        def __init__(self, pool_size=(2,) * nd if nd > 1 else 2, strides=None, padding=0, ceil_mode=False,
                     layout=default_layout, count_include_pad=True):
            _Pooling.__init__(self, _tup(pool_size, nd), strides, padding, ceil_mode, False, 'avg', layout, count_include_pad)
    return type(name, (_Pooling,), {'__init__': __init__})


for _nd, _lay in ((1, 'NCW'), (2, 'NCHW'), (3, 'NCDHW')):
    globals()['MaxPool%dD' % _nd] = _make_pool('MaxPool%dD' % _nd, _nd, 'max', False, _lay)
    globals()['AvgPool%dD' % _nd] = _make_pool('AvgPool%dD' % _nd, _nd, 'avg', False, _lay)
    globals()['GlobalMaxPool%dD' % _nd] = _make_pool('GlobalMaxPool%dD' % _nd, _nd, 'max', True, _lay)
    globals()['GlobalAvgPool%dD' % _nd] = _make_pool('GlobalAvgPool%dD' % _nd, _nd, 'avg', True, _lay)


class ReflectionPad2D(HybridBlock):
    def __init__(self, padding=0):
        super().__init__()
        if isinstance(padding, int):
            padding = (0, 0, 0, 0, padding, padding, padding, padding)
        assert len(padding) == 8
        self._padding = padding

    def forward(self, x):
        return _op('Pad', [x], mode='reflect', pad_width=self._padding)


class DeformableConvolution(HybridBlock):
    """Deformable convolution v1: a regular convolution predicts per-tap sampling offsets, the input
    is bilinearly sampled at the shifted taps and contracted with the weights
    (``src/operator/contrib/deformable_convolution-inl.h``)."""

    def __init__(self, channels, kernel_size=(1, 1), strides=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1,
                 num_deformable_group=1, layout='NCHW', use_bias=True, in_channels=0, activation=None,
                 weight_initializer=None, bias_initializer='zeros', offset_weight_initializer='zeros',
                 offset_bias_initializer='zeros', offset_use_bias=True, modulated=False):
        super().__init__()
        k = _tup(kernel_size, 2)
        self._k, self._s, self._p, self._d = k, _tup(strides, 2), _tup(padding, 2), _tup(dilation, 2)
        self._channels, self._groups, self._dg, self._modulated = channels, groups, num_deformable_group, modulated
        off_ch = num_deformable_group * k[0] * k[1] * (3 if modulated else 2)
        self.offset = Conv2D(off_ch, k, strides, padding, dilation, 1, layout, None, offset_use_bias,
                             offset_weight_initializer, offset_bias_initializer, in_channels)
        self.weight = Parameter('weight', shape=(channels, in_channels // groups) + k, init=weight_initializer,
                                allow_deferred_init=True)
        self.bias = Parameter('bias', shape=(channels,), init=bias_initializer) if use_bias else None
        self.act = Activation(activation) if activation is not None else None

    def infer_shape(self, x, *args):
        self.weight.shape = (self._channels, x.shape[1] // self._groups) + self._k

    def forward(self, x):
        import torch
        import torch.nn.functional as F
        off = self.offset(x)
        ctx = x.context
        w = self.weight.data(ctx)._data
        xt, ot = x._data, off._data
        n, c, h, wd = xt.shape
        kh, kw = self._k
        oh, ow = ot.shape[2], ot.shape[3]
        kk = kh * kw
        if self._modulated:
            mask = torch.sigmoid(ot[:, 2 * self._dg * kk:])
            ot = ot[:, :2 * self._dg * kk]
        base_y = (torch.arange(oh, device=xt.device) * self._s[0] - self._p[0]).view(1, 1, oh, 1).float()
        base_x = (torch.arange(ow, device=xt.device) * self._s[1] - self._p[1]).view(1, 1, 1, ow).float()
        cols = []
        cpg = c // self._dg
        for g in range(self._dg):
            xg = xt[:, g * cpg:(g + 1) * cpg]
            for i in range(kh):
                for j in range(kw):
                    t = i * kw + j
                    dy = ot[:, g * 2 * kk + 2 * t].unsqueeze(1)
                    dx = ot[:, g * 2 * kk + 2 * t + 1].unsqueeze(1)
                    py = base_y + i * self._d[0] + dy
                    px = base_x + j * self._d[1] + dx
                    grid = torch.stack([2 * px / max(wd - 1, 1) - 1, 2 * py / max(h - 1, 1) - 1], -1).squeeze(1)
                    samp = F.grid_sample(xg, grid, mode='bilinear', padding_mode='zeros', align_corners=True)
                    if self._modulated:
                        samp = samp * mask[:, g * kk + t].unsqueeze(1)
                    cols.append(samp)
        col = torch.stack(cols, 2).reshape(n, self._dg, kk, cpg, oh, ow).permute(0, 1, 3, 2, 4, 5).reshape(n, c * kk, oh * ow)
        wmat = w.reshape(self._groups, self._channels // self._groups, -1)
        col = col.reshape(n, self._groups, (c // self._groups) * kk, oh * ow)
        out = torch.einsum('gok,ngkp->ngop', wmat, col).reshape(n, self._channels, oh, ow)
        if self.bias is not None:
            out = out + self.bias.data(ctx)._data.view(1, -1, 1, 1)
        res = x.__class__._from_tensor(out, ctx)
        return self.act(res) if self.act is not None else res


class ModulatedDeformableConvolution(DeformableConvolution):
    def __init__(self, *args, **kwargs):
        kwargs['modulated'] = True
        super().__init__(*args, **kwargs)


class _PixelShuffle(HybridBlock):
    def __init__(self, factor, nd):
        super().__init__()
        self._factors = _tup(factor, nd)
        self._nd = nd

    def forward(self, x):
        import torch
        t = x._data
        n, c = t.shape[0], t.shape[1]
        f = self._factors
        prod = 1
        for v in f:
            prod *= v
        sp = t.shape[2:]
        t = t.reshape((n, c // prod) + tuple(f) + tuple(sp))
        nd = self._nd
        perm = [0, 1]
        for i in range(nd):
            perm += [2 + nd + i, 2 + i]
        t = t.permute(perm).reshape((n, c // prod) + tuple(s * k for s, k in zip(sp, f)))
        return x.__class__._from_tensor(t, x.context)


class PixelShuffle1D(_PixelShuffle):
    def __init__(self, factor):
        super().__init__(factor, 1)


class PixelShuffle2D(_PixelShuffle):
    def __init__(self, factor):
        super().__init__(factor, 2)


class PixelShuffle3D(_PixelShuffle):
    def __init__(self, factor):
        super().__init__(factor, 3)

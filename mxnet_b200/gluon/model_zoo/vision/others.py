"""AlexNet, VGG, SqueezeNet, DenseNet, MobileNet V1/V2, Inception V3
(``python/mxnet/gluon/model_zoo/vision/{alexnet,vgg,squeezenet,densenet,mobilenet,inception}.py``)."""
from ....ops import registry as _reg
from ...block import HybridBlock
from ... import nn

__all__ = ['get_vgg', 'get_mobilenet', 'get_mobilenet_v2', 'AlexNet', 'alexnet', 'VGG', 'vgg11', 'vgg13', 'vgg16', 'vgg19', 'vgg11_bn', 'vgg13_bn', 'vgg16_bn',
           'vgg19_bn', 'SqueezeNet', 'squeezenet1_0', 'squeezenet1_1', 'DenseNet', 'densenet121', 'densenet161',
           'densenet169', 'densenet201', 'MobileNet', 'MobileNetV2', 'mobilenet1_0', 'mobilenet0_75', 'mobilenet0_5',
           'mobilenet0_25', 'mobilenet_v2_1_0', 'mobilenet_v2_0_75', 'mobilenet_v2_0_5', 'mobilenet_v2_0_25',
           'Inception3', 'inception_v3']


def _op(name, arrays, **attrs):
    return _reg.invoke(name, arrays, attrs)


class AlexNet(HybridBlock):
    def __init__(self, classes=1000, **kwargs):
        super().__init__()
        f = self.features = nn.HybridSequential()
        f.add(nn.Conv2D(64, kernel_size=11, strides=4, padding=2, activation='relu'), nn.MaxPool2D(pool_size=3, strides=2),
              nn.Conv2D(192, kernel_size=5, padding=2, activation='relu'), nn.MaxPool2D(pool_size=3, strides=2),
              nn.Conv2D(384, kernel_size=3, padding=1, activation='relu'),
              nn.Conv2D(256, kernel_size=3, padding=1, activation='relu'),
              nn.Conv2D(256, kernel_size=3, padding=1, activation='relu'), nn.MaxPool2D(pool_size=3, strides=2),
              nn.Flatten(), nn.Dense(4096, activation='relu'), nn.Dropout(0.5), nn.Dense(4096, activation='relu'),
              nn.Dropout(0.5))
        self.output = nn.Dense(classes)

    def forward(self, x):
        return self.output(self.features(x))


def alexnet(pretrained=False, **kwargs):
    return AlexNet(**{k: v for k, v in kwargs.items() if k not in ('ctx', 'device', 'root')})


class VGG(HybridBlock):
    def __init__(self, layers, filters, classes=1000, batch_norm=False, **kwargs):
        super().__init__()
        assert len(layers) == len(filters)
        f = self.features = nn.HybridSequential()
        for i, num in enumerate(layers):
            for _ in range(num):
                f.add(nn.Conv2D(filters[i], kernel_size=3, padding=1))
                if batch_norm:
                    f.add(nn.BatchNorm())
                f.add(nn.Activation('relu'))
            f.add(nn.MaxPool2D(strides=2))
        f.add(nn.Dense(4096, activation='relu', weight_initializer='normal'), nn.Dropout(rate=0.5),
              nn.Dense(4096, activation='relu', weight_initializer='normal'), nn.Dropout(rate=0.5))
        self.output = nn.Dense(classes, weight_initializer='normal')

    def forward(self, x):
        return self.output(self.features(x))


vgg_spec = {11: ([1, 1, 2, 2, 2], [64, 128, 256, 512, 512]), 13: ([2, 2, 2, 2, 2], [64, 128, 256, 512, 512]),
            16: ([2, 2, 3, 3, 3], [64, 128, 256, 512, 512]), 19: ([2, 2, 4, 4, 4], [64, 128, 256, 512, 512])}


def _vgg(n, bn=False):
    def f(pretrained=False, **kwargs):
        layers, filters = vgg_spec[n]
        return VGG(layers, filters, batch_norm=bn, **{k: v for k, v in kwargs.items() if k not in ('ctx', 'device', 'root')})
    return f


def get_vgg(num_layers, pretrained=False, ctx=None, root=None, **kwargs):
    """VGG with 11, 13, 16 or 19 layers (``batch_norm=True`` for the normalised variants), as
    ``gluon/model_zoo/vision/vgg.py:get_vgg``."""
    if num_layers not in vgg_spec:
        raise ValueError('VGG has 11, 13, 16 or 19 layers, not %s' % num_layers)
    layers, filters = vgg_spec[num_layers]
    kwargs.pop('device', None)
    return VGG(layers, filters, **kwargs)


vgg11, vgg13, vgg16, vgg19 = _vgg(11), _vgg(13), _vgg(16), _vgg(19)
vgg11_bn, vgg13_bn, vgg16_bn, vgg19_bn = _vgg(11, True), _vgg(13, True), _vgg(16, True), _vgg(19, True)


class _Fire(HybridBlock):
    def __init__(self, squeeze, e1, e3):
        super().__init__()
        self.squeeze = nn.Conv2D(squeeze, 1, activation='relu')
        self.e1 = nn.Conv2D(e1, 1, activation='relu')
        self.e3 = nn.Conv2D(e3, 3, padding=1, activation='relu')

    def forward(self, x):
        x = self.squeeze(x)
        return _op('Concat', [self.e1(x), self.e3(x)], dim=1)


class SqueezeNet(HybridBlock):
    def __init__(self, version, classes=1000, **kwargs):
        super().__init__()
        assert version in ['1.0', '1.1']
        f = self.features = nn.HybridSequential()
        if version == '1.0':
            f.add(nn.Conv2D(96, kernel_size=7, strides=2, activation='relu'), nn.MaxPool2D(3, 2, ceil_mode=True),
                  _Fire(16, 64, 64), _Fire(16, 64, 64), _Fire(32, 128, 128), nn.MaxPool2D(3, 2, ceil_mode=True),
                  _Fire(32, 128, 128), _Fire(48, 192, 192), _Fire(48, 192, 192), _Fire(64, 256, 256),
                  nn.MaxPool2D(3, 2, ceil_mode=True), _Fire(64, 256, 256))
        else:
            f.add(nn.Conv2D(64, kernel_size=3, strides=2, activation='relu'), nn.MaxPool2D(3, 2, ceil_mode=True),
                  _Fire(16, 64, 64), _Fire(16, 64, 64), nn.MaxPool2D(3, 2, ceil_mode=True), _Fire(32, 128, 128),
                  _Fire(32, 128, 128), nn.MaxPool2D(3, 2, ceil_mode=True), _Fire(48, 192, 192), _Fire(48, 192, 192),
                  _Fire(64, 256, 256), _Fire(64, 256, 256))
        f.add(nn.Dropout(0.5))
        self.output = nn.HybridSequential()
        self.output.add(nn.Conv2D(classes, kernel_size=1, activation='relu'), nn.GlobalAvgPool2D(), nn.Flatten())

    def forward(self, x):
        return self.output(self.features(x))


def squeezenet1_0(pretrained=False, **kwargs): return SqueezeNet('1.0', **{k: v for k, v in kwargs.items() if k not in ('ctx', 'device', 'root')})
def squeezenet1_1(pretrained=False, **kwargs): return SqueezeNet('1.1', **{k: v for k, v in kwargs.items() if k not in ('ctx', 'device', 'root')})


class _DenseLayer(HybridBlock):
    def __init__(self, growth_rate, bn_size, dropout):
        super().__init__()
        b = self.body = nn.HybridSequential()
        b.add(nn.BatchNorm(), nn.Activation('relu'), nn.Conv2D(bn_size * growth_rate, kernel_size=1, use_bias=False),
              nn.BatchNorm(), nn.Activation('relu'), nn.Conv2D(growth_rate, kernel_size=3, padding=1, use_bias=False))
        if dropout:
            b.add(nn.Dropout(dropout))

    def forward(self, x):
        return _op('Concat', [x, self.body(x)], dim=1)


class DenseNet(HybridBlock):
    def __init__(self, num_init_features, growth_rate, block_config, bn_size=4, dropout=0, classes=1000, **kwargs):
        super().__init__()
        f = self.features = nn.HybridSequential()
        f.add(nn.Conv2D(num_init_features, kernel_size=7, strides=2, padding=3, use_bias=False), nn.BatchNorm(),
              nn.Activation('relu'), nn.MaxPool2D(pool_size=3, strides=2, padding=1))
        num_features = num_init_features
        for i, num_layers in enumerate(block_config):
            blk = nn.HybridSequential()
            for _ in range(num_layers):
                blk.add(_DenseLayer(growth_rate, bn_size, dropout))
            f.add(blk)
            num_features += num_layers * growth_rate
            if i != len(block_config) - 1:
                tr = nn.HybridSequential()
                tr.add(nn.BatchNorm(), nn.Activation('relu'), nn.Conv2D(num_features // 2, kernel_size=1, use_bias=False),
                       nn.AvgPool2D(pool_size=2, strides=2))
                f.add(tr)
                num_features //= 2
        f.add(nn.BatchNorm(), nn.Activation('relu'), nn.AvgPool2D(pool_size=7), nn.Flatten())
        self.output = nn.Dense(classes)

    def forward(self, x):
        return self.output(self.features(x))


densenet_spec = {121: (64, 32, [6, 12, 24, 16]), 161: (96, 48, [6, 12, 36, 24]), 169: (64, 32, [6, 12, 32, 32]),
                 201: (64, 32, [6, 12, 48, 32])}


def _densenet(n):
    def f(pretrained=False, **kwargs):
        a, b, c = densenet_spec[n]
        return DenseNet(a, b, c, **{k: v for k, v in kwargs.items() if k not in ('ctx', 'device', 'root')})
    return f


densenet121, densenet161, densenet169, densenet201 = _densenet(121), _densenet(161), _densenet(169), _densenet(201)


class _RELU6(HybridBlock):
    def forward(self, x):
        return _op('clip', [x], a_min=0.0, a_max=6.0)


def _add_conv(out, channels=1, kernel=1, stride=1, pad=0, num_group=1, active=True, relu6=False):
    out.add(nn.Conv2D(channels, kernel, stride, pad, groups=num_group, use_bias=False))
    out.add(nn.BatchNorm(scale=True))
    if active:
        out.add(_RELU6() if relu6 else nn.Activation('relu'))


class _LinearBottleneck(HybridBlock):
    def __init__(self, in_channels, channels, t, stride):
        super().__init__()
        self.use_shortcut = stride == 1 and in_channels == channels
        self.out = nn.HybridSequential()
        _add_conv(self.out, in_channels * t, relu6=True)
        _add_conv(self.out, in_channels * t, kernel=3, stride=stride, pad=1, num_group=in_channels * t, relu6=True)
        _add_conv(self.out, channels, active=False, relu6=True)

    def forward(self, x):
        out = self.out(x)
        return out + x if self.use_shortcut else out


class MobileNet(HybridBlock):
    def __init__(self, multiplier=1.0, classes=1000, **kwargs):
        super().__init__()
        f = self.features = nn.HybridSequential()
        _add_conv(f, channels=int(32 * multiplier), kernel=3, pad=1, stride=2)
        dw_channels = [int(x * multiplier) for x in [32, 64] + [128] * 2 + [256] * 2 + [512] * 6 + [1024]]
        channels = [int(x * multiplier) for x in [64] + [128] * 2 + [256] * 2 + [512] * 6 + [1024] * 2]
        strides = [1, 2] * 3 + [1] * 5 + [2, 1]
        for dwc, c, s in zip(dw_channels, channels, strides):
            _add_conv(f, channels=dwc, kernel=3, stride=s, pad=1, num_group=dwc)
            _add_conv(f, channels=c)
        f.add(nn.GlobalAvgPool2D(), nn.Flatten())
        self.output = nn.Dense(classes)

    def forward(self, x):
        return self.output(self.features(x))


class MobileNetV2(HybridBlock):
    def __init__(self, multiplier=1.0, classes=1000, **kwargs):
        super().__init__()
        f = self.features = nn.HybridSequential()
        _add_conv(f, int(32 * multiplier), kernel=3, stride=2, pad=1, relu6=True)
        in_channels_group = [int(x * multiplier) for x in [32] + [16] + [24] * 2 + [32] * 3 + [64] * 4 + [96] * 3 + [160] * 3]
        channels_group = [int(x * multiplier) for x in [16] + [24] * 2 + [32] * 3 + [64] * 4 + [96] * 3 + [160] * 3 + [320]]
        ts = [1] + [6] * 16
        strides = [1, 2] * 2 + [1, 1, 2] + [1] * 6 + [2] + [1] * 3
        for in_c, c, t, s in zip(in_channels_group, channels_group, ts, strides):
            f.add(_LinearBottleneck(in_c, c, t, s))
        last = int(1280 * multiplier) if multiplier > 1.0 else 1280
        _add_conv(f, last, relu6=True)
        f.add(nn.GlobalAvgPool2D())
        self.output = nn.HybridSequential()
        self.output.add(nn.Conv2D(classes, 1, use_bias=False), nn.Flatten())

    def forward(self, x):
        return self.output(self.features(x))


def _mobilenet(cls, m):
    def f(pretrained=False, **kwargs):
        return cls(m, **{k: v for k, v in kwargs.items() if k not in ('ctx', 'device', 'root')})
    return f


def get_mobilenet(multiplier, pretrained=False, ctx=None, root=None, **kwargs):
    """MobileNet (v1) with the given width multiplier (``gluon/model_zoo/vision/mobilenet.py:get_mobilenet``)."""
    kwargs.pop('device', None)
    return MobileNet(multiplier, **kwargs)


def get_mobilenet_v2(multiplier, pretrained=False, ctx=None, root=None, **kwargs):
    """MobileNetV2 with the given width multiplier."""
    kwargs.pop('device', None)
    return MobileNetV2(multiplier, **kwargs)


mobilenet1_0, mobilenet0_75, mobilenet0_5, mobilenet0_25 = (_mobilenet(MobileNet, m) for m in (1.0, 0.75, 0.5, 0.25))
mobilenet_v2_1_0, mobilenet_v2_0_75, mobilenet_v2_0_5, mobilenet_v2_0_25 = (_mobilenet(MobileNetV2, m) for m in (1.0, 0.75, 0.5, 0.25))


def _basic_conv(**kwargs):
    out = nn.HybridSequential()
    out.add(nn.Conv2D(use_bias=False, **kwargs), nn.BatchNorm(epsilon=0.001), nn.Activation('relu'))
    return out


class _Branches(HybridBlock):
    """Parallel branches concatenated on the channel axis."""

    def __init__(self, branches):
        super().__init__()
        for i, b in enumerate(branches):
            setattr(self, 'b%d' % i, b)
        self._n = len(branches)

    def forward(self, x):
        return _op('Concat', [getattr(self, 'b%d' % i)(x) for i in range(self._n)], dim=1)


def _branch(use_pool, *conv_settings):
    out = nn.HybridSequential()
    if use_pool == 'avg':
        out.add(nn.AvgPool2D(pool_size=3, strides=1, padding=1))
    elif use_pool == 'max':
        out.add(nn.MaxPool2D(pool_size=3, strides=2))
    for setting in conv_settings:
        kw = {}
        for i, name in enumerate(['channels', 'kernel_size', 'strides', 'padding']):
            if setting[i] is not None:
                kw[name] = setting[i]
        out.add(_basic_conv(**kw))
    return out


def _make_A(pool_features):
    return _Branches([_branch(None, (64, 1, None, None)), _branch(None, (48, 1, None, None), (64, 5, None, 2)),
                      _branch(None, (64, 1, None, None), (96, 3, None, 1), (96, 3, None, 1)),
                      _branch('avg', (pool_features, 1, None, None))])


def _make_B():
    return _Branches([_branch(None, (384, 3, 2, None)), _branch(None, (64, 1, None, None), (96, 3, None, 1), (96, 3, 2, None)),
                      _branch('max')])


def _make_C(c7):
    return _Branches([_branch(None, (192, 1, None, None)),
                      _branch(None, (c7, 1, None, None), (c7, (1, 7), None, (0, 3)), (192, (7, 1), None, (3, 0))),
                      _branch(None, (c7, 1, None, None), (c7, (7, 1), None, (3, 0)), (c7, (1, 7), None, (0, 3)),
                              (c7, (7, 1), None, (3, 0)), (192, (1, 7), None, (0, 3))),
                      _branch('avg', (192, 1, None, None))])


def _make_D():
    return _Branches([_branch(None, (192, 1, None, None), (320, 3, 2, None)),
                      _branch(None, (192, 1, None, None), (192, (1, 7), None, (0, 3)), (192, (7, 1), None, (3, 0)), (192, 3, 2, None)),
                      _branch('max')])


class _SplitBranch(HybridBlock):
    def __init__(self, head, a, b):
        super().__init__()
        self.head, self.a, self.b = head, a, b

    def forward(self, x):
        x = self.head(x)
        return _op('Concat', [self.a(x), self.b(x)], dim=1)


def _make_E():
    b1 = _SplitBranch(_branch(None, (384, 1, None, None)), _branch(None, (384, (1, 3), None, (0, 1))),
                      _branch(None, (384, (3, 1), None, (1, 0))))
    b2 = _SplitBranch(_branch(None, (448, 1, None, None), (384, 3, None, 1)), _branch(None, (384, (1, 3), None, (0, 1))),
                      _branch(None, (384, (3, 1), None, (1, 0))))
    return _Branches([_branch(None, (320, 1, None, None)), b1, b2, _branch('avg', (192, 1, None, None))])


class Inception3(HybridBlock):
    def __init__(self, classes=1000, **kwargs):
        super().__init__()
        f = self.features = nn.HybridSequential()
        f.add(_basic_conv(channels=32, kernel_size=3, strides=2), _basic_conv(channels=32, kernel_size=3),
              _basic_conv(channels=64, kernel_size=3, padding=1), nn.MaxPool2D(pool_size=3, strides=2),
              _basic_conv(channels=80, kernel_size=1), _basic_conv(channels=192, kernel_size=3),
              nn.MaxPool2D(pool_size=3, strides=2), _make_A(32), _make_A(64), _make_A(64), _make_B(), _make_C(128),
              _make_C(160), _make_C(160), _make_C(192), _make_D(), _make_E(), _make_E(), nn.AvgPool2D(pool_size=8),
              nn.Dropout(0.5))
        self.output = nn.Dense(classes)

    def forward(self, x):
        return self.output(self.features(x))


def inception_v3(pretrained=False, **kwargs):
    return Inception3(**{k: v for k, v in kwargs.items() if k not in ('ctx', 'device', 'root')})

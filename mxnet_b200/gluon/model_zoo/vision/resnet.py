"""ResNets V1/V2 (``python/mxnet/gluon/model_zoo/vision/resnet.py``) with two additions used by the
ImageNet benchmark: ``layout='NHWC'`` and the "v1b" bottleneck (stride in the 3×3 instead of the
first 1×1; the reference's ``BottleneckV1`` strides the first 1×1).  With ``fused=True`` the
BatchNorm+ReLU(+residual add) groups run as single kernels."""
from ....device import cpu
from ...block import HybridBlock
from ... import nn

__all__ = ['ResNetV1', 'ResNetV2', 'BasicBlockV1', 'BasicBlockV2', 'BottleneckV1', 'BottleneckV2', 'resnet18_v1',
           'resnet34_v1', 'resnet50_v1', 'resnet101_v1', 'resnet152_v1', 'resnet18_v2', 'resnet34_v2', 'resnet50_v2',
           'resnet101_v2', 'resnet152_v2', 'resnet50_v1b', 'get_resnet']


def _conv3x3(channels, stride, in_channels, layout):
    return nn.Conv2D(channels, kernel_size=3, strides=stride, padding=1, use_bias=False, in_channels=in_channels,
                     layout=layout)


def _bn_axis(layout):
    return 3 if layout == 'NHWC' else 1


class BasicBlockV1(HybridBlock):
    def __init__(self, channels, stride, downsample=False, in_channels=0, layout='NCHW', fused=False, **kwargs):
        super().__init__()
        ax = _bn_axis(layout)
        self.fused = fused
        self.conv1 = _conv3x3(channels, stride, in_channels, layout)
        self.bn1 = (nn.BatchNormReLU if fused else nn.BatchNorm)(axis=ax)
        self.conv2 = _conv3x3(channels, 1, channels, layout)
        self.bn2 = (nn.BatchNormReLU if fused else nn.BatchNorm)(axis=ax)
        if downsample:
            self.ds_conv = nn.Conv2D(channels, kernel_size=1, strides=stride, use_bias=False, in_channels=in_channels,
                                     layout=layout)
            self.ds_bn = nn.BatchNorm(axis=ax)
        else:
            self.ds_conv = None

    def forward(self, x):
        from ....ops import registry as _reg
        residual = x
        if self.ds_conv is not None:
            residual = self.ds_bn(self.ds_conv(x))
        if self.fused:
            out = self.bn1(self.conv1(x))
            return self.bn2(self.conv2(out), residual)
        out = _reg.invoke('Activation', [self.bn1(self.conv1(x))], {'act_type': 'relu'})
        out = self.bn2(self.conv2(out))
        return _reg.invoke('Activation', [out + residual], {'act_type': 'relu'})


class BottleneckV1(HybridBlock):
    def __init__(self, channels, stride, downsample=False, in_channels=0, layout='NCHW', fused=False, v1b=False, **kwargs):
        super().__init__()
        ax = _bn_axis(layout)
        self.fused = fused
        s1, s2 = (1, stride) if v1b else (stride, 1)
        BN = nn.BatchNormReLU if fused else nn.BatchNorm
        self.conv1 = nn.Conv2D(channels // 4, kernel_size=1, strides=s1, use_bias=False, in_channels=in_channels, layout=layout)
        self.bn1 = BN(axis=ax)
        self.conv2 = _conv3x3(channels // 4, s2, channels // 4, layout)
        self.bn2 = BN(axis=ax)
        self.conv3 = nn.Conv2D(channels, kernel_size=1, strides=1, use_bias=False, in_channels=channels // 4, layout=layout)
        self.bn3 = BN(axis=ax)
        if downsample:
            self.ds_conv = nn.Conv2D(channels, kernel_size=1, strides=stride, use_bias=False, in_channels=in_channels,
                                     layout=layout)
            self.ds_bn = nn.BatchNorm(axis=ax)
        else:
            self.ds_conv = None

    def forward(self, x):
        from ....ops import registry as _reg
        residual = x
        if self.ds_conv is not None:
            residual = self.ds_bn(self.ds_conv(x))
        if self.fused:
            if self.ds_conv is None and self.conv1._kwargs.get('stride') in ((1, 1), 1):
                # identity block: the convolution and the skip connection leave the same tensor as one operator, so the
                # backward pass adds the skip gradient inside the data-gradient kernel
                out, residual = _reg.invoke('_contrib_conv_skip', [x, self.conv1.weight.data(x.context)],
                                            {k: v for k, v in self.conv1._kwargs.items() if k != 'no_bias'})
                out = self.bn1(out)
            else:
                out = self.bn1(self.conv1(x))
            out = self.bn2(self.conv2(out))
            return self.bn3(self.conv3(out), residual)
        relu = lambda t: _reg.invoke('Activation', [t], {'act_type': 'relu'})
        out = relu(self.bn1(self.conv1(x)))
        out = relu(self.bn2(self.conv2(out)))
        out = self.bn3(self.conv3(out))
        return relu(out + residual)


class BasicBlockV2(HybridBlock):
    def __init__(self, channels, stride, downsample=False, in_channels=0, layout='NCHW', **kwargs):
        super().__init__()
        ax = _bn_axis(layout)
        self.bn1 = nn.BatchNorm(axis=ax)
        self.conv1 = _conv3x3(channels, stride, in_channels, layout)
        self.bn2 = nn.BatchNorm(axis=ax)
        self.conv2 = _conv3x3(channels, 1, channels, layout)
        self.downsample = nn.Conv2D(channels, 1, stride, use_bias=False, in_channels=in_channels, layout=layout) \
            if downsample else None

    def forward(self, x):
        from ....ops import registry as _reg
        relu = lambda t: _reg.invoke('Activation', [t], {'act_type': 'relu'})
        residual = x
        x = relu(self.bn1(x))
        if self.downsample is not None:
            residual = self.downsample(x)
        x = self.conv1(x)
        x = relu(self.bn2(x))
        x = self.conv2(x)
        return x + residual


class BottleneckV2(HybridBlock):
    def __init__(self, channels, stride, downsample=False, in_channels=0, layout='NCHW', **kwargs):
        super().__init__()
        ax = _bn_axis(layout)
        self.bn1 = nn.BatchNorm(axis=ax)
        self.conv1 = nn.Conv2D(channels // 4, kernel_size=1, strides=1, use_bias=False, layout=layout)
        self.bn2 = nn.BatchNorm(axis=ax)
        self.conv2 = _conv3x3(channels // 4, stride, channels // 4, layout)
        self.bn3 = nn.BatchNorm(axis=ax)
        self.conv3 = nn.Conv2D(channels, kernel_size=1, strides=1, use_bias=False, layout=layout)
        self.downsample = nn.Conv2D(channels, 1, stride, use_bias=False, in_channels=in_channels, layout=layout) \
            if downsample else None

    def forward(self, x):
        from ....ops import registry as _reg
        relu = lambda t: _reg.invoke('Activation', [t], {'act_type': 'relu'})
        residual = x
        x = relu(self.bn1(x))
        if self.downsample is not None:
            residual = self.downsample(x)
        x = self.conv1(x)
        x = relu(self.bn2(x))
        x = self.conv2(x)
        x = relu(self.bn3(x))
        x = self.conv3(x)
        return x + residual


class ResNetV1(HybridBlock):
    def __init__(self, block, layers, channels, classes=1000, thumbnail=False, layout='NCHW', fused=False, v1b=False,
                 **kwargs):
        super().__init__()
        assert len(layers) == len(channels) - 1
        ax = _bn_axis(layout)
        self.features = nn.HybridSequential()
        if thumbnail:
            self.features.add(_conv3x3(channels[0], 1, 0, layout))
        else:
            self.features.add(nn.Conv2D(channels[0], 7, 2, 3, use_bias=False, layout=layout))
            if fused:
                self.features.add(nn.BatchNormReLU(axis=ax))
            else:
                self.features.add(nn.BatchNorm(axis=ax))
                self.features.add(nn.Activation('relu'))
            self.features.add(nn.MaxPool2D(3, 2, 1, layout=layout))
        for i, num_layer in enumerate(layers):
            stride = 1 if i == 0 else 2
            self.features.add(self._make_layer(block, num_layer, channels[i + 1], stride, channels[i], layout, fused, v1b))
        self.features.add(nn.GlobalAvgPool2D(layout=layout))
        self.output = nn.Dense(classes, in_units=channels[-1])

    def _make_layer(self, block, layers, channels, stride, in_channels, layout, fused, v1b):
        layer = nn.HybridSequential()
        layer.add(block(channels, stride, channels != in_channels, in_channels=in_channels, layout=layout, fused=fused, v1b=v1b))
        for _ in range(layers - 1):
            layer.add(block(channels, 1, False, in_channels=channels, layout=layout, fused=fused, v1b=v1b))
        return layer

    def forward(self, x):
        x = self.features(x)
        return self.output(x)


class ResNetV2(HybridBlock):
    def __init__(self, block, layers, channels, classes=1000, thumbnail=False, layout='NCHW', **kwargs):
        super().__init__()
        assert len(layers) == len(channels) - 1
        ax = _bn_axis(layout)
        self.features = nn.HybridSequential()
        self.features.add(nn.BatchNorm(axis=ax, scale=False, center=False))
        if thumbnail:
            self.features.add(_conv3x3(channels[0], 1, 0, layout))
        else:
            self.features.add(nn.Conv2D(channels[0], 7, 2, 3, use_bias=False, layout=layout))
            self.features.add(nn.BatchNorm(axis=ax))
            self.features.add(nn.Activation('relu'))
            self.features.add(nn.MaxPool2D(3, 2, 1, layout=layout))
        in_channels = channels[0]
        for i, num_layer in enumerate(layers):
            stride = 1 if i == 0 else 2
            layer = nn.HybridSequential()
            layer.add(block(channels[i + 1], stride, channels[i + 1] != in_channels, in_channels=in_channels, layout=layout))
            for _ in range(num_layer - 1):
                layer.add(block(channels[i + 1], 1, False, in_channels=channels[i + 1], layout=layout))
            self.features.add(layer)
            in_channels = channels[i + 1]
        self.features.add(nn.BatchNorm(axis=ax))
        self.features.add(nn.Activation('relu'))
        self.features.add(nn.GlobalAvgPool2D(layout=layout))
        self.features.add(nn.Flatten())
        self.output = nn.Dense(classes, in_units=in_channels)

    def forward(self, x):
        x = self.features(x)
        return self.output(x)


resnet_spec = {18: ('basic_block', [2, 2, 2, 2], [64, 64, 128, 256, 512]),
               34: ('basic_block', [3, 4, 6, 3], [64, 64, 128, 256, 512]),
               50: ('bottle_neck', [3, 4, 6, 3], [64, 256, 512, 1024, 2048]),
               101: ('bottle_neck', [3, 4, 23, 3], [64, 256, 512, 1024, 2048]),
               152: ('bottle_neck', [3, 8, 36, 3], [64, 256, 512, 1024, 2048])}
resnet_net_versions = [ResNetV1, ResNetV2]
resnet_block_versions = [{'basic_block': BasicBlockV1, 'bottle_neck': BottleneckV1},
                         {'basic_block': BasicBlockV2, 'bottle_neck': BottleneckV2}]


def get_resnet(version, num_layers, pretrained=False, device=cpu(), root=None, ctx=None, **kwargs):
    assert num_layers in resnet_spec, 'Invalid number of layers: %d. Options are %s' % (num_layers, str(resnet_spec.keys()))
    block_type, layers, channels = resnet_spec[num_layers]
    assert 1 <= version <= 2, 'Invalid resnet version: %d. Options are 1 and 2.' % version
    net = resnet_net_versions[version - 1](resnet_block_versions[version - 1][block_type], layers, channels, **kwargs)
    if pretrained:
        from ..model_store import get_model_file
        net.load_parameters(get_model_file('resnet%d_v%d' % (num_layers, version), root=root), device=ctx or device)
    return net


def resnet18_v1(**kwargs): return get_resnet(1, 18, **kwargs)
def resnet34_v1(**kwargs): return get_resnet(1, 34, **kwargs)
def resnet50_v1(**kwargs): return get_resnet(1, 50, **kwargs)
def resnet101_v1(**kwargs): return get_resnet(1, 101, **kwargs)
def resnet152_v1(**kwargs): return get_resnet(1, 152, **kwargs)
def resnet18_v2(**kwargs): return get_resnet(2, 18, **kwargs)
def resnet34_v2(**kwargs): return get_resnet(2, 34, **kwargs)
def resnet50_v2(**kwargs): return get_resnet(2, 50, **kwargs)
def resnet101_v2(**kwargs): return get_resnet(2, 101, **kwargs)
def resnet152_v2(**kwargs): return get_resnet(2, 152, **kwargs)
def resnet50_v1b(**kwargs): return get_resnet(1, 50, v1b=True, **kwargs)

"""ResNet-50 v1b for the ImageNet training benchmark: bottleneck blocks [3, 4, 6, 3], widths
64/128/256/512 ×4, stride in the 3×3 convolution, NHWC activations, BatchNorm+ReLU(+residual add)
fused into single kernels, 1000-way classifier (25.6 M parameters)."""
from ..gluon.model_zoo.vision.resnet import ResNetV1, BottleneckV1, resnet_spec

ResNetV1b = ResNetV1


def resnet50_v1b(classes=1000, layout='NHWC', fused=True, **kwargs):
    _, layers, channels = resnet_spec[50]
    return ResNetV1(BottleneckV1, layers, channels, classes=classes, layout=layout, fused=fused, v1b=True, **kwargs)

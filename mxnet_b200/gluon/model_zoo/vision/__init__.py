"""``gluon.model_zoo.vision``: model constructors and ``get_model``."""
from .resnet import *    # noqa: F401,F403
from .others import *    # noqa: F401,F403
from . import resnet as _r, others as _o


def get_model(name, **kwargs):
    models = {}
    for mod in (_r, _o):
        for k in mod.__all__:
            v = getattr(mod, k)
            if callable(v) and k[0].islower():
                models[k] = v
    models.update({'mobilenetv2_1.0': _o.mobilenet_v2_1_0, 'mobilenetv2_0.75': _o.mobilenet_v2_0_75,
                   'mobilenetv2_0.5': _o.mobilenet_v2_0_5, 'mobilenetv2_0.25': _o.mobilenet_v2_0_25,
                   'mobilenet1.0': _o.mobilenet1_0, 'mobilenet0.75': _o.mobilenet0_75, 'mobilenet0.5': _o.mobilenet0_5,
                   'mobilenet0.25': _o.mobilenet0_25, 'squeezenet1.0': _o.squeezenet1_0, 'squeezenet1.1': _o.squeezenet1_1,
                   'inceptionv3': _o.inception_v3})
    name = name.lower()
    if name not in models:
        raise ValueError('Model %s is not supported. Available options are\n\t%s' % (name, '\n\t'.join(sorted(models.keys()))))
    return models[name](**kwargs)

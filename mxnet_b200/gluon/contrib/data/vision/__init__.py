"""Image classification / detection loaders and box-aware transforms (``python/mxnet/gluon/contrib/data/vision``)."""
from . import transforms   # noqa: F401
from .dataloader import (create_image_augment, ImageDataLoader, create_bbox_augment, ImageBboxDataLoader,   # noqa: F401
                         BboxLabelTransform)

"""``mx.image``: decoding, resizing, augmenters and the Python image iterators
(``python/mxnet/image/image.py``, ``detection.py``).  JPEG/PNG decoding uses Pillow (the reference
uses OpenCV); decoded arrays are HWC uint8 in RGB order like ``mx.image.imdecode`` returns."""
from .image import *       # noqa: F401,F403
from .image import _decode_to_numpy
from . import detection
from .detection import *     # noqa: F401,F403
from .detection import ImageDetIter, CreateDetAugmenter

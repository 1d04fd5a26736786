"""``mx.contrib``: quantization, text utilities, tensorboard bridge, ONNX aliases."""
from . import quantization, text, tensorboard, io, tensorrt   # noqa: F401
from .. import onnx
from ..ndarray import contrib as ndarray   # noqa: F401
from ..ndarray import contrib as nd        # noqa: F401
from ..symbol import contrib as symbol      # noqa: F401
from ..symbol import contrib as sym         # noqa: F401

"""``gluon.nn`` layers."""
from ..block import *           # noqa: F401,F403  (Block, HybridBlock, SymbolBlock: `nn.HybridBlock` as in the reference)
from .activations import *     # noqa: F401,F403
from .basic_layers import *    # noqa: F401,F403
from .conv_layers import *     # noqa: F401,F403
from . import conv_layers as _cl
for _k in _cl.__all__:
    globals()[_k] = getattr(_cl, _k)

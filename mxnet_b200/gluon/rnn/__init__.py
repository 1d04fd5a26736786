"""``gluon.rnn``."""
from .rnn_cell import *        # noqa: F401,F403
from .rnn_layer import *       # noqa: F401,F403
from .conv_rnn_cell import *   # noqa: F401,F403
from . import conv_rnn_cell as _c
for _k in _c.__all__:
    globals()[_k] = getattr(_c, _k)

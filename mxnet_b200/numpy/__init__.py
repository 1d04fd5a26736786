"""``mx.np`` namespace."""
from .multiarray import *   # noqa: F401,F403
from . import multiarray as _ma
from .multiarray import ndarray, array, asarray
from . import linalg, random, fft   # noqa: F401

# re-export every public callable/constant of the implementation module (including the ones
# created in loops, which `import *` with __all__ would hide)
for _k, _v in list(vars(_ma).items()):
    if not _k.startswith('_') and _k not in globals():
        globals()[_k] = _v
for _k in ('sum', 'max', 'min', 'all', 'any', 'abs', 'round', 'bool', 'pad', 'shape', 'size', 'copy'):
    globals()[_k] = getattr(_ma, _k)
del _k, _v

"""``mx.amp``: automatic mixed precision."""
from .amp import *          # noqa: F401,F403
from .amp import _reset
from .loss_scaler import LossScaler

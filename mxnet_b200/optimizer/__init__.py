"""``mx.optimizer``."""
from .optimizer import *          # noqa: F401,F403
from .optimizer import Optimizer, Test, create, register
from .updater import Updater, get_updater
from . import optimizer, updater   # noqa: F401

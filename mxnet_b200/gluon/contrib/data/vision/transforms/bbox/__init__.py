"""Transforms that move an image and its bounding boxes together, and the box arithmetic behind them."""
from .bbox import *    # noqa: F401,F403
from .utils import *   # noqa: F401,F403

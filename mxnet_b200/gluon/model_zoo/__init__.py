"""``gluon.model_zoo``."""
from . import model_store, vision
from .vision import get_model

"""``gluon.contrib.data``: data loaders and transforms beyond the core ``gluon.data`` package."""
from . import vision   # noqa: F401

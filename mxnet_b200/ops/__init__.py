"""Operator library.  Importing this package populates the registry (the counterpart of the static
``NNVM_REGISTER_OP`` initialisers run when the reference's shared library is loaded)."""
from . import registry
from .registry import register, get, has, list_ops, invoke, make_frontend, OpDef
from . import tensor, nn, optimizer_ops, random, contrib, image_ops, sparse_ops, numpy_ops  # noqa: F401
from . import extra_ops  # noqa: F401,E402

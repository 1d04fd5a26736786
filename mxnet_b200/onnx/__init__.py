"""ONNX export (``python/mxnet/onnx``): ``export_model`` turns a Symbol and its parameters into an ONNX file written by
an in-tree protobuf writer (no ``onnx`` package needed); ``backend.run_model`` evaluates such a file with the tensor
library so that an export can be checked against the network it came from."""
from .mx2onnx import export_model, get_operator_support, register   # noqa: F401
from . import backend                                               # noqa: F401
from .backend import run_model                                      # noqa: F401

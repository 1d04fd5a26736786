"""ONNX export (``python/mxnet/onnx/mx2onnx``): Symbol + params → ONNX ModelProto.  Needs the ``onnx``
package at call time; the operator translation table covers the layers of the model zoo."""
from .mx2onnx import export_model, get_operator_support

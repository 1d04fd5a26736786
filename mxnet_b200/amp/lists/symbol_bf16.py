"""Operator lists of the bf16 AMP policy (``python/mxnet/amp/lists/symbol_bf16.py``)."""
from .symbol_fp16 import FP16_FUNCS as BF16_FUNCS, FP32_FUNCS, FP16_FP32_FUNCS as BF16_FP32_FUNCS, WIDEST_TYPE_CASTS, \
    CONDITIONAL_FP32_FUNCS, LOSS_OUTPUT_FUNCTIONS   # noqa: F401

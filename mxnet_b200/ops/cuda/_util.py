"""Helpers shared by the kernel wrappers."""
import torch

from . import lib, ptr, stream_ptr, count_launch, check

DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def dt(t):
    return DT[t.dtype]


def f32(t):
    """fp32 contiguous view/copy of a small per-channel tensor."""
    return t if (t.dtype == torch.float32 and t.is_contiguous()) else t.float().contiguous()

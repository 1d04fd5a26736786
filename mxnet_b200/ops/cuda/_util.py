"""Helpers shared by the kernel wrappers."""
import torch

from . import lib, ptr, stream_ptr, count_launch, check

DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def dt(t):
    return DT[t.dtype]


def f32(t):
    """fp32 contiguous view/copy of a small per-channel tensor."""
    return t if (t.dtype == torch.float32 and t.is_contiguous()) else t.float().contiguous()


def require(t, name, numel=None, dtype=None, device=None, shape=None):
    """Validate one kernel operand before its raw pointer crosses the C boundary: the kernels index
    from the sizes they are told, so a mis-sized or misplaced tensor must fail here, in Python."""
    if t is None:
        raise ValueError('%s is required' % name)
    if not t.is_cuda:
        raise ValueError('%s must live on a CUDA device' % name)
    if device is not None and t.device != device:
        raise ValueError('%s is on %s, expected %s' % (name, t.device, device))
    if not t.is_contiguous():
        raise ValueError('%s must be contiguous' % name)
    if dtype is not None and t.dtype != dtype:
        raise ValueError('%s has dtype %s, expected %s' % (name, t.dtype, dtype))
    if numel is not None and t.numel() != numel:
        raise ValueError('%s has %d elements, expected %d' % (name, t.numel(), numel))
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise ValueError('%s has shape %s, expected %s' % (name, tuple(t.shape), tuple(shape)))
    return t


def job_wide(choice):
    """The autotuning verdict of rank 0 for every rank of a multi-process job: each rank times the candidates itself (so
    all of them reach this point together, after the same work), then adopts rank 0's choice, so that one layer runs the
    same kernel, with the same rounding, on every GPU of the job.  A single process returns its own verdict."""
    from ...parallel import dist
    if not dist.is_initialized() or dist.world_size() < 2:
        return bool(choice)
    flag = torch.tensor([1 if choice else 0], dtype=torch.int32, device='cuda')
    dist.broadcast_(flag, 0)
    return bool(int(flag.item()))

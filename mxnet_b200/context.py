"""Legacy alias module (``python/mxnet/context.py``): Context == Device."""
from .device import *          # noqa: F401,F403
from .device import Device, Context, cpu, gpu, cpu_pinned, cpu_shared, num_gpus, gpu_memory_info, current_device, current_context

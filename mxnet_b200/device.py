"""Device (a.k.a. Context) objects.

Reference: ``python/mxnet/device.py`` / ``context.py`` and the on-disk encoding of
``include/mxnet/base.h:147-150`` (``dev_type`` cpu=1, gpu=2, cpu_pinned=3, cpu_shared=5).
A Device is a (type, id) pair with a thread-local "current device" stack.  Several CPU device
ids are allowed (``mx.cpu(0)``, ``mx.cpu(1)``): they share host memory but are distinct
replicas for Gluon parameters and KVStore, which is how data-parallel logic is tested
without GPUs.
"""
import threading

import torch

__all__ = ['Device', 'Context', 'cpu', 'gpu', 'cpu_pinned', 'cpu_shared', 'num_gpus',
           'gpu_memory_info', 'current_device', 'current_context']


class Device(object):
    """A device on which arrays live and operators run."""
    _default = threading.local()
    devtype2str = {1: 'cpu', 2: 'gpu', 3: 'cpu_pinned', 5: 'cpu_shared'}
    devstr2type = {'cpu': 1, 'gpu': 2, 'cpu_pinned': 3, 'cpu_shared': 5}

    def __init__(self, device_type, device_id=0):
        if isinstance(device_type, Device):
            self.device_typeid = device_type.device_typeid
            self.device_id = device_type.device_id
        else:
            if device_type == 'cuda':
                device_type = 'gpu'
            self.device_typeid = Device.devstr2type[device_type]
            self.device_id = int(device_id)
        self._old_ctx = None

    @property
    def device_type(self):
        return Device.devtype2str[self.device_typeid]

    def __hash__(self):
        return hash((self.device_typeid, self.device_id))

    def __eq__(self, other):
        return isinstance(other, Device) and self.device_typeid == other.device_typeid \
            and self.device_id == other.device_id

    def __str__(self):
        return '%s(%d)' % (self.device_type, self.device_id)

    __repr__ = __str__

    def __enter__(self):
        stack = getattr(Device._default, 'stack', None)
        if stack is None:
            stack = Device._default.stack = []
        stack.append(self)
        return self

    def __exit__(self, ptype, value, trace):
        Device._default.stack.pop()

    @property
    def torch_device(self):
        """The torch.device that backs this Device."""
        if self.device_typeid == 2:
            return torch.device('cuda', self.device_id)
        return torch.device('cpu')

    def empty_cache(self):
        """Release cached device memory back to the driver (``MXStorageEmptyCache``)."""
        if self.device_typeid == 2 and torch.cuda.is_available():
            with torch.cuda.device(self.device_id):
                torch.cuda.empty_cache()


Context = Device


def cpu(device_id=0):
    return Device('cpu', device_id)


def cpu_pinned(device_id=0):
    return Device('cpu_pinned', device_id)


def cpu_shared(device_id=0):
    return Device('cpu_shared', device_id)


def gpu(device_id=0):
    return Device('gpu', device_id)


def num_gpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def gpu_memory_info(device_id=0):
    """(free, total) bytes of a GPU (``MXGetGPUMemoryInformation64``)."""
    free, total = torch.cuda.mem_get_info(device_id)
    return int(free), int(total)


def current_device():
    stack = getattr(Device._default, 'stack', None)
    if stack:
        return stack[-1]
    base = getattr(Device, '_process_default', None)
    return base if base is not None else Device('cpu', 0)


current_context = current_device


def set_default_device(dev):
    """Process-wide default (used by GPU test modules that re-run the CPU suite)."""
    Device._process_default = Device(dev)


def from_torch_device(tdev):
    tdev = torch.device(tdev)
    if tdev.type == 'cuda':
        return Device('gpu', tdev.index or 0)
    return Device('cpu', 0)

"""All-reduce of small fp32 vectors over NVLink peer memory (``ops/cuda/peer_reduce.cu``).

Used for the batch statistics of SyncBatchNorm (a few KB per layer): one kernel stores the vector into every rank's
receive area, publishes a flag and waits (bounded) for the other ranks, instead of a library collective per layer.
One process per GPU on one node; the receive areas are shared through CUDA IPC at first use."""
import ctypes as C

import torch

from . import dist
from .. import env
from ..base import MXNetError

_instances = {}


def _lib():
    from ..ops import cuda
    return cuda.lib()


def available(device):
    """Peer all-reduce is used for CUDA tensors of an initialised NCCL group that fits one node's fused path."""
    if not (device.type == 'cuda' and dist.is_initialized() and env.get('MXNET_KVSTORE_FUSED')):
        return False
    if dist.backend() != 'nccl':
        return False
    from ..ops import cuda
    return cuda.available() and dist.world_size() <= _lib().mxb_peer_max_ranks()


def get(device, cap=8192):
    """The process-wide instance for `device` (vectors of up to `cap` floats)."""
    key = (device.index, cap)
    inst = _instances.get(key)
    if inst is None:
        inst = _instances[key] = PeerAllReduce(device, cap)
    return inst


class PeerAllReduce(object):
    def __init__(self, device, cap=8192):
        L = _lib()
        self.device, self.cap = device, int(cap)
        self.rank, self.nranks = dist.rank(), dist.world_size()
        self.step = 0
        torch.cuda.set_device(device)
        nbytes = L.mxb_peer_slab_bytes(self.cap)
        ptr = C.c_void_p()
        rc = L.mxb_dev_alloc(C.byref(ptr), nbytes)
        if rc != 0:
            raise MXNetError('cudaMalloc of the peer receive area failed: %s' % L.mxb_error_string(rc).decode())
        self.slab = ptr.value
        self.peers = [self.slab] * self.nranks
        self._opened = []
        if self.nranks > 1:
            handle = C.create_string_buffer(L.mxb_ipc_handle_bytes())
            rc = L.mxb_ipc_get_handle(C.c_void_p(self.slab), handle)
            if rc != 0:
                raise MXNetError('cudaIpcGetMemHandle failed: %s' % L.mxb_error_string(rc).decode())
            for r, (h, cap_r) in enumerate(dist.all_gather_object((handle.raw, self.cap))):
                if cap_r != self.cap:
                    raise MXNetError('rank %d uses a different receive-area size' % r)
                if r == self.rank:
                    continue
                p2 = C.c_void_p()
                rc = L.mxb_ipc_open(C.c_char_p(h), C.byref(p2))
                if rc != 0:
                    raise MXNetError('cudaIpcOpenMemHandle(rank %d) failed: %s' % (r, L.mxb_error_string(rc).decode()))
                self.peers[r] = p2.value
                self._opened.append(p2.value)
        self._slabs = (C.c_void_p * self.nranks)(*self.peers)
        self._status_off = L.mxb_peer_status_offset()

    def allreduce(self, vec):
        """Sum of `vec` (1-D fp32, at most `cap` elements) over all ranks; bit-identical on every rank."""
        from ..ops import cuda
        if vec.dtype != torch.float32 or vec.dim() != 1 or not vec.is_contiguous() or vec.numel() > self.cap or vec.numel() < 1:
            raise ValueError('peer all-reduce takes a contiguous 1-D fp32 tensor of at most %d elements' % self.cap)
        if vec.device != self.device:
            raise ValueError('tensor is on %s, the receive area on %s' % (vec.device, self.device))
        out = torch.empty_like(vec)
        self.step += 1
        timeout_ns = int(env.get('MXNET_KVSTORE_WAIT_MS')) * 1000000
        rc = _lib().mxb_peer_allreduce(self._slabs, self.rank, self.nranks, self.cap, C.c_void_p(vec.data_ptr()),
                                       C.c_void_p(out.data_ptr()), vec.numel(), self.step & 0xffffffff, timeout_ns,
                                       cuda.stream_ptr(self.device))
        if rc != 0:
            raise MXNetError('peer all-reduce launch failed with CUDA error %d' % rc)
        cuda.count_launch(1)
        return out

    def status(self):
        """1 when a wait for the other ranks ran out since the last call (the sums are then incomplete); clears it."""
        buf = torch.zeros(1, dtype=torch.int32, device=self.device)
        L = _lib()
        src = C.c_void_p(self.slab + self._status_off)
        torch.cuda.synchronize(self.device)
        host = C.c_uint32(0)
        L.mxb_memcpy_d2h(C.byref(host), src, 4, None)
        torch.cuda.synchronize(self.device)
        if host.value:
            zero = C.c_uint32(0)
            L.mxb_memcpy_h2d(src, C.byref(zero), 4, None)
            torch.cuda.synchronize(self.device)
        del buf
        return int(host.value)

    def __del__(self):
        try:
            L = _lib()
            for p in self._opened:
                L.mxb_ipc_close(C.c_void_p(p))
        except Exception:  # pylint: disable=broad-except
            pass

"""Process-group plumbing: one process per GPU over ``torch.distributed`` (NCCL on GPUs, gloo on
CPU ranks), plus host-side liveness tracking.

The reference's multi-process modes are a ZeroMQ parameter server (``src/kvstore/kvstore_dist.h``)
with heartbeats behind ``get_num_dead_node``; here ranks are peers.  Liveness: every rank bumps a
counter in the rendezvous store from a background thread; a rank whose counter has not moved for
``timeout`` seconds counts as dead.  Nothing here touches a GPU, so failure handling is testable
with CPU ranks.
"""
from __future__ import annotations

import datetime
import os
import threading
import time

import torch
import torch.distributed as tdist

_hb = {'thread': None, 'stop': False, 'store': None}


def is_initialized():
    return tdist.is_available() and tdist.is_initialized()


def ensure_initialized(backend=None, timeout_s=None):
    """Initialise from the torchrun/launcher environment (RANK, WORLD_SIZE, MASTER_ADDR, MASTER_PORT or
    the reference's DMLC_* names).  A single process without those variables stays uninitialised."""
    if is_initialized():
        return True
    env = os.environ
    if 'RANK' not in env and 'DMLC_WORKER_ID' in env:
        env['RANK'] = env['DMLC_WORKER_ID']
        env['WORLD_SIZE'] = env.get('DMLC_NUM_WORKER', '1')
        env.setdefault('MASTER_ADDR', env.get('DMLC_PS_ROOT_URI', '127.0.0.1'))
        env.setdefault('MASTER_PORT', env.get('DMLC_PS_ROOT_PORT', '29500'))
    if 'RANK' not in env or 'WORLD_SIZE' not in env:
        return False
    env.setdefault('MASTER_ADDR', '127.0.0.1')
    env.setdefault('MASTER_PORT', '29500')
    if backend is None:
        backend = 'nccl' if torch.cuda.is_available() else 'gloo'
    if backend == 'nccl':
        torch.cuda.set_device(local_rank())
    kw = {}
    if timeout_s is not None:
        kw['timeout'] = datetime.timedelta(seconds=timeout_s)
    if backend == 'nccl':
        kw['device_id'] = torch.device('cuda', local_rank())
    tdist.init_process_group(backend=backend, **kw)
    return True


def backend():
    return tdist.get_backend() if is_initialized() else None


def rank():
    return tdist.get_rank() if is_initialized() else 0


def world_size():
    return tdist.get_world_size() if is_initialized() else 1


def local_rank():
    return int(os.environ.get('LOCAL_RANK', os.environ.get('RANK', '0'))) if torch.cuda.device_count() == 0 else \
        int(os.environ.get('LOCAL_RANK', '0')) % max(torch.cuda.device_count(), 1)


def barrier():
    if is_initialized():
        if torch.cuda.is_available() and tdist.get_backend() == 'nccl':
            tdist.barrier(device_ids=[torch.cuda.current_device()])
        else:
            tdist.barrier()


def all_reduce_sum(t):
    """In-place sum over ranks; half precision is summed as is (NCCL accumulates in fp32 internally)."""
    if not t.is_contiguous():
        t = t.contiguous()
    if t.dtype == torch.bool:
        x = t.to(torch.int32)
        tdist.all_reduce(x)
        return x.bool()
    if tdist.get_backend() == 'gloo' and t.dtype == torch.bfloat16:
        x = t.float()
        tdist.all_reduce(x)
        return x.to(torch.bfloat16)
    tdist.all_reduce(t)
    return t


def all_gather_tensor(t):
    """The tensor ``t`` of every rank (same shape and dtype everywhere), as a list in rank order."""
    parts = [torch.empty_like(t) for _ in range(world_size())]
    tdist.all_gather(parts, t.contiguous())
    return parts


def broadcast_(t, src=0):
    tdist.broadcast(t, src)
    return t


def all_gather_object(obj):
    out = [None] * world_size()
    tdist.all_gather_object(out, obj)
    return out


def destroy():
    stop_heartbeat()
    if is_initialized():
        tdist.destroy_process_group()


# ---- liveness ----------------------------------------------------------------------------------
def _store():
    if _hb['store'] is None and is_initialized():
        _hb['store'] = tdist.distributed_c10d._get_default_store()
    return _hb['store']


def start_heartbeat(interval=0.5):
    """Bump ``hb/<rank>`` in the rendezvous store every ``interval`` seconds."""
    if _hb['thread'] is not None or not is_initialized():
        return
    st = _store()
    r = rank()
    _hb['stop'] = False

    def loop():
        while not _hb['stop']:
            try:
                st.set('hb/%d' % r, str(time.time()))
            except Exception:  # pylint: disable=broad-except
                return
            time.sleep(interval)
    th = threading.Thread(target=loop, name='mxb-heartbeat', daemon=True)
    _hb['thread'] = th
    th.start()


def stop_heartbeat():
    _hb['stop'] = True
    th = _hb['thread']
    if th is not None:
        th.join(timeout=2)
    _hb['thread'] = None


def num_dead_nodes(timeout=60):
    """Ranks whose last heartbeat is older than ``timeout`` seconds (never-seen ranks count)."""
    if not is_initialized():
        return 0
    st = _store()
    now, dead = time.time(), 0
    for r in range(world_size()):
        key = 'hb/%d' % r
        try:
            if hasattr(st, 'check') and not st.check([key]):
                dead += 1
                continue
            last = float(st.get(key).decode())
            if now - last > timeout:
                dead += 1
        except Exception:  # pylint: disable=broad-except
            dead += 1
    return dead


def _small_allreduce(t):
    """Sum of a small fp32 tensor over the ranks: the peer-memory kernel on one NVLink node, else the library."""
    from . import peer_reduce
    if t.dtype == torch.float32 and t.is_cuda and peer_reduce.available(t.device):
        flat = t.contiguous().reshape(-1)
        pr = peer_reduce.get(t.device)
        if flat.numel() <= pr.cap:
            return pr.allreduce(flat).reshape(t.shape)
    t = t.contiguous()
    tdist.all_reduce(t)
    return t


class SyncMoments(torch.autograd.Function):
    """Mean/variance over the batch of every rank (SyncBatchNorm statistics) with exact gradients."""

    @staticmethod
    def forward(ctx, x, red):
        n_local = 1
        for a in red:
            n_local *= x.shape[a]
        s = torch.stack([x.sum(red), (x * x).sum(red)])
        # every rank contributes the same number of rows in data-parallel training; unequal batches take the general
        # path with the counts reduced as well
        n = float(n_local) * world_size()
        s = _small_allreduce(s)
        mean = s[0] / n
        var = s[1] / n - mean * mean
        ctx.save_for_backward(x, mean)
        ctx.red, ctx.n = red, n
        return mean, var

    @staticmethod
    def backward(ctx, gmean, gvar):
        x, mean = ctx.saved_tensors
        g = _small_allreduce(torch.stack([gmean, gvar]))
        shape = [1] * x.dim()
        for i in range(x.dim()):
            if i not in ctx.red:
                shape[i] = x.shape[i]
        gm, gv = g[0].reshape(shape), g[1].reshape(shape)
        gx = gm / ctx.n + gv * 2.0 * (x - mean.reshape(shape)) / ctx.n
        return gx, None

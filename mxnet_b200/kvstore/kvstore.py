"""Native KVStore: ``local`` / ``device`` / ``nccl`` / ``dist_*`` semantics.

Reference: ``src/kvstore/kvstore_local.h`` (``PushImpl :232-277``, ``PullImpl :279-306``,
``GroupKVPairs :436-465``), ``comm.h`` (CPU tree-sum ``:388-441``; device gather→sum→broadcast
``:535-654``), ``kvstore_nccl.h`` (Reduce/Bcast), ``kvstore_dist.h`` (parameter server) and the
Python wrapper ``python/mxnet/kvstore/kvstore.py``.

Checklist kept: ``init`` once per key; ``push`` sums all values given for a key (list = one per
device) then runs the updater ``(key, merged, stored)`` or overwrites; ``pull`` copies the stored
value to every output; ``pushpull(key, value, out=None)`` defaults out to value; ``broadcast`` =
init + pull; int or str keys, never mixed; higher ``priority`` first; ``nccl`` rejects sparse
values and compression.

Process model: inside one process a key may carry several replicas (one per device, CPU ids
included).  Across processes (one per GPU, ``torch.distributed`` initialised) every store type
sums over all ranks; the ``device``/``nccl`` stores of a Trainer use the fused peer-memory kernels
of ``parallel.fused`` for dense half/float gradients and fall back to NCCL collectives otherwise.
"""
from __future__ import annotations

import pickle
from contextlib import nullcontext as _nullcontext

import torch

from .. import env
from ..base import MXNetError
from ..ndarray.ndarray import NDArray
from ..ndarray import sparse as _sparse
from ..optimizer import Updater, get_updater
from .base import KVStoreBase, _ctype_key_value
from .gradient_compression import GradientCompression

__all__ = ['KVStore']

_TYPES = ('local', 'device', 'nccl', 'dist_sync', 'dist_async', 'dist_device_sync', 'dist_sync_device', 'dist',
          'local_allreduce_cpu', 'local_allreduce_device', 'local_update_cpu', 'dist_p3', 'p3')


class KVStore(KVStoreBase):
    def __init__(self, name='local'):
        if name not in _TYPES:
            raise MXNetError('Unknown KVStore type "%s"' % name)
        self._type = name
        self._store = {}
        self._updater = None
        self._updater_func = None
        self._str_keys = None
        self._compression = None
        self._pending_remote = []     # (other CUDA device, event): copies of merged values onto replicas of that device
        self._pending = {}            # CUDA device -> event of the last reduction queued on its communication streams
        self.rows_pulled = 0          # rows moved by row_sparse_pull (observable by tests)
        self.wire_bytes = 0           # bytes of compressed gradients sent to other devices / ranks (observable by tests)
        self._barrier_before_exit = True
        from ..parallel import dist
        self._dist = dist
        self._server = self._client = None
        if name.startswith('dist') or name == 'p3':
            dist.ensure_initialized()
        if name == 'dist_async':
            self._connect_server()

    def _connect_server(self):
        """``dist_async``: a parameter server (``kvstore/server.py``, a thread in the process of rank 0) that applies
        every push on arrival, as the reference's servers do in async mode (kvstore_dist_server.h ApplyUpdates): no worker
        waits for another.  Every rank, rank 0 included, talks to it over its own connection."""
        from .server import ParameterServer, ServerClient
        world = self._dist.world_size() if self._dist.is_initialized() else 1
        address = None
        if self.rank == 0:
            self._server = ParameterServer(world, sync_mode=False)
            address = self._server.address
        if world > 1:
            address = [a for a in self._dist.all_gather_object(address) if a is not None][0]
        self._client = ServerClient(address)

    # ------------------------------------------------------------------ properties
    @property
    def type(self):
        return self._type

    @property
    def rank(self):
        return self._dist.rank() if self._dist.is_initialized() else 0

    @property
    def num_workers(self):
        return self._dist.world_size() if self._dist.is_initialized() else 1

    @staticmethod
    def is_capable(capability):
        if capability.lower() == KVStoreBase.OPTIMIZER:
            return True
        raise ValueError('Unknown capability: {}'.format(capability))

    # ------------------------------------------------------------------ helpers
    def _check_key(self, k):
        is_str = isinstance(k, str)
        if self._str_keys is None:
            self._str_keys = is_str
        elif self._str_keys != is_str:
            raise MXNetError('inconsistent key types: string and integer keys cannot be mixed')

    def _group(self, key, value):
        """GroupKVPairs: duplicate keys are merged into per-key value lists."""
        if isinstance(key, (list, tuple)):
            if value is not None and len(key) != len(value):
                raise MXNetError('key and value lists differ in length')
            grouped, order = {}, []
            for i, k in enumerate(key):
                self._check_key(k)
                v = value[i] if value is not None else None
                if k not in grouped:
                    grouped[k] = []
                    order.append(k)
                if isinstance(v, (list, tuple)):
                    grouped[k].extend(v)
                elif v is not None:
                    grouped[k].append(v)
            return [(k, grouped[k]) for k in order]
        self._check_key(key)
        if value is None:
            return [(key, [])]
        return [(key, list(value) if isinstance(value, (list, tuple)) else [value])]

    # ---- communication streams: the key's priority picks the stream its reduction runs on ------------------------
    _URGENT = -8        # the Trainer pushes parameter i with priority -i: the first few are needed first by the next forward

    def _comm_stream(self, dev, priority):
        """The side stream for a reduction whose merge buffer lives on the CUDA device ``dev``: high priority for the
        keys the next forward pass needs first, low for the rest (src/engine/threaded_engine_perdevice.cc gives copy
        operations their own prioritised workers).  The stream starts after everything queued so far on the compute
        stream (the backward pass that produced the values)."""
        from .. import engine
        st = engine.streams(dev)
        comm = st.comm_high if priority >= self._URGENT else st.comm_low
        comm.wait_stream(torch.cuda.current_stream(dev))
        return comm

    def wait_pending(self):
        """Make the compute streams wait (on the device, not the host) for the reductions still running on the
        communication streams; called before anything consumes the merged values."""
        for dev, ev in self._pending.items():
            torch.cuda.current_stream(dev).wait_event(ev)
        for dev, ev in self._pending_remote:
            torch.cuda.current_stream(dev).wait_event(ev)
        self._pending.clear()
        del self._pending_remote[:]

    def _reduce(self, key, values, target_ctx=None, priority=0):
        """Sum replicas on the device of the stored value (merge buffer), then across ranks."""
        if self._type == 'nccl':
            for v in values:
                if getattr(v, '_stype', 'default') != 'default':
                    raise MXNetError('kvstore nccl does not support sparse values')
        first = values[0]
        dev = first._data.device
        side = dev.type == 'cuda' and len(values) > 1 and not torch.cuda.is_current_stream_capturing()
        if not side:
            return self._reduce_on_current(key, values)
        comm = self._comm_stream(dev, priority)
        for v in values:                          # replicas on other GPUs: their producers must have finished too
            if v._data.is_cuda and v._data.device != dev:
                comm.wait_stream(torch.cuda.current_stream(v._data.device))
        with torch.cuda.stream(comm):
            merged = self._reduce_on_current(key, values)
            for v in values:
                v._data.record_stream(comm)
        ev = torch.cuda.Event()
        ev.record(comm)
        self._pending[dev] = ev                   # later reductions on this device are ordered after this one or ahead of it
        merged._data.record_stream(torch.cuda.current_stream(dev))
        return merged

    def _reduce_on_current(self, key, values):
        first = values[0]
        dev = first._data.device
        if self._compression is not None and first._data.dtype == torch.float32:
            # what crosses to the merge device are the packed 2-bit / 1-bit codes (a sixteenth / thirty-second of the
            # bytes); they are expanded where they are summed (src/kvstore/comm.h Reduce with gradient compression)
            n, shape = first._data.numel(), first._data.shape
            parts = []
            for i, v in enumerate(values):
                packed = self._compression.quantize((key, i), v._data).to(torch.int32)      # 32-bit words on the wire
                self.wire_bytes += packed.numel() * packed.element_size() if v._data.device != dev else 0
                parts.append(self._compression.dequantize(packed.to(dev, non_blocking=True), n, torch.float32).reshape(shape))
        else:
            parts = [v._data if v._data.device == dev else v._data.to(dev, non_blocking=True) for v in values]
        if len(parts) == 1:
            merged = parts[0].clone() if self._dist.is_initialized() and self._dist.world_size() > 1 else parts[0]
        else:
            acc = parts[0].float() if parts[0].dtype in (torch.float16, torch.bfloat16) else parts[0].clone()
            for p in parts[1:]:
                acc.add_(p.to(acc.dtype))
            merged = acc.to(parts[0].dtype)
        if self._client is None and self._dist.is_initialized() and self._dist.world_size() > 1 and \
                (self._type.startswith('dist') or self._type in ('nccl', 'device', 'p3')):
            if self._compression is not None and merged.dtype == torch.float32:
                # between workers the packed codes travel as well: every rank gathers the others' words and expands them
                # (the reference's workers send compressed gradients to the server, which decompresses and sums)
                packed = self._compression.quantize((key, 'wire'), merged).to(torch.int32).contiguous()
                words = self._dist.all_gather_tensor(packed)
                self.wire_bytes += packed.numel() * packed.element_size() * (len(words) - 1)
                n, shape = merged.numel(), merged.shape
                merged = sum(self._compression.dequantize(w, n, torch.float32) for w in words).reshape(shape)
            else:
                merged = self._dist.all_reduce_sum(merged)
        cls = first.__class__ if not isinstance(first, _sparse.BaseSparseNDArray) else NDArray
        return cls._from_tensor(merged, first._ctx)

    # ------------------------------------------------------------------ API
    def init(self, key, value):
        for k, vals in self._group(key, value):
            if k in self._store:
                raise MXNetError('duplicate init of key %s' % str(k))
            v = vals[0]
            stored = v.__class__._from_tensor(v._data.detach().clone(), v._ctx)
            stored._stype = getattr(v, '_stype', 'default')
            if self._client is not None:
                self._client.init(k, stored._data)                    # the first value to arrive is kept
                stored._data.copy_(self._client.pull(k).to(stored._data.device))
            elif self._dist.is_initialized() and self._dist.world_size() > 1 and self._type != 'local':
                self._dist.broadcast_(stored._data, src=0)
            self._store[k] = stored

    def push(self, key, value, priority=0):
        for k, vals in self._group(key, value):
            if k not in self._store:
                raise MXNetError('key %s has not been initialized' % str(k))
            merged = self._reduce(k, vals, priority=priority)
            stored = self._store[k]
            if self._client is not None:
                self.wait_pending()
                self._client.push(k, merged._data)                   # applied by the server on arrival
                continue
            if self._updater is not None:
                self.wait_pending()
                if merged._data.device != stored._data.device:
                    merged = merged.as_in_context(stored._ctx)
                self._updater(k if not isinstance(k, str) else k, merged, stored)
            else:
                with torch.no_grad():
                    if stored._data.shape != merged._data.shape:
                        raise MXNetError('shape mismatch for key %s' % str(k))
                    stored._data.copy_(merged._data)

    def pull(self, key, out=None, priority=0, ignore_sparse=True):
        assert out is not None
        self.wait_pending()
        for k, outs in self._group(key, out):
            if k not in self._store:
                raise MXNetError('key %s has not been initialized' % str(k))
            stored = self._store[k]
            if self._client is not None:
                with torch.no_grad():
                    stored._data.copy_(self._client.pull(k).to(stored._data.device))     # whatever the server holds now
            for o in outs:
                if ignore_sparse and getattr(o, '_stype', 'default') != 'default':
                    continue
                with torch.no_grad():
                    o._data.copy_(stored._data, non_blocking=True)

    def pushpull(self, key, value, out=None, priority=0):
        if out is None:
            out = value
        if self._updater is None and self._client is None:
            # fast path without touching the stored value when no updater is installed
            for (k, vals), (_, outs) in zip(self._group(key, value), self._group(key, out)):
                merged = self._reduce(k, vals, priority=priority)
                dev = merged._data.device
                ev = self._pending.get(dev)
                # the copies back to the replicas stay on the communication stream of the reduction; the compute
                # streams pick the result up at `wait_pending` (the Trainer calls it once after the last key)
                comm = None
                if ev is not None and dev.type == 'cuda':
                    from .. import engine
                    st = engine.streams(dev)
                    comm = st.comm_high if priority >= self._URGENT else st.comm_low
                with torch.cuda.stream(comm) if comm is not None else _nullcontext():
                    with torch.no_grad():
                        if k in self._store and self._store[k]._data.shape == merged._data.shape:
                            self._store[k]._data.copy_(merged._data)
                        for o in outs:
                            if o._data is not merged._data:
                                o._data.copy_(merged._data, non_blocking=True)
                    if comm is not None:
                        ev = torch.cuda.Event()
                        ev.record(comm)
                        self._pending[dev] = ev
                        for o in outs:          # replicas on other GPUs wait for their copy as well
                            if o._data.is_cuda and o._data.device != dev:
                                self._pending_remote.append((o._data.device, ev))
            return
        self.push(key, value, priority)
        self.pull(key, out, priority)

    def broadcast(self, key, value, out, priority=0):
        for k, vals in self._group(key, value):
            if k not in self._store:
                self.init(k, vals[0])
            else:
                with torch.no_grad():
                    self._store[k]._data.copy_(vals[0]._data)
        self.pull(key, out=out, priority=priority)

    def row_sparse_pull(self, key, out=None, priority=0, row_ids=None):
        """Pull only the rows named by ``row_ids`` (unique, sorted on device like ``kvstore_utils.cu``)."""
        assert out is not None and row_ids is not None
        self.wait_pending()
        groups = self._group(key, out)
        if isinstance(row_ids, NDArray):
            row_ids = [row_ids]
        flat_ids = []
        for (k, outs) in groups:
            flat_ids.append([row_ids[min(len(flat_ids), len(row_ids) - 1)]] * len(outs) if len(row_ids) != len(outs)
                            else row_ids)
        for (k, outs), ids in zip(groups, flat_ids):
            stored = self._store[k]
            for o, rid in zip(outs, ids):
                # only the requested rows leave the store's device: unique ids (sorted on the device like
                # src/kvstore/kvstore_utils.cu), a gather of those rows, one copy, a scatter into the cleared output
                idx = torch.unique(rid._data.long().reshape(-1).to(stored._data.device))
                rows = stored._data.index_select(0, idx)
                with torch.no_grad():
                    o._data.zero_()
                    o._data.index_copy_(0, idx.to(o._data.device), rows.to(o._data.device, non_blocking=True))
                self.rows_pulled += int(idx.numel())

    def set_gradient_compression(self, compression_params):
        if self._type == 'nccl':
            raise MXNetError('Gradient compression is not supported for kvstore nccl')
        if self._type == 'local':
            raise MXNetError('Gradient compression is not supported for this type of kvstore')
        self._compression = GradientCompression(**compression_params)

    def set_optimizer(self, optimizer):
        """Install an optimizer: updates then run where the merged value lives (for ``dist_async``: on the server, which
        receives the pickled optimizer like the reference's servers do)."""
        if self._client is not None:
            self._client.set_optimizer(optimizer)
            if self._dist.is_initialized() and self._dist.world_size() > 1:
                self._dist.barrier()                                # no push before every server-side updater exists
            return
        self._set_updater(get_updater(optimizer))

    def _set_updater(self, updater):
        self._updater = updater

    def set_updater(self, updater):
        self._set_updater(updater)

    def save_optimizer_states(self, fname, dump_optimizer=False):
        assert self._updater is not None, 'Cannot save states for distributed training'
        with open(fname, 'wb') as fout:
            fout.write(self._updater.get_states(dump_optimizer))

    def load_optimizer_states(self, fname):
        assert self._updater is not None, 'Cannot load states for distributed training'
        with open(fname, 'rb') as f:
            self._updater.set_states(f.read())

    def barrier(self):
        from .. import engine
        engine.waitall()
        if self._dist.is_initialized():
            self._dist.barrier()

    _barrier = barrier

    def _send_command_to_servers(self, head, body):
        pass

    def get_num_dead_node(self, node_id=0, timeout=60):
        """Number of ranks whose heartbeat is older than ``timeout`` seconds (``kvstore.h:411``)."""
        return self._dist.num_dead_nodes(timeout) if self._dist.is_initialized() else 0

    def is_recovery(self):
        import os
        return os.environ.get('DMLC_IS_RECOVERY', '0') == '1'

    def set_barrier_before_exit(self, flag):
        self._barrier_before_exit = bool(flag)

"""Fused data-parallel optimizer step over peer memory (host side of ``ops/cuda/fused_step.cu``).

Replaces the per-parameter ``pushpull`` + ``multi_all_finite`` + ``multi_mp_sgd_mom_update`` + broadcast
sequence of the reference Trainer (``python/mxnet/gluon/trainer.py:392-486``) by two kernel launches
per step, with no NCCL call and no host synchronisation:

* all trainable parameters of the process are re-homed into one flat *weight arena* and their
  gradients into a *gradient arena* of identical layout (16-byte aligned segments), allocated with
  ``cudaMalloc`` so the memory can be opened by the other ranks through CUDA IPC;
* rank ``r`` owns shard ``r`` of the arena: fp32 master weights and momentum exist for that shard
  only (optimizer state memory is divided by the number of GPUs);
* ``step`` launches the reduce kernel (sum of this rank's shard over all ranks' gradient arenas,
  unscale, inf/nan + sum-of-squares) and the update kernel (global skip/clip decision, SGD-momentum or
  NAG on the master shard, new low-precision weights stored into every rank's arena, gradient arena
  cleared, loss scale adapted on the device).

The host only advances the step counter and the learning-rate schedule.  Device-side waits are
bounded; a time-out is reported through a status word that the next ``step`` turns into an error.
"""
from __future__ import annotations

import ctypes as C
import weakref

import numpy as np
import torch

from .. import autograd, env
from ..base import MXNetError
from . import dist

_MAXR = 8
MODE_SGD, MODE_NAG, MODE_PLAIN, MODE_ADAM, MODE_ADAMW, MODE_LAMB = 0, 1, 2, 3, 4, 5
_ERRORS = {1: 'waiting for the other ranks to finish their backward pass',
           2: 'waiting for the other ranks to publish their reduced shard',
           3: 'waiting for the other ranks to finish writing weights',
           4: 'waiting for the other ranks to publish their parameter norms'}


_live = weakref.WeakSet()          # FusedStep objects whose status word `check_all` looks at


def check_all():
    """Wait for the launched steps of every live ``FusedStep`` of this process and raise if one of them recorded a
    device-side wait time-out (called by ``nd.waitall`` and at interpreter exit, so a failed last step is not silent)."""
    for fs in list(_live):
        fs.check_status(wait=True)


class StepParams(C.Structure):
    _fields_ = [('grads', C.c_void_p * _MAXR), ('weights', C.c_void_p * _MAXR), ('ctrl', C.c_void_p * _MAXR),
                ('rank', C.c_int), ('nranks', C.c_int), ('total', C.c_int64), ('shard_begin', C.c_int64),
                ('shard_end', C.c_int64), ('gred', C.c_void_p), ('master', C.c_void_p), ('mom', C.c_void_p),
                ('seg_end', C.c_void_p), ('lr_mult', C.c_void_p), ('wd_mult', C.c_void_p), ('nseg', C.c_int),
                ('step', C.c_uint32), ('rescale', C.c_float), ('use_loss_scale', C.c_int), ('lr', C.c_float),
                ('wd', C.c_float), ('momentum', C.c_float), ('clip_gradient', C.c_float), ('max_norm', C.c_float),
                ('scale_window', C.c_float), ('scale_max', C.c_float), ('mode', C.c_int),
                ('timeout_ns', C.c_ulonglong), ('var', C.c_void_p), ('beta1', C.c_float), ('beta2', C.c_float),
                ('epsilon', C.c_float), ('coef1', C.c_float), ('coef2', C.c_float), ('lower_bound', C.c_float),
                ('upper_bound', C.c_float), ('norm_acc', C.c_void_p), ('norm_in', C.c_void_p * _MAXR),
                ('seg_skip', C.c_void_p), ('seg_coef', C.c_void_p), ('grads_mc', C.c_void_p), ('weights_mc', C.c_void_p)]


class _DevBuf(object):
    """Zero-copy view of raw device memory for the tensor library."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {'shape': (int(nbytes),), 'typestr': '|u1', 'data': (int(ptr), False),
                                         'version': 2, 'strides': None}


def _lib():
    from ..ops import cuda
    return cuda.lib()


def supports(optimizer, params):
    """SGD / NAG / Adam / AdamW / LAMB on dense parameters of one floating dtype living on one CUDA device."""
    from ..optimizer import optimizer as opt
    if type(optimizer) not in (opt.SGD, opt.NAG, opt.Adam, opt.AdamW, opt.LAMB):
        return False
    if type(optimizer) is opt.Adam and getattr(optimizer, 'lazy_update', False) and any(
            p._grad_stype != 'default' for p in params):
        return False
    dtypes = set()
    for p in params:
        if p.grad_req == 'null':
            continue
        if p._data is None or p._stype != 'default' or p._grad_stype != 'default':
            return False
        arr = next(iter(p._data.values()))
        if not arr._data.is_cuda or arr._data.numel() == 0:
            return False
        dtypes.add(arr._data.dtype)
    if len(dtypes) != 1:
        return False
    dt = next(iter(dtypes))
    if dt not in (torch.float16, torch.bfloat16, torch.float32):
        return False
    if dt != torch.float32 and not optimizer.multi_precision:
        return False
    return True


class FusedStep(object):
    """The fused step of ONE GPU.  Its peers are either the other processes of the job (one GPU each, connected through
    CUDA IPC) or, with ``local_group=(i, n)``, the other GPUs of this process (see :class:`FusedStepGroup`)."""

    def __init__(self, params, optimizer, ctx, local_group=None):
        L = _lib()
        assert L.mxb_step_params_bytes() == C.sizeof(StepParams), 'StepParams layout mismatch'
        self.optimizer = optimizer
        self.ctx = ctx
        self.device = ctx.torch_device
        torch.cuda.set_device(self.device)
        self.params = [p for p in params if p.grad_req != 'null']
        self.index = {id(p): i for i, p in enumerate(params)}
        self.param_ids = [self.index[id(p)] for p in self.params]
        arrs = [p._data[ctx] for p in self.params]
        self.dtype = arrs[0]._data.dtype
        self.esize = arrs[0]._data.element_size()
        self.local_group = local_group
        if local_group is not None:
            self.rank, self.nranks = local_group
        else:
            self.rank = dist.rank() if dist.is_initialized() else 0
            self.nranks = dist.world_size() if dist.is_initialized() else 1
        if self.nranks > _MAXR:
            raise MXNetError('the fused step supports at most %d ranks per node' % _MAXR)
        # ---- layout: every segment starts on a 16-byte boundary ------------------------------------
        vec = 8
        offs, cur = [], 0
        for a in arrs:
            offs.append(cur)
            cur += (a._data.numel() + vec - 1) // vec * vec
        gran = vec * self.nranks
        self.total = (cur + gran - 1) // gran * gran
        self.offsets = offs
        self.sizes = [a._data.numel() for a in arrs]
        shard = self.total // self.nranks
        self.shard_begin, self.shard_end = self.rank * shard, (self.rank + 1) * shard
        # ---- one IPC-exportable slab: [control block | weight arena | gradient arena] ---------------
        self.nseg = len(arrs)
        self._norm_off = (L.mxb_step_ctrl_bytes() + 255) // 256 * 256
        self.ctrl_bytes = (self._norm_off + _MAXR * 2 * self.nseg * 4 + 255) // 256 * 256
        arena_bytes = self.total * self.esize
        # The rank's fp32 state (master weights, first and second moment of its shard) sits in the same IPC-visible slab,
        # so that ONE rank can collect every shard with peer copies when it writes a checkpoint: saving optimizer states is
        # a local call in the reference (python/mxnet/gluon/trainer.py:489-516), not a collective.
        from ..optimizer import optimizer as _opt
        kind = type(optimizer)
        self.mode = {_opt.NAG: MODE_NAG, _opt.Adam: MODE_ADAM, _opt.AdamW: MODE_ADAMW, _opt.LAMB: MODE_LAMB}.get(kind, MODE_SGD)
        two_moments = self.mode in (MODE_ADAM, MODE_ADAMW, MODE_LAMB)
        need_mom = two_moments or getattr(optimizer, 'momentum', 0.0) != 0.0
        shard_bytes = (shard * 4 + 255) // 256 * 256
        self._state_off = {}
        cur_off = self.ctrl_bytes + 2 * arena_bytes
        cur_off = (cur_off + 255) // 256 * 256
        for name, wanted in (('master', self.dtype != torch.float32), ('mom', need_mom), ('var', two_moments)):
            if wanted:
                self._state_off[name] = cur_off
                cur_off += shard_bytes
        self.slab_bytes = cur_off
        self.mc_base = 0                  # NVLS multicast address of the slab (0: plain peer loads and stores)
        self._symm = self._alloc_symmetric() if (local_group is None and self.nranks > 1 and env.get('MXNET_KVSTORE_NVLS')) else None
        if self._symm is not None:
            self.slab = self._symm[0].data_ptr()
        else:
            ptr = C.c_void_p()
            rc = L.mxb_dev_alloc(C.byref(ptr), self.slab_bytes)
            if rc != 0:
                raise MXNetError('cudaMalloc of the parameter arena failed: %s' % L.mxb_error_string(rc).decode())
            self.slab = ptr.value
        self._w_off, self._g_off = self.ctrl_bytes, self.ctrl_bytes + arena_bytes
        # Each tensor below wraps its own piece of the slab as an independent storage: tensors that were
        # views of one base would share a version counter, and the in-place gradient accumulation of one
        # parameter would then invalidate every weight the autograd graph has saved for backward.
        self._bufs = []
        self.ctrl = self._blob(0, self.ctrl_bytes)
        self.weights = self._blob(self._w_off, arena_bytes).view(self.dtype)
        self.grads = self._blob(self._g_off, arena_bytes).view(self.dtype)
        for p, off, n in zip(self.params, offs, self.sizes):
            shape = p._data[ctx]._data.shape
            w = self._blob(self._w_off + off * self.esize, n * self.esize).view(self.dtype).view(shape)
            g = self._blob(self._g_off + off * self.esize, n * self.esize).view(self.dtype).view(shape)
            p._rebind(ctx, w, g)
        # ---- peers ---------------------------------------------------------------------------------
        self.peer_base = [self.slab] * self.nranks
        self._opened = []
        self._layout = (offs, vec)
        if local_group is None:
            self._connect_processes()
            self._init_state()

    def _alloc_symmetric(self):
        """The slab as symmetric memory of the job (CUDA virtual-memory allocations that every rank maps, bound to an
        NVLink-switch multicast object where the machine has one): the kernels can then reduce and broadcast through the
        switch (``multimem`` instructions).  The tensor library does the allocation and the handle exchange; all ranks
        fall back to ``cudaMalloc`` + CUDA IPC together when any of them cannot allocate."""
        t = None
        try:
            import torch.distributed._symmetric_memory as symm
            t = symm.empty(self.slab_bytes, dtype=torch.uint8, device=self.device)
            t.zero_()
        except Exception:   # pylint: disable=broad-except
            t = None
        oks = dist.all_gather_object(t is not None)
        return (t,) if all(oks) else None

    def _connect_processes(self):
        """Open the slabs of the other processes (symmetric-memory rendezvous, or CUDA IPC) and start from rank 0's
        weights."""
        L = _lib()
        if self.nranks > 1 and self._symm is not None:
            import torch.distributed._symmetric_memory as symm
            layout = (self.total, [int(s) for s in self.sizes])
            for r, lay in enumerate(dist.all_gather_object(layout)):
                if lay != layout:
                    raise MXNetError('rank %d has a different parameter layout than rank %d' % (r, self.rank))
            hdl = symm.rendezvous(self._symm[0], torch.distributed.group.WORLD)
            self._symm = (self._symm[0], hdl)
            self.peer_base = [int(p) for p in hdl.buffer_ptrs]
            self.peer_base[self.rank] = self.slab
            self.mc_base = int(hdl.multicast_ptr or 0)
            dist.broadcast_(self.weights, 0)
        elif self.nranks > 1:
            hb = L.mxb_ipc_handle_bytes()
            handle = C.create_string_buffer(hb)
            rc = L.mxb_ipc_get_handle(C.c_void_p(self.slab), handle)
            if rc != 0:
                raise MXNetError('cudaIpcGetMemHandle failed: %s' % L.mxb_error_string(rc).decode())
            layout = (self.total, [int(s) for s in self.sizes])
            gathered = dist.all_gather_object((handle.raw, layout))
            for r, (h, lay) in enumerate(gathered):
                if lay != layout:
                    raise MXNetError('rank %d has a different parameter layout than rank %d' % (r, self.rank))
                if r == self.rank:
                    continue
                p2 = C.c_void_p()
                rc = L.mxb_ipc_open(C.c_char_p(h), C.byref(p2))
                if rc != 0:
                    raise MXNetError('cudaIpcOpenMemHandle(rank %d) failed: %s' % (r, L.mxb_error_string(rc).decode()))
                self.peer_base[r] = p2.value
                self._opened.append(p2.value)
            # every rank starts from rank 0's values
            dist.broadcast_(self.weights, 0)

    def _init_state(self):
        """Shard-local optimizer state and the per-parameter tables (after the peers are known and the weights agree)."""
        L = _lib()
        offs, vec = self._layout
        n_shard = self.shard_end - self.shard_begin
        self.gred = torch.zeros(n_shard, dtype=torch.float32, device=self.device)

        def state(name):
            off = self._state_off.get(name)
            return self._blob(off, n_shard * 4).view(torch.float32) if off is not None else None
        self.master, self.mom, self.var = state('master'), state('mom'), state('var')     # the slab starts zeroed
        if self.master is not None:
            self.master.copy_(self.weights[self.shard_begin:self.shard_end])
        self.norm_acc = torch.zeros(2 * self.nseg, dtype=torch.float32, device=self.device)
        seg_end = np.asarray([o + (s + vec - 1) // vec * vec for o, s in zip(offs, self.sizes)], dtype=np.int64)
        seg_end[-1] = self.total
        self.seg_end = torch.from_numpy(seg_end).to(self.device)
        self._mults = ([float(p.lr_mult) for p in self.params], [float(p.wd_mult) for p in self.params])
        self.lr_mult = torch.tensor(self._mults[0], dtype=torch.float32, device=self.device)
        self.wd_mult = torch.tensor(self._mults[1], dtype=torch.float32, device=self.device)
        self.seg_skip = torch.zeros(self.nseg, dtype=torch.int32, device=self.device)
        self.seg_coef = torch.ones(2 * self.nseg, dtype=torch.float32, device=self.device)
        self._skip_set = False
        self.step_no = 0
        self.timeout_ms = int(env.get('MXNET_KVSTORE_WAIT_MS'))
        off_status = L.mxb_step_ctrl_offset(0)
        off_scale = L.mxb_step_ctrl_offset(2)
        self.status = self.ctrl[off_status:off_status + 8].view(torch.int32)        # [status, status_step]
        self.scale_state = self.ctrl[off_scale:off_scale + 16].view(torch.float32)  # [scale, clean, skipped, norm]
        self.scale_state[0] = 1.0
        self._status_host = torch.zeros(2, dtype=torch.int32).pin_memory()
        self._status_event = None
        self._grad_arrays = [p._grad[self.ctx] for p in self.params]
        self._data_arrays = [p._data[self.ctx] for p in self.params]
        self._scaler_attached = None
        self.max_norm = -1.0
        self._dt_code = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[self.dtype]
        if self.nranks > 1 and self.local_group is None:
            torch.cuda.synchronize(self.device)
            dist.barrier()
        _live.add(self)

    def _blob(self, byte_offset, nbytes):
        """A uint8 tensor over ``nbytes`` of the slab starting at ``byte_offset`` (its own storage object)."""
        buf = _DevBuf(self.slab + byte_offset, nbytes)
        self._bufs.append(buf)
        return torch.as_tensor(buf, device=self.device)

    # ------------------------------------------------------------------------------------------------
    def set_global_norm_clip(self, max_norm):
        """Clip by the global gradient norm inside the update kernel (``gluon.utils.clip_global_norm``
        semantics: ``scale = min(1, max_norm / (norm + 1e-8))``); ``None`` turns it off."""
        self.max_norm = -1.0 if max_norm is None else float(max_norm)

    def _params(self, rescale, mode, use_ls, lr, wd):
        sp = StepParams()
        for r in range(self.nranks):
            sp.grads[r] = self.peer_base[r] + self._g_off
            sp.weights[r] = self.peer_base[r] + self._w_off
            sp.ctrl[r] = self.peer_base[r]
        if self.mc_base:
            sp.grads_mc, sp.weights_mc = self.mc_base + self._g_off, self.mc_base + self._w_off
        sp.rank, sp.nranks, sp.total = self.rank, self.nranks, self.total
        sp.shard_begin, sp.shard_end = self.shard_begin, self.shard_end
        sp.gred = self.gred.data_ptr()
        sp.master = self.master.data_ptr() if self.master is not None else None
        sp.mom = self.mom.data_ptr() if self.mom is not None else None
        sp.seg_end, sp.lr_mult, sp.wd_mult = self.seg_end.data_ptr(), self.lr_mult.data_ptr(), self.wd_mult.data_ptr()
        sp.nseg = len(self.params)
        sp.step = self.step_no
        sp.rescale = rescale
        sp.use_loss_scale = use_ls
        opt = self.optimizer
        sp.lr, sp.wd, sp.momentum = lr, wd, float(getattr(opt, 'momentum', 0.0))
        sp.clip_gradient = -1.0 if opt.clip_gradient is None else float(opt.clip_gradient)
        sp.max_norm = self.max_norm
        sp.scale_window, sp.scale_max = 2000.0, float(2 ** 24)
        if self._scaler_attached is not None:
            sp.scale_window = float(self._scaler_attached._scale_seq_len)
            sp.scale_max = float(self._scaler_attached._max_loss_scale)
        sp.mode = mode
        sp.timeout_ns = self.timeout_ms * 1000000
        if self.var is not None:
            sp.var = self.var.data_ptr()
            sp.beta1, sp.beta2, sp.epsilon = float(opt.beta1), float(opt.beta2), float(opt.epsilon)
            # every parameter keeps its own update count (a parameter skipped for a stale gradient falls behind); the
            # bias corrections travel as scalars while the counts agree and as a per-parameter table otherwise
            counts = [max(int(opt._index_update_count.get(i, opt.begin_num_update)), 1) for i in self.param_ids] or [1]
            correct = getattr(opt, 'bias_correction', True) if mode == MODE_LAMB else getattr(opt, 'correct_bias', True)
            t = counts[0]
            sp.coef1 = 1.0 - opt.beta1 ** t if correct else 1.0
            sp.coef2 = 1.0 - opt.beta2 ** t if correct else 1.0
            if correct and any(c != t for c in counts):
                table = [1.0 - opt.beta1 ** c for c in counts] + [1.0 - opt.beta2 ** c for c in counts]
                self.seg_coef.copy_(torch.tensor(table, dtype=torch.float32))
                sp.seg_coef = self.seg_coef.data_ptr()
            lo, hi = getattr(opt, 'lower_bound', None), getattr(opt, 'upper_bound', None)
            sp.lower_bound = -1.0 if lo is None else float(lo)
            sp.upper_bound = -1.0 if hi is None else float(hi)
        sp.norm_acc = self.norm_acc.data_ptr()
        for r in range(self.nranks):
            sp.norm_in[r] = self.peer_base[r] + self._norm_off
        if self._skip_set:
            sp.seg_skip = self.seg_skip.data_ptr()
        return sp

    def check_status(self, wait=False):
        """Raise if a launched step recorded a wait time-out.  ``wait=False`` only looks at steps that have finished
        (what the next ``step`` does); ``wait=True`` first waits for the last launched step."""
        ev = self._status_event
        if ev is not None and wait:
            ev.synchronize()
        if ev is not None and ev.query():
            self._status_event = None
            code = int(self._status_host[0])
            if code != 0:
                step = int(self._status_host[1])
                self.status.zero_()
                raise MXNetError('fused optimizer step %d timed out after %d ms while %s (rank %d of %d)' % (
                    step, self.timeout_ms, _ERRORS.get(code, 'waiting'), self.rank, self.nranks))

    _check_status = check_status

    def _refresh_multipliers(self):
        lr_m, wd_m = [float(p.lr_mult) for p in self.params], [float(p.wd_mult) for p in self.params]
        if lr_m != self._mults[0]:
            self.lr_mult.copy_(torch.tensor(lr_m, dtype=torch.float32))
        if wd_m != self._mults[1]:
            self.wd_mult.copy_(torch.tensor(wd_m, dtype=torch.float32))
        self._mults = (lr_m, wd_m)

    def _set_stale(self, stale):
        """``stale``: positions (in ``self.params``) of parameters whose gradient was not refreshed; they are left out of
        this step (``ignore_stale_grad=True``, python/mxnet/gluon/trainer.py:437-458)."""
        if stale:
            flags = torch.zeros(self.nseg, dtype=torch.int32)
            flags[list(stale)] = 1
            self.seg_skip.copy_(flags)
            self._skip_set = True
        else:
            self._skip_set = False

    def _begin_step(self, mode, stale=(), count_updates=True):
        """Host bookkeeping of one step: status of the previous one, step number, stale flags, multipliers, update counts
        (``count_updates=False`` for the followers of a group: the optimizer object is shared)."""
        self._check_status()
        self.step_no += 1
        self._set_stale(stale if mode != MODE_PLAIN else ())
        if mode != MODE_PLAIN:
            self._refresh_multipliers()
            if count_updates:
                skip = set(stale)
                self.optimizer._update_count([i for k, i in enumerate(self.param_ids) if k not in skip])
        opt = self.optimizer
        return self._params(float(self._rescale), mode, self._use_ls, float(opt.learning_rate), float(opt.wd))

    def _launch_reduce(self, sp):
        from ..ops import cuda
        L = _lib()
        with torch.cuda.device(self.device):
            rc = L.mxb_fused_reduce(self._dt_code, C.byref(sp), cuda.stream_ptr(self.device))
        if rc != 0:
            raise MXNetError('fused step launch failed: %s' % (L.mxb_error_string(rc).decode() if rc > 0 else rc))
        cuda.count_launch(1)

    def _launch_update(self, sp, mode):
        from ..ops import cuda
        L = _lib()
        with torch.cuda.device(self.device):
            st = cuda.stream_ptr(self.device)
            rc = L.mxb_fused_lamb(self._dt_code, C.byref(sp), st) if mode == MODE_LAMB else \
                L.mxb_fused_update(self._dt_code, C.byref(sp), st)
            if rc != 0:
                raise MXNetError('fused step launch failed: %s' % (L.mxb_error_string(rc).decode() if rc > 0 else rc))
            cuda.count_launch(2 if mode == MODE_LAMB else 1)
            self._status_host.copy_(self.status, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
        self._status_event = ev

    def _launch(self, rescale, mode, use_ls, stale=()):
        self._rescale, self._use_ls = rescale, use_ls
        sp = self._begin_step(mode, stale)
        self._launch_reduce(sp)
        self._launch_update(sp, mode)

    def _attach_scaler(self, scaler):
        """Move the loss scale onto the device.  Returns the ``use_loss_scale`` code for this step: 1 when
        the kernel divides by the device scale, 2 when the host already folded 1/scale into ``rescale``."""
        if scaler is None:
            return 0
        unscaled = getattr(scaler, '_grads_unscaled', False)      # amp.unscale() already divided the gradients
        scaler._grads_unscaled = False
        if self._scaler_attached is scaler:
            return 2 if unscaled else 1
        self.scale_state[0] = float(scaler._loss_scale)
        self.scale_state[1] = float(scaler._unskipped)
        if scaler._device_state is None:
            scaler._device_state = self.scale_state
        scaler._device_states[self.device] = self.scale_state        # one copy per GPU of a group; they evolve alike
        self._scaler_attached = scaler
        return 2

    def attach_scaler(self, scaler):
        if scaler is not None and self._scaler_attached is not scaler:
            self._attach_scaler(scaler)

    def step(self, rescale, scaler=None, stale=()):
        use_ls = self._attach_scaler(scaler)
        self._launch(rescale, self.mode, use_ls, stale)
        autograd.mark_grads_consumed(self._data_arrays)

    def allreduce_only(self):
        """Sum the gradient arenas of all ranks in place (``Trainer.allreduce_grads``)."""
        self._launch(1.0, MODE_PLAIN, 0)

    def update_only(self, rescale, scaler=None, stale=()):
        """Update after ``allreduce_only``: every arena already holds the sum, so the reduction over
        ranks is compensated by 1/nranks."""
        use_ls = self._attach_scaler(scaler)
        self._launch(rescale / self.nranks, self.mode, use_ls, stale)
        autograd.mark_grads_consumed(self._data_arrays)

    def wait_probe(self, timeout_ms=50):
        """Launch a wait on a flag that nothing sets and return the status code it leaves behind (the
        time-out path of the kernels, exercised without any other rank)."""
        from ..ops import cuda
        L = _lib()
        self.status.zero_()
        rc = L.mxb_wait_probe(C.c_void_p(self.slab), _MAXR - 1, 0x7fffffff, int(timeout_ms) * 1000000,
                              cuda.stream_ptr(self.device))
        if rc != 0:
            raise MXNetError('probe launch failed')
        torch.cuda.synchronize(self.device)
        code = int(self.status[0].item())
        self.status.zero_()
        return code

    # ---- optimizer state exchange with the generic Updater (checkpoints) ---------------------------------
    def _gather(self, name):
        """The whole fp32 state vector `name`, collected by THIS rank alone: its own shard plus peer copies
        (``cudaMemcpyAsync`` from the other ranks' slabs).  No other rank takes part, so `if rank == 0: save_states(...)`
        works.  The caller runs between steps: the last step's update kernel returns only after every rank has finished
        writing its state, and no rank can start the next update before this rank launches its next step."""
        shard = getattr(self, name)
        if shard is None:
            return None
        if self.nranks == 1:
            return shard
        from ..ops import cuda
        L = _lib()
        n = shard.numel()
        out = torch.empty(n * self.nranks, dtype=torch.float32, device=self.device)
        st = cuda.stream_ptr(self.device)
        for r in range(self.nranks):
            rc = L.mxb_memcpy_d2d(C.c_void_p(out.data_ptr() + r * n * 4), C.c_void_p(self.peer_base[r] + self._state_off[name]),
                                  n * 4, st)
            if rc != 0:
                raise MXNetError('peer copy of optimizer state from rank %d failed: %s' % (r, L.mxb_error_string(rc).decode()))
        return out

    def export_states(self, updater):
        """Write the sharded state into ``updater.states`` in the layout the generic optimizers use:
        ``momentum`` (SGD/NAG) or ``(mean, var)`` (Adam/AdamW/LAMB), wrapped as ``(master, inner)`` for
        multi-precision."""
        from ..ndarray.ndarray import NDArray
        self.check_status(wait=True)
        master, mom, var = self._gather('master'), self._gather('mom'), self._gather('var')
        for p, idx, off, n in zip(self.params, self.param_ids, self.offsets, self.sizes):
            shape = p._data[self.ctx]._data.shape

            def piece(flat):
                return NDArray._from_tensor(flat[off:off + n].view(shape).clone(), self.ctx) if flat is not None else None
            inner = (piece(mom), piece(var)) if var is not None else piece(mom)
            updater.states[idx] = (piece(master), inner) if master is not None else inner
            updater.states_synced[idx] = True

    def import_states(self, updater, optimizer):
        self.optimizer = optimizer
        for p, idx, off, n in zip(self.params, self.param_ids, self.offsets, self.sizes):
            st = updater.states.get(idx)
            if st is None:
                continue
            master, inner = (st if self.master is not None and isinstance(st, (tuple, list)) else (None, st))
            mom, var = (inner if self.var is not None and isinstance(inner, (tuple, list)) else (inner, None))
            lo, hi = max(off, self.shard_begin), min(off + n, self.shard_end)
            if lo >= hi:
                continue
            src = slice(lo - off, hi - off)
            dst = slice(lo - self.shard_begin, hi - self.shard_begin)
            for mine, theirs in ((self.master, master), (self.mom, mom), (self.var, var)):
                if mine is not None and theirs is not None:
                    mine[dst].copy_(theirs._data.reshape(-1)[src].to(self.device))

    def __del__(self):
        try:
            L = _lib()
            for p in self._opened:
                L.mxb_ipc_close(C.c_void_p(p))
        except Exception:  # pylint: disable=broad-except
            pass


class FusedStepGroup(object):
    """The fused step over the GPUs of ONE process: the reference's main multi-GPU mode (``kvstore='device'`` with
    ``ctx=[gpu(0), ...]``, src/kvstore/comm.h:482-654 reduces on a merge buffer and copies back).  Here every GPU runs the
    same two kernels as in the one-process-per-GPU mode on its own stream: GPU ``i`` owns shard ``i`` of the arena,
    reads the gradient arenas of the other GPUs through peer access, and stores the new weights into every arena.  The
    kernels of different GPUs wait for each other's flags; the host launches them back to back without blocking."""

    def __init__(self, params, optimizer, ctxs):
        L = _lib()
        n = len(ctxs)
        if n > _MAXR:
            raise MXNetError('the fused step supports at most %d GPUs per process' % _MAXR)
        for a in ctxs:
            for b in ctxs:
                if a.device_id != b.device_id:
                    rc = L.mxb_enable_peer_access(a.device_id, b.device_id)
                    if rc != 0:
                        raise MXNetError('no peer access from gpu(%d) to gpu(%d): %s'
                                         % (a.device_id, b.device_id, L.mxb_error_string(rc).decode()))
        self.members = [FusedStep(params, optimizer, ctx, local_group=(i, n)) for i, ctx in enumerate(ctxs)]
        lead = self.members[0]
        for m in self.members:
            m.peer_base = [t.slab for t in self.members]
        for m in self.members[1:]:
            if (m.total, m.sizes) != (lead.total, lead.sizes):
                raise MXNetError('the replicas of the parameters differ in shape between devices')
            m.weights.copy_(lead.weights)           # every replica starts from the first device's values
        for m in self.members:
            with torch.cuda.device(m.device):
                m._init_state()
        for m in self.members:
            torch.cuda.synchronize(m.device)
        self.optimizer = optimizer
        self.params = lead.params
        self.nranks = n

    # what the Trainer reads
    @property
    def _data_arrays(self):
        return self.members[0]._data_arrays

    def replica_arrays(self):
        return [m._data_arrays for m in self.members]

    def set_global_norm_clip(self, max_norm):
        for m in self.members:
            m.set_global_norm_clip(max_norm)

    def attach_scaler(self, scaler):
        for m in self.members:
            m.attach_scaler(scaler)

    def check_status(self, wait=False):
        for m in self.members:
            m.check_status(wait)

    def _run(self, rescale, mode, scaler, stale):
        sps = []
        for k, m in enumerate(self.members):
            # the unscaled flag is consumed by the first member; the others follow its verdict
            if k == 0:
                use_ls = m._attach_scaler(scaler)
            else:
                m.attach_scaler(scaler)
                use_ls = use_ls if scaler is not None else 0
            m._rescale, m._use_ls = rescale, use_ls
            sps.append(m._begin_step(mode, stale, count_updates=(k == 0)))
        for m, sp in zip(self.members, sps):       # every GPU's reduce is in flight before the first update is queued
            m._launch_reduce(sp)
        for m, sp in zip(self.members, sps):
            m._launch_update(sp, mode)
        if mode != MODE_PLAIN:
            for m in self.members:
                autograd.mark_grads_consumed(m._data_arrays)

    def step(self, rescale, scaler=None, stale=()):
        self._run(rescale, self.members[0].mode, scaler, stale)

    def allreduce_only(self):
        self._run(1.0, MODE_PLAIN, None, ())

    def update_only(self, rescale, scaler=None, stale=()):
        self._run(rescale / self.nranks, self.members[0].mode, scaler, stale)

    def export_states(self, updater):
        self.members[0].export_states(updater)      # collects the other GPUs' shards with peer copies

    def import_states(self, updater, optimizer):
        self.optimizer = optimizer
        for m in self.members:
            m.import_states(updater, optimizer)

"""Cached executor behind ``HybridBlock.hybridize()``.

Reference: ``CachedOp`` (``src/imperative/cached_op.cc:385-899``: ``StaticForward`` with
pre-allocated buffers and pre-built op segments; backward ``:901-1143``) and its optional CUDA-graph
replay of bulked segments (``src/imperative/cuda_graphs.h:174-586``: one conventional warm-up run,
then stream capture, re-capture when a pointer changes).

Here the whole forward, and the whole backward, are each ONE captured CUDA graph replayed on static
buffers when ``static_alloc`` and ``static_shape`` are set on a GPU: the first call with a given
signature (training flag, input shapes/dtypes, parameter-storage version) runs eagerly, the second
captures, later calls replay.  The pair is exposed to autograd as a single node (the counterpart of
the ``_CachedOp`` / ``_backward_CachedOp`` tape node) whose inputs include every parameter, so
gradients still land in the parameters' own buffers.  Anything that cannot be captured (host
synchronisation inside ``forward``, data-dependent shapes) makes the block fall back to eager
execution permanently, the analogue of the reference's split around incompatible operators.
"""
from __future__ import annotations

import logging

import torch

from .. import _state, autograd, env
from ..ndarray.ndarray import NDArray

_log = logging.getLogger('mxnet_b200.cached_op')


class _Graphed(object):
    """Forward/backward graph pair for one call signature."""

    def __init__(self, block, args, training, recording, forward=None):
        self.block = block
        self.forward = forward if forward is not None else block.forward    # a pass-rewritten graph of the block, or its code
        self.training, self.recording = training, recording
        from .block import _flatten
        flat, self.in_fmt = _flatten(args, 'input')
        self.arg_slots = [i for i, a in enumerate(flat) if isinstance(a, NDArray)]
        self.flat_template = list(flat)
        arrays = [flat[i] for i in self.arg_slots]
        self.cls = arrays[0].__class__
        self.ctx = arrays[0]._ctx
        dev = arrays[0]._data.device
        params = [p for p in block.collect_params().values() if p._data is not None]
        self.param_arrays, self.param_tensors = [], []
        for p in params:
            arr = p._data.get(self.ctx)
            if arr is None:
                arr = next(iter(p._data.values()))
            if arr._data.requires_grad:
                self.param_arrays.append(arr)
                self.param_tensors.append(arr._data)
        self.static_in = []
        for a in arrays:
            t = a._data.detach().clone()
            if recording and a._data.requires_grad:
                t.requires_grad_(True)
            self.static_in.append(t)
        stream = torch.cuda.Stream(device=dev)
        stream.wait_stream(torch.cuda.current_stream(dev))
        # The graphs differentiate with respect to fresh leaf aliases of the parameters (same storage).  The
        # parameters' own gradient accumulators were created by earlier eager passes on the default stream;
        # differentiating with respect to them would make the autograd engine order the legacy stream after
        # the capturing stream, which stream capture forbids.  The aliases only ever see the capture stream,
        # and they carry none of the parameters' Python hooks.
        with torch.cuda.stream(stream):
            self.alias = [t.detach().requires_grad_(True) for t in self.param_tensors] if recording else []
        self.grad_inputs = [t for t in self.static_in if t.requires_grad] + self.alias
        from ..ops import cuda as _kernels
        self._kernels = _kernels
        self.pool = torch.cuda.graph_pool_handle()
        self.fwd = torch.cuda.CUDAGraph()
        n0 = _kernels.launches()
        # No garbage collection while a capture is open: a collection that frees the graphs of an earlier, dropped block
        # destroys them in the middle of this capture ("operation not permitted when stream is capturing") and invalidates
        # it.  Whatever is collectable is collected now, and the collector stays off until both graphs are recorded.
        import gc
        gc.collect()
        self._gc_was_enabled = gc.isenabled()
        gc.disable()
        try:
            self._capture(stream, n0, recording, dev)
        finally:
            if self._gc_was_enabled:
                gc.enable()

    def _capture(self, stream, n0, recording, dev):
        from .block import _flatten
        _kernels = self._kernels
        with torch.cuda.stream(stream):
            with torch.cuda.graph(self.fwd, pool=self.pool, stream=stream):
                outs = self._run_forward()
        self.fwd_launches = _kernels.launches() - n0     # in-tree kernels recorded in the forward graph
        self.bwd_launches = 0
        flat_out, self.out_fmt = _flatten(outs, 'output')
        self.out_is_array = [isinstance(o, NDArray) for o in flat_out]
        self.flat_out_template = list(flat_out)
        self.static_out = [o._data for o in flat_out if isinstance(o, NDArray)]
        self.bwd = None
        if recording and self.grad_inputs and any(o.requires_grad for o in self.static_out):
            self.out_needs_grad = [o.requires_grad for o in self.static_out]
            self.static_gout = [torch.zeros_like(o) if o.requires_grad else None for o in self.static_out]
            self.bwd = torch.cuda.CUDAGraph()
            n1 = _kernels.launches()
            with torch.cuda.stream(stream):
                with torch.cuda.graph(self.bwd, pool=self.pool, stream=stream):
                    gin = torch.autograd.grad([o for o in self.static_out if o.requires_grad], self.grad_inputs,
                                              [g for g in self.static_gout if g is not None], allow_unused=True)
                    # Parameter gradients are added to the parameters' gradient buffers by nodes of this graph, instead
                    # of being handed to the autograd engine, which would launch one accumulation kernel per parameter
                    # after every replay.  The buffers are kept alive here; a parameter whose buffer is replaced later
                    # falls back to the engine (see _Replay.backward).
                    n_in = sum(1 for t in self.static_in if t.requires_grad)
                    self.grad_targets = []
                    acc_dst, acc_src = [], []
                    for arr, gi in zip(self.param_arrays, gin[n_in:]):
                        tgt = arr._grad._data if getattr(arr, '_grad', None) is not None else None
                        ok = (gi is not None and tgt is not None and arr._grad_req in ('write', 'add')
                              and tgt.shape == gi.shape and tgt.dtype == gi.dtype and tgt.device == gi.device)
                        if ok:
                            acc_dst.append(tgt)
                            acc_src.append(gi)
                        self.grad_targets.append(tgt if ok else None)
                    if acc_dst:
                        if env.get('MXNET_B200_KERNELS') and _kernels.available():
                            from ..ops.cuda import optim_ops
                            optim_ops.multi_add_(acc_dst, acc_src)      # one launch per 48 parameters
                        else:
                            for tgt, gi in zip(acc_dst, acc_src):
                                tgt.add_(gi)
            self.static_gin = list(gin)
            self.bwd_launches = _kernels.launches() - n1
        torch.cuda.current_stream(dev).wait_stream(stream)
        self.static_out_detached = [o.detach() for o in self.static_out]

    def _run_forward(self):
        flat = list(self.flat_template)
        for slot, t in zip(self.arg_slots, self.static_in):
            flat[slot] = self.cls._from_tensor(t, self.ctx)
        from .block import _regroup
        args, _ = _regroup(flat, self.in_fmt)
        if not isinstance(args, (list, tuple)):
            args = [args]
        prev_r, prev_t = _state.state.recording, _state.state.training
        _state.state.recording, _state.state.training = self.recording, self.training
        for arr, a in zip(self.param_arrays, self.alias):
            arr._data = a
        try:
            if self.recording:
                with torch.enable_grad():
                    return self.forward(*args)
            with torch.no_grad():
                return self.forward(*args)
        finally:
            _state.state.recording, _state.state.training = prev_r, prev_t
            if self.alias:
                for arr, t in zip(self.param_arrays, self.param_tensors):
                    arr._data = t

    def __call__(self, args):
        from .block import _flatten, _regroup
        flat, _ = _flatten(args, 'input')
        arrays = [flat[i] for i in self.arg_slots]
        g = self

        class _Replay(torch.autograd.Function):
            @staticmethod
            def forward(ctx, *tensors):
                n = len(g.static_in)
                for dst, src in zip(g.static_in, tensors[:n]):
                    if dst.data_ptr() != src.data_ptr():
                        dst.copy_(src)
                g.fwd.replay()
                g._kernels.count_launch(g.fwd_launches)
                return tuple(g.static_out_detached)

            @staticmethod
            def backward(ctx, *gouts):
                for dst, src in zip(g.static_gout, gouts):
                    if dst is not None and src is not None and dst.data_ptr() != src.data_ptr():
                        dst.copy_(src)
                # what the leaf hook of a parameter does before the engine accumulates into its buffer, for the
                # parameters whose gradients the graph itself adds to their buffers
                cur = autograd._pass_id[0]
                direct = []
                for arr, tgt in zip(g.param_arrays, g.grad_targets):
                    buf = arr._grad._data if getattr(arr, '_grad', None) is not None else None
                    d = tgt is not None and buf is not None and buf.data_ptr() == tgt.data_ptr() and arr._grad_req != 'null'
                    if d:
                        if arr._grad_req == 'write' and arr._fresh_grad and arr._grad_pass != cur:
                            buf.zero_()
                        arr._fresh_grad = True
                        arr._grad_pass = cur
                    direct.append(d)
                g.bwd.replay()
                g._kernels.count_launch(g.bwd_launches)
                res, k = [], 0
                for t in g.static_in:
                    if t.requires_grad:
                        gi = g.static_gin[k]
                        res.append(gi.detach() if gi is not None else None)
                        k += 1
                    else:
                        res.append(None)
                for gi, d in zip(g.static_gin[k:], direct):
                    res.append(None if d else (gi.detach() if gi is not None else None))
                return tuple(res)

        tensors = [a._data for a in arrays]
        if self.bwd is not None and _state.state.recording:
            with torch.enable_grad():
                outs = _Replay.apply(*(tensors + self.param_tensors))
        else:
            with torch.no_grad():
                for dst, src in zip(self.static_in, tensors):
                    dst.copy_(src)
                self.fwd.replay()
                self._kernels.count_launch(self.fwd_launches)
                outs = tuple(self.static_out_detached)
        flat_out, k = list(self.flat_out_template), 0
        for i, is_arr in enumerate(self.out_is_array):
            if is_arr:
                flat_out[i] = self.cls._from_tensor(outs[k], self.ctx)
                k += 1
        res, _ = _regroup(flat_out, self.out_fmt)
        return res


class CachedOp(object):
    """Per-block cache of executors keyed by call signature."""

    def __init__(self, block, flags):
        self.block = block
        self.flags = dict(flags or {})
        self._seen = {}
        self._graphs = {}
        self._disabled = False

    def _static(self):
        return bool(self.flags.get('static_alloc') and self.flags.get('static_shape'))

    def _use_graphs(self, arrays):
        if self._disabled or not env.get('MXNET_ENABLE_CUDA_GRAPHS'):
            return False
        if not self._static() and not env.get('MXNET_CUDA_GRAPHS_AUTO'):
            return False
        if not (bool(arrays) and all(a._data.is_cuda for a in arrays)):
            return False
        return not torch.cuda.is_current_stream_capturing()      # a block called inside an outer block's capture is part of it

    def _signature(self, flat):
        from . import block as blk
        sig = [blk._storage_version[0], _state.state.training, _state.state.recording]
        for a in flat:
            if isinstance(a, NDArray):
                sig.append((tuple(a.shape), str(a._data.dtype), a._data.requires_grad))
            else:
                sig.append(repr(a))
        return tuple(sig)

    def __call__(self, *args, graph_forward=None, graph_tag=None):
        """``graph_forward``: a callable that evaluates the block's traced graph after a graph pass (layout management);
        it replaces ``block.forward`` both in the eager runs and inside the captured graphs.  ``graph_tag`` names the pass
        in the signature, so that switching it on or off never reuses the other form's graphs."""
        from .block import _flatten
        flat, _ = _flatten(args, 'input')
        arrays = [a for a in flat if isinstance(a, NDArray)]
        eager = graph_forward if graph_forward is not None else self.block._call_forward
        if not self._use_graphs(arrays):
            return eager(*args)
        sig = self._signature(flat) + ((graph_tag,) if graph_forward is not None else ())
        g = self._graphs.get(sig)
        if g is not None:
            return g(args)
        # With static_alloc + static_shape the second call of a signature is captured.  A plain hybridize() makes no promise
        # about shapes: a signature is captured once it has repeated (fourth call), and at most four signatures per block,
        # so that a workload whose shapes keep changing stays eager instead of collecting graphs.
        seen = self._seen.get(sig, 0)
        need = 1 if self._static() else 3
        if seen < need or (not self._static() and len(self._graphs) >= 4):
            self._seen[sig] = seen + 1   # warm-up runs with this signature stay eager
            return eager(*args)
        try:
            g = _Graphed(self.block, args, _state.state.training, _state.state.recording, forward=graph_forward)
        except Exception as e:  # pylint: disable=broad-except
            self._disabled = True
            _log.warning('CUDA graph capture failed (%s); block %s runs eagerly', e, type(self.block).__name__,
                         exc_info=bool(env.get('MXNET_CUDA_GRAPHS_VERBOSE')))
            return eager(*args)
        self._graphs[sig] = g
        if env.get('MXNET_CUDA_GRAPHS_VERBOSE'):
            _log.info('captured CUDA graphs for %s signature %s', type(self.block).__name__, sig[:3])
        return g(args)

"""Gluon ``Trainer`` (``python/mxnet/gluon/trainer.py``).

``step(batch_size)`` = rescale (``rescale_grad = _scale / batch_size``, ``trainer.py:359-360``) →
``_allreduce_grads`` (one ``pushpull`` per parameter with ``priority=-i``, ``:392-416``) →
``_update`` (AMP overflow check, then one ``Updater`` call per device, ``:451-486``).  Branches kept:
``update_on_kvstore`` (optimizer runs where the merged gradient lives), stores without optimizer
capability (Horovod/BytePS/TestStore), ``kvstore=None`` and single-device short cuts, state
save/load through the Updater pickle.

Fast path: when every parameter lives on one CUDA device of this process and the optimizer is one
the fused kernels implement, gradient reduction over all ranks, AMP unscale + finite check, the
multi-precision update and the weight broadcast run as the two launches of
``parallel.fused.FusedStep`` over peer memory; nothing else is launched by ``step``.
"""
from __future__ import annotations

import pickle
import warnings

import torch

from .. import env, optimizer as opt
from ..device import Device
from ..kvstore import create as kv_create, KVStoreBase
from ..ndarray.ndarray import NDArray
from .parameter import Parameter

__all__ = ['Trainer']


class Trainer(object):
    def __init__(self, params, optimizer, optimizer_params=None, kvstore='device', compression_params=None,
                 update_on_kvstore=None):
        param_list = []
        if isinstance(params, dict):
            for key in sorted(list(params.keys())):
                param_list.append(params[key])
            params = param_list
        if not isinstance(params, (list, tuple)):
            raise ValueError('First argument must be a list or dict of Parameters, got %s.' % (type(params)))
        self._params = []
        self._contains_sparse_weight = False
        self._contains_sparse_grad = False
        self._param2idx = {}
        for i, param in enumerate(params):
            if not isinstance(param, Parameter):
                raise ValueError('First argument must be a list or dict of Parameters, got list of %s.' % (type(param)))
            if param._uuid in self._param2idx:
                continue
            self._param2idx[param._uuid] = len(self._params)
            self._params.append(param)
            param._set_trainer(self)
            if param._stype != 'default':
                self._contains_sparse_weight = True
            if param._grad_stype != 'default':
                self._contains_sparse_grad = True
        self._compression_params = compression_params
        self._devices = self._check_devices()
        optimizer_params = optimizer_params if optimizer_params else {}
        self._init_optimizer(optimizer, optimizer_params)
        self._scale = self._optimizer.rescale_grad
        if self._optimizer.aggregate_num > 1 and update_on_kvstore is not None:
            if update_on_kvstore:
                raise ValueError('Cannot set update_on_kvstore=True when optimizer.aggregate_num > 1.')
        self._update_on_kvstore_asked = update_on_kvstore       # what the caller passed (None: decide here)
        if update_on_kvstore is None and self._optimizer.aggregate_num > 1:
            update_on_kvstore = False
        self._kvstore_params = {'kvstore': kvstore, 'update_on_kvstore': update_on_kvstore}
        self._kv_initialized = False
        self._kvstore = None
        self._update_on_kvstore = None
        self._distributed = None
        self._params_to_init = []
        self._fused = None
        self._consumed_pass = {}
        self._amp_loss_scaler = None
        self._reset_kvstore()

    def _check_devices(self):
        devices = None
        for param in self._params:
            try:
                dev = param.list_ctx()
            except RuntimeError:
                continue
            assert devices is None or devices == dev, \
                'All Parameters must be initialized on the same set of devices, but Parameter %s is initialized on ' \
                '%s while previous Parameters are initialized on %s.' % (param.name, str(dev), str(devices))
            devices = dev
        return devices

    def _init_optimizer(self, optimizer, optimizer_params):
        param_dict = {i: param for i, param in enumerate(self._params)}
        if isinstance(optimizer, opt.Optimizer):
            assert not optimizer_params, 'optimizer_params must be None if optimizer is an instance of Optimizer ' \
                                         'instead of str'
            self._optimizer = optimizer
            self._optimizer.param_dict = param_dict
        else:
            self._optimizer = opt.create(optimizer, param_dict=param_dict, **optimizer_params)
        self._updaters = [opt.get_updater(self._optimizer) for _ in (self._devices or [None])]

    def _reset_kvstore(self):
        if self._kvstore and 'dist' in self._kvstore.type:
            raise RuntimeError('Cannot reset distributed KVStore.')
        self._kv_initialized = False
        self._kvstore = None
        self._distributed = None
        self._update_on_kvstore = None
        self._params_to_init = [param for param in self._params]
        self._fused = None

    def _init_kvstore(self):
        config = self._kvstore_params
        devices = self._devices = self._check_devices() or self._devices
        if len(self._updaters) != len(devices or [None]):
            self._updaters = [opt.get_updater(self._optimizer) for _ in devices]
        kvstore = config['kvstore']
        update_on_kvstore = config['update_on_kvstore']
        from ..parallel import dist
        multi_proc = dist.is_initialized() and dist.world_size() > 1
        kv = None
        if isinstance(kvstore, KVStoreBase):
            kv = kvstore
        elif isinstance(kvstore, str):
            if kvstore.startswith('dist') or len(devices) > 1 or multi_proc or kvstore in ('horovod', 'byteps') \
                    or kvstore.lower() in KVStoreBase.kv_registry:
                kv = kv_create(kvstore)
        elif kvstore is not None:
            raise ValueError('kvstore must be a string, a KVStore or None')
        if self._contains_sparse_weight and kv is None:
            kv = kv_create('device')
        if kv is not None and 'dist' in kv.type:
            self._distributed = True
        else:
            self._distributed = multi_proc
        if kv is not None:
            if self._compression_params:
                kv.set_gradient_compression(self._compression_params)
            if not kv.is_capable(KVStoreBase.OPTIMIZER):
                if update_on_kvstore:
                    raise ValueError('Please set update_on_kvstore=False when training with %s' % type(kv).__name__)
                update_on_kvstore = False
            elif 'async' in kv.type:
                # asynchronous training has no merged gradient to update from: the optimizer runs on the server
                if self._update_on_kvstore_asked is False:
                    raise ValueError('Please set update_on_kvstore=True when training in async mode.')
                update_on_kvstore = True
            elif update_on_kvstore is None:
                update_on_kvstore = bool(env.get('MXNET_UPDATE_ON_KVSTORE')) and \
                    ('dist' in kv.type or self._contains_sparse_weight) and self._optimizer.aggregate_num <= 1
            if kv.type == 'nccl' and update_on_kvstore:
                update_on_kvstore = False
            if update_on_kvstore:
                kv.set_optimizer(self._optimizer)
        else:
            update_on_kvstore = False
        self._kvstore = kv
        self._update_on_kvstore = bool(update_on_kvstore)
        self._kv_initialized = True
        self._maybe_init_fused()

    def _maybe_init_fused(self):
        """Switch to the fused peer-memory step when its preconditions hold."""
        self._fused = None
        if not env.get('MXNET_KVSTORE_FUSED') or not env.get('MXNET_B200_KERNELS'):
            return
        if self._update_on_kvstore or self._contains_sparse_grad or self._contains_sparse_weight:
            return
        devices = self._devices or []
        if not devices or any(d.device_type != 'gpu' for d in devices) or not torch.cuda.is_available():
            return
        from ..parallel import dist
        if len(devices) > 1 and dist.is_initialized() and dist.world_size() > 1:
            return                       # several GPUs per process AND several processes: the generic kvstore path
        kv = self._kvstore
        if kv is not None and kv.type not in ('device', 'nccl', 'dist_sync', 'dist_device_sync', 'dist_sync_device'):
            return
        if kv is not None and self._compression_params:
            return
        from ..parallel import fused
        if not fused.supports(self._optimizer, self._params):
            return
        if len(devices) == 1:
            self._fused = fused.FusedStep(self._params, self._optimizer, devices[0])
        else:
            # the reference's main multi-GPU mode: one process, ctx=[gpu(0), gpu(1), ...]
            self._fused = fused.FusedStepGroup(self._params, self._optimizer, devices)

    def _init_params(self):
        assert self._kv_initialized, 'Cannot initialize parameters in KVStore when KVStore is not initialized.'
        params_to_init = []
        if self._kvstore:
            for param in self._params_to_init:
                if param._deferred_init:
                    params_to_init.append(param)
                else:
                    idx = self._param2idx[param._uuid]
                    param_arrays = param._check_and_get(param._data, list)
                    if self._fused is None:
                        self._kvstore.broadcast(idx, param_arrays[0], param_arrays)
        else:
            params_to_init = [p for p in self._params_to_init if p._deferred_init]
        self._params_to_init = params_to_init

    # ------------------------------------------------------------------ properties
    @property
    def learning_rate(self):
        if not isinstance(self._optimizer, opt.Optimizer):
            raise UserWarning('Optimizer has to be defined before its learning rate can be accessed.')
        return self._optimizer.learning_rate

    @property
    def optimizer(self):
        if isinstance(self._optimizer, opt.Optimizer):
            return self._optimizer
        raise UserWarning('Optimizer has not been initialized yet')

    def set_learning_rate(self, lr):
        if not isinstance(self._optimizer, opt.Optimizer):
            raise UserWarning('Optimizer has to be defined before its learning rate is mutated.')
        self._optimizer.set_learning_rate(lr)

    def _row_sparse_pull(self, parameter, out, row_id, full_idx=False):
        if not self._kv_initialized:
            self._init_kvstore()
        if self._params_to_init:
            self._init_params()
        idx = self._param2idx[parameter._uuid]
        self._kvstore.row_sparse_pull(idx, out=out, row_ids=row_id, priority=-idx)

    # ------------------------------------------------------------------ stepping
    def _check_and_rescale_grad(self, scale):
        if self._update_on_kvstore and self._distributed and self._kv_initialized:
            if self._optimizer.rescale_grad != scale:
                raise UserWarning('Possible change in the `batch_size` from previous `step` detected. Optimizer '
                                  'gradient normalizing factor will not change w.r.t new batch_size when '
                                  'update_on_kvstore=True and when distributed kvstore is used.')
        self._optimizer.rescale_grad = scale

    def step(self, batch_size, ignore_stale_grad=False):
        """One optimisation step: gradients are normalised by ``1/batch_size``."""
        rescale_grad = self._scale / batch_size
        self._check_and_rescale_grad(rescale_grad)
        if not self._kv_initialized:
            self._init_kvstore()
        if self._params_to_init:
            self._init_params()
        if self._fused is not None:
            self._fused.step(rescale_grad, self._amp_loss_scaler, self._fused_stale(ignore_stale_grad))
            return
        self._allreduce_grads()
        self._update(ignore_stale_grad)

    def allreduce_grads(self):
        if not self._kv_initialized:
            self._init_kvstore()
        if self._params_to_init:
            self._init_params()
        assert not (self._kvstore and self._update_on_kvstore), \
            'allreduce_grads() when parameters are updated on kvstore is not supported. Try setting ' \
            '`update_on_kvstore` to False when creating trainer.'
        if self._fused is not None:
            self._fused.allreduce_only()
            return
        self._allreduce_grads()

    def _allreduce_grads(self):
        if not self._kvstore:
            return
        for i, param in enumerate(self._params):
            if param.grad_req != 'null':
                idx = self._param2idx[param._uuid]
                grad_list = param.list_grad()
                if not self._update_on_kvstore:
                    self._kvstore.pushpull(idx, grad_list, out=grad_list, priority=-i)
                else:
                    self._kvstore.pushpull(idx, grad_list, out=param.list_data(), priority=-i)
        if hasattr(self._kvstore, 'wait_pending'):
            self._kvstore.wait_pending()       # the update that follows reads what the communication streams wrote

    def update(self, batch_size, ignore_stale_grad=False):
        if not self._kv_initialized:
            self._init_kvstore()
        if self._params_to_init:
            self._init_params()
        assert not (self._kvstore and self._update_on_kvstore), \
            'update() when parameters are updated on kvstore is not supported. Try setting `update_on_kvstore` ' \
            'to False when creating trainer.'
        self._check_and_rescale_grad(self._scale / batch_size)
        if self._fused is not None:
            self._fused.update_only(self._optimizer.rescale_grad, self._amp_loss_scaler, self._fused_stale(ignore_stale_grad))
            return
        self._update(ignore_stale_grad)

    def _fused_stale(self, ignore_stale_grad):
        """Positions (in the fused step's parameter list) whose gradient backward has not refreshed: an error unless
        ``ignore_stale_grad``, in which case the fused kernels leave those parameters and their state untouched."""
        replicas = self._fused.replica_arrays() if hasattr(self._fused, 'replica_arrays') else [self._fused._data_arrays]
        stale = [k for k in range(len(replicas[0])) if not all(arrs[k]._fresh_grad for arrs in replicas)]
        if stale and not ignore_stale_grad:
            p, arr = self._fused.params[stale[0]], self._fused._data_arrays[stale[0]]
            raise UserWarning('Gradient of Parameter `%s` on device %s has not been updated by backward since last `step`; '
                              'call step with ignore_stale_grad=True to suppress this check' % (p.name, str(arr.context)))
        return stale

    def _is_fresh(self, arr):
        """True when backward wrote this replica's gradient since the last update that consumed it
        (the `_fresh_grad` flag of python/mxnet/gluon/trainer.py:437-458).  The write-mode hook needs
        its own flag to stay set until the next pass, so consumption is tracked by backward-pass id."""
        return arr._fresh_grad and self._consumed_pass.get(id(arr)) != arr._grad_pass

    def _update(self, ignore_stale_grad=False):
        loss_scaler = self._amp_loss_scaler
        if loss_scaler is not None:
            loss_scaler._grads_unscaled = False      # only the fused step needs to know about amp.unscale()
            if loss_scaler.has_overflow(self._params):
                loss_scaler.update_scale(True)
                return          # skip the step, gradients are garbage
            loss_scaler.update_scale(False)
        if self._kvstore and self._update_on_kvstore:
            return
        updates = [[] for _ in self._updaters]
        for i, param in enumerate(self._params):
            if param.grad_req == 'null':
                continue
            datas = param._check_and_get(param._data, list)
            fresh = [self._is_fresh(d) for d in datas]
            if not ignore_stale_grad and not all(fresh):
                d = datas[fresh.index(False)]
                raise UserWarning(
                    'Gradient of Parameter `%s` on device %s has not been updated by backward since last `step`. This '
                    'could mean a bug in your model that made it only use a subset of the Parameters (Blocks) for this '
                    'iteration. If you are intentionally only using a subset, call step with ignore_stale_grad=True to '
                    'suppress this warning and skip updating of Parameters with stale gradient' % (param.name, str(d.context)))
            for upd, arr, grad, ok in zip(updates, datas, param.list_grad(), fresh):
                if ok:
                    upd.append((i, grad, arr))
        for updater, upd in zip(self._updaters, updates):
            if upd:
                i, g, w = zip(*upd)
                for arr in w:                    # consumed only now: a step refused for a stale gradient consumes nothing
                    self._consumed_pass[id(arr)] = arr._grad_pass
                updater(list(i), list(g), list(w))

    # ------------------------------------------------------------------ states
    def save_states(self, fname):
        assert self._optimizer is not None
        if not self._kv_initialized:
            self._init_kvstore()
        if self._params_to_init:
            self._init_params()
        if self._fused is not None:
            # local: this rank alone collects every shard through peer copies (no other rank has to call save_states)
            self._fused.export_states(self._updaters[0])
        if self._update_on_kvstore:
            assert not self._params_to_init, 'Cannot save trainer states when some parameters are not yet ' \
                                             'initialized in kvstore.'
            self._kvstore.save_optimizer_states(fname, dump_optimizer=True)
        else:
            with open(fname, 'wb') as fout:
                fout.write(self._updaters[0].get_states(dump_optimizer=True))

    def load_states(self, fname):
        if not self._kv_initialized:
            self._init_kvstore()
        if self._params_to_init:
            self._init_params()
        if self._update_on_kvstore:
            self._kvstore.load_optimizer_states(fname)
            self._optimizer = self._kvstore._updater.optimizer
        else:
            with open(fname, 'rb') as f:
                states = f.read()
            for updater in self._updaters:
                updater.set_states(states)
                updater.optimizer = self._updaters[0].optimizer
            self._optimizer = self._updaters[0].optimizer
        param_dict = {i: param for i, param in enumerate(self._params)}
        self._optimizer.param_dict = param_dict
        if self._fused is not None:
            self._fused.import_states(self._updaters[0], self._optimizer)

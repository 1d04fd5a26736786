"""Optimizers.  API of ``python/mxnet/optimizer/*`` (base class, registry, 20 update rules).

Semantics kept: per-index ``lr_mult``/``wd_mult`` (from ``param_dict`` or symbol attributes),
``rescale_grad``, ``clip_gradient``, per-index update counts that drive the lr scheduler,
``multi_precision`` (fp32 master copy as first element of the state, ``optimizer.py:226-253``),
``aggregate_num`` (how many tensors one fused call may take) and ``use_fused_step``.

Update math operates on the wrapped tensors directly; the multi-tensor "fused" steps of SGD/NAG/
Adam(W)/LAMB go through the registered ``multi_*`` operators, which on CUDA are single
multi-tensor-apply launches of the sm_100a kernels.
"""
from __future__ import annotations

import math
import pickle

import numpy as np
import torch

from .. import env
from ..ndarray.ndarray import NDArray
from ..ops import registry as _reg

__all__ = ['Optimizer', 'Test', 'create', 'register', 'SGD', 'NAG', 'Adam', 'AdamW', 'Adamax', 'Nadam', 'AdaGrad',
           'AdaDelta', 'AdaBelief', 'RMSProp', 'Ftrl', 'FTML', 'Signum', 'SGLD', 'DCASGD', 'LAMB', 'LANS', 'LARS',
           'GroupAdaGrad']


def _zeros_like(w, dtype=None):
    return w.__class__._from_tensor(torch.zeros_like(w._data, dtype=dtype), w._ctx)


class Optimizer(object):
    """Base class of all optimizers."""
    opt_registry = {}

    def __init__(self, rescale_grad=1., param_idx2name=None, wd=0., clip_gradient=None, learning_rate=None,
                 lr_scheduler=None, sym=None, begin_num_update=0, multi_precision=False, param_dict=None,
                 aggregate_num=None, use_fused_step=None, **kwargs):
        self.rescale_grad = rescale_grad
        self.lr_scheduler = lr_scheduler
        if self.lr_scheduler is None and learning_rate is None:
            learning_rate = 0.01
        self.lr = learning_rate
        if self.lr_scheduler is not None and learning_rate is not None:
            if self.lr_scheduler.base_lr != learning_rate:
                self.lr_scheduler.base_lr = learning_rate
        self.wd = wd
        self.lr_mult, self.wd_mult = {}, {}
        self.begin_num_update = begin_num_update
        self.num_update = begin_num_update
        self._all_index_update_counts = {0: {}}
        self._index_update_count = self._all_index_update_counts[0]
        self.clip_gradient = clip_gradient
        self.multi_precision = multi_precision
        self.aggregate_num = 1 if aggregate_num is None else aggregate_num
        param_idx2name = param_idx2name or {}
        assert isinstance(param_idx2name, dict), 'param_idx2name should be a dict of param indexes to names.'
        self.idx2name = param_idx2name.copy()
        self.sym_info = (sym.attr_dict(), sym.list_arguments()) if sym is not None else ()
        self.param_dict = param_dict if param_dict else {}
        self.use_fused_step = use_fused_step if use_fused_step is not None else False
        self.set_lr_mult({})
        self.set_wd_mult({})

    # ------------------------------------------------------------------ registry
    @staticmethod
    def register(klass):
        assert isinstance(klass, type)
        Optimizer.opt_registry[klass.__name__.lower()] = klass
        return klass

    @staticmethod
    def create_optimizer(name, **kwargs):
        if name.lower() in Optimizer.opt_registry:
            return Optimizer.opt_registry[name.lower()](**kwargs)
        raise ValueError('Cannot find optimizer %s' % name)

    # ------------------------------------------------------------------ state
    @property
    def learning_rate(self):
        if self.lr_scheduler is not None:
            return self.lr_scheduler(self.num_update)
        return self.lr

    def create_state(self, index, weight):
        return None

    def create_state_multi_precision(self, index, weight):
        if self.multi_precision and weight._data.dtype in (torch.float16, torch.bfloat16):
            master = weight.__class__._from_tensor(weight._data.detach().float(), weight._ctx)
            return (master, self.create_state(index, master))
        if weight._data.dtype == torch.float16 and not self.multi_precision:
            import warnings
            warnings.warn('Accumulating with float16 in optimizer can lead to poor accuracy or slow convergence. '
                          'Consider using multi_precision=True option of the optimizer')
        return self.create_state(index, weight)

    # ------------------------------------------------------------------ stepping
    def step(self, indices, weights, grads, states):
        raise NotImplementedError

    def fused_step(self, indices, weights, grads, states):
        self.step(indices, weights, grads, states)

    def update(self, indices, weights, grads, states):
        if not isinstance(indices, (list, tuple)):
            indices, weights, grads, states = [indices], [weights], [grads], [states]
        for w, g in zip(weights, grads):
            assert isinstance(w, NDArray) and isinstance(g, NDArray)
        lazy = [self._is_lazy(g) for g in grads]
        with torch.no_grad():
            if any(lazy):
                for i, w, g, s, is_lazy in zip(indices, weights, grads, states, lazy):
                    if is_lazy:
                        self._lazy_rows_step(i, w, g, s)
                rest = [k for k, is_lazy in enumerate(lazy) if not is_lazy]
                if not rest:
                    return
                indices, weights, grads, states = ([x[k] for k in rest] for x in (indices, weights, grads, states))
            if not self.use_fused_step:
                self.step(indices, weights, grads, states)
            else:
                self.fused_step(indices, weights, grads, states)

    def _is_lazy(self, grad):
        return getattr(self, 'lazy_update', False) and getattr(grad, 'stype', 'default') == 'row_sparse'

    def _lazy_rows_step(self, index, weight, grad, state):
        """Lazy update with a row-sparse gradient (``lazy_update=True``; ``src/operator/optimizer_op.cc`` SGDUpdateRspImpl,
        AdamLazyUpdate ...): only the rows present in the gradient are touched: weight decay, momentum decay and the moment
        estimates of all other rows stay as they are.  The rows of the weight and of every state tensor are gathered, the
        optimizer's ordinary step runs on them, and the results are scattered back."""
        vals, rows = grad._components()
        if rows.numel() == 0:
            self._update_count([index])
            return
        rows = rows.long()
        n = weight._data.shape[0]

        def gather(x):
            if isinstance(x, NDArray):
                return NDArray._from_tensor(x._data[rows], x._ctx) if x._data.dim() and x._data.shape[0] == n else x
            if isinstance(x, (list, tuple)):
                return type(x)(gather(v) for v in x)
            return x

        def scatter(full, part):
            if isinstance(full, NDArray):
                if part is not full:
                    full._data[rows] = part._data
            elif isinstance(full, (list, tuple)):
                for f, q in zip(full, part):
                    scatter(f, q)
        sub_w, sub_s = gather(weight), gather(state)
        self.step([index], [sub_w], [NDArray._from_tensor(vals.to(sub_w._data.dtype), weight._ctx)], [sub_s])
        scatter(weight, sub_w)
        scatter(state, sub_s)

    def update_multi_precision(self, indices, weights, grads, states):
        if not isinstance(indices, (list, tuple)):
            indices, weights, grads, states = [indices], [weights], [grads], [states]
        mp = [self.multi_precision and w._data.dtype in (torch.float16, torch.bfloat16) for w in weights]
        if not any(mp):
            self.update(indices, weights, grads, states)
            return
        if self.use_fused_step and all(mp) and hasattr(self, '_fused_step_mp') and not any(self._is_lazy(g) for g in grads):
            with torch.no_grad():
                self._fused_step_mp(indices, weights, grads, states)
            return
        w32, g32, st = [], [], []
        for w, g, s, is_mp in zip(weights, grads, states, mp):
            if is_mp:
                w32.append(s[0])
                g32.append(g.astype('float32') if self._is_lazy(g) else g.__class__._from_tensor(g._data.float(), g._ctx))
                st.append(s[1])
            else:
                w32.append(w); g32.append(g); st.append(s)
        self.update(indices, w32, g32, st)
        with torch.no_grad():
            for w, m, is_mp in zip(weights, w32, mp):
                if is_mp:
                    w._data.copy_(m._data)

    # ------------------------------------------------------------------ hyper-parameters
    def set_learning_rate(self, lr):
        if self.lr_scheduler is not None:
            raise UserWarning('LRScheduler of the optimizer has already been defined. Note that set_learning_rate '
                              'can mutate the value of the learning rate of the optimizer only when the LRScheduler '
                              'of the optimizer is undefined.')
        self.lr = lr

    def set_lr_mult(self, args_lr_mult):
        self.lr_mult = {}
        if self.sym_info:
            attr, arg_names = self.sym_info
            for name in arg_names:
                if name in attr and '__lr_mult__' in attr[name]:
                    self.lr_mult[name] = float(attr[name]['__lr_mult__'])
        self.lr_mult.update(args_lr_mult)

    def set_wd_mult(self, args_wd_mult):
        self.wd_mult = {}
        if self.sym_info:
            attr, arg_names = self.sym_info
            for name in arg_names:
                if name in attr and '__wd_mult__' in attr[name]:
                    self.wd_mult[name] = float(attr[name]['__wd_mult__'])
        self.wd_mult.update(args_wd_mult)

    def _set_current_context(self, device_id):
        if device_id not in self._all_index_update_counts:
            self._all_index_update_counts[device_id] = {}
        self._index_update_count = self._all_index_update_counts[device_id]

    _set_current_device = _set_current_context

    def _update_count(self, index):
        if not isinstance(index, (list, tuple)):
            index = [index]
        for idx in index:
            if idx not in self._index_update_count:
                self._index_update_count[idx] = self.begin_num_update
            self._index_update_count[idx] += 1
            self.num_update = max(self._index_update_count[idx], self.num_update)

    def _get_lrs(self, indices):
        lr = self.lr_scheduler(self.num_update) if self.lr_scheduler is not None else self.lr
        lrs = [lr for _ in indices]
        for i, index in enumerate(indices):
            if index in self.param_dict:
                lrs[i] *= self.param_dict[index].lr_mult
            elif index in self.lr_mult:
                lrs[i] *= self.lr_mult[index]
            elif index in self.idx2name:
                lrs[i] *= self.lr_mult.get(self.idx2name[index], 1.0)
        return lrs

    def _get_lr(self, index):
        return self._get_lrs([index])[0]

    def _get_wds(self, indices):
        wds = [self.wd for _ in indices]
        for i, index in enumerate(indices):
            if index in self.param_dict:
                wds[i] *= self.param_dict[index].wd_mult
            elif index in self.wd_mult:
                wds[i] *= self.wd_mult[index]
            elif index in self.idx2name:
                wds[i] *= self.wd_mult.get(self.idx2name[index], 1.0)
        return wds

    def _get_wd(self, index):
        return self._get_wds([index])[0]

    def _grad(self, g, w=None, wd=0.0):
        """``clip(rescale_grad * g)`` (+ ``wd * w`` when a weight is given)."""
        t = g._data
        if self.rescale_grad != 1.0:
            t = t * self.rescale_grad
        if self.clip_gradient is not None:
            t = t.clamp(-self.clip_gradient, self.clip_gradient)
        if w is not None and wd != 0.0:
            t = t + wd * w._data
        return t

    def __getstate__(self):
        ret = self.__dict__.copy()
        # parameters are not pickled with the optimizer (they hold device memory)
        ret['param_dict'] = {}
        return ret

    def __setstate__(self, state):
        self.__dict__ = state
        self.param_dict = {}


register = Optimizer.register
create = Optimizer.create_optimizer


@register
class Test(Optimizer):
    """``w += rescale_grad * g`` — the deterministic rule used by KVStore tests (``optimizer.py:564-583``)."""

    def create_state(self, index, weight):
        return _zeros_like(weight)

    def step(self, indices, weights, grads, states):
        for w, g, s in zip(weights, grads, states):
            w._data.add_(g._data * self.rescale_grad)
            s._data.copy_(w._data)


@register
class SGD(Optimizer):
    """SGD with momentum; ``m ← μ·m − lr·(g' + wd·w)``, ``w ← w + m`` (``optimizer/sgd.py``)."""

    def __init__(self, learning_rate=0.1, momentum=0.0, lazy_update=False, multi_precision=False,
                 use_fused_step=True, aggregate_num=None, **kwargs):
        if aggregate_num is None:
            aggregate_num = max(1, min(50, int(env.get('MXNET_OPTIMIZER_AGGREGATION_SIZE'))))
        super().__init__(learning_rate=learning_rate, multi_precision=multi_precision, aggregate_num=aggregate_num,
                         use_fused_step=use_fused_step, **kwargs)
        self.momentum = momentum
        self.lazy_update = lazy_update

    def create_state(self, index, weight):
        return _zeros_like(weight) if self.momentum != 0.0 else None

    def step(self, indices, weights, grads, states):
        self._update_count(indices)
        lrs, wds = self._get_lrs(indices), self._get_wds(indices)
        for w, g, s, lr, wd in zip(weights, grads, states, lrs, wds):
            gg = self._grad(g, w, wd)
            if s is not None:
                s._data.mul_(self.momentum).add_(gg, alpha=-lr)
                w._data.add_(s._data)
            else:
                w._data.add_(gg, alpha=-lr)

    def _multi(self, indices, weights, grads, moms, masters):
        self._update_count(indices)
        lrs, wds = self._get_lrs(indices), self._get_wds(indices)
        clip = -1.0 if self.clip_gradient is None else self.clip_gradient
        n = len(weights)
        name = ('multi_mp_sgd' if masters else 'multi_sgd') + ('_mom_update' if moms else '_update')
        flat = []
        for i in range(n):
            flat += [weights[i], grads[i]]
            if moms:
                flat.append(moms[i])
            if masters:
                flat.append(masters[i])
        attrs = {'lrs': lrs, 'wds': wds, 'rescale_grad': self.rescale_grad, 'clip_gradient': clip, 'num_weights': n}
        if moms:
            attrs['momentum'] = self.momentum
        _reg.invoke(name, flat, attrs, out=list(weights))

    def fused_step(self, indices, weights, grads, states):
        self._multi(indices, weights, grads, list(states) if self.momentum != 0.0 else None, None)

    def _fused_step_mp(self, indices, weights, grads, states):
        masters = [s[0] for s in states]
        moms = [s[1] for s in states] if self.momentum != 0.0 else None
        self._multi(indices, weights, grads, moms, masters)


@register
class NAG(SGD):
    """Nesterov momentum (``optimizer_op-inl.h:1107-1131``)."""

    def __init__(self, learning_rate=0.1, momentum=0.9, multi_precision=False, use_fused_step=True, **kwargs):
        super().__init__(learning_rate=learning_rate, momentum=momentum, multi_precision=multi_precision,
                         use_fused_step=use_fused_step, **kwargs)

    def step(self, indices, weights, grads, states):
        self._update_count(indices)
        lrs, wds = self._get_lrs(indices), self._get_wds(indices)
        for w, g, s, lr, wd in zip(weights, grads, states, lrs, wds):
            gg = self._grad(g, w, wd)
            if s is not None:
                s._data.mul_(self.momentum).add_(gg, alpha=-lr)
                w._data.add_(s._data, alpha=self.momentum).add_(gg, alpha=-lr)
            else:
                w._data.add_(gg, alpha=-lr)

    fused_step = step

    def _fused_step_mp(self, indices, weights, grads, states):
        masters = [s[0] for s in states]
        moms = [s[1] for s in states]
        g32 = [g.__class__._from_tensor(g._data.float(), g._ctx) for g in grads]
        self.step(indices, masters, g32, moms)
        for w, m in zip(weights, masters):
            w._data.copy_(m._data)


@register
class SGLD(Optimizer):
    """Stochastic gradient Langevin dynamics."""

    def step(self, indices, weights, grads, states):
        self._update_count(indices)
        lrs, wds = self._get_lrs(indices), self._get_wds(indices)
        for w, g, lr, wd in zip(weights, grads, lrs, wds):
            gg = self._grad(g, w, wd)
            w._data.add_(gg, alpha=-lr / 2).add_(torch.randn_like(w._data) * math.sqrt(lr))


@register
class Signum(Optimizer):
    def __init__(self, learning_rate=0.01, momentum=0.9, wd_lh=0.0, use_fused_step=True, **kwargs):
        super().__init__(learning_rate=learning_rate, use_fused_step=use_fused_step, **kwargs)
        self.momentum, self.wd_lh = momentum, wd_lh

    def create_state(self, index, weight):
        return _zeros_like(weight) if self.momentum != 0.0 else None

    def step(self, indices, weights, grads, states):
        self._update_count(indices)
        lrs, wds = self._get_lrs(indices), self._get_wds(indices)
        for w, g, s, lr, wd in zip(weights, grads, states, lrs, wds):
            gg = self._grad(g, w, wd)
            if s is not None:
                s._data.mul_(self.momentum).sub_(gg, alpha=1 - self.momentum)
                w._data.mul_(1 - lr * self.wd_lh).add_(torch.sign(s._data), alpha=lr)
            else:
                w._data.mul_(1 - lr * self.wd_lh).sub_(torch.sign(gg), alpha=lr)


@register
class DCASGD(Optimizer):
    """Delay-compensated asynchronous SGD."""

    def __init__(self, learning_rate=0.1, momentum=0.0, lamda=0.04, use_fused_step=False, **kwargs):
        super().__init__(learning_rate=learning_rate, use_fused_step=use_fused_step, **kwargs)
        self.momentum, self.lamda = momentum, lamda

    def create_state(self, index, weight):
        return (_zeros_like(weight) if self.momentum != 0.0 else None, weight.copy())

    def step(self, indices, weights, grads, states):
        self._update_count(indices)
        lrs, wds = self._get_lrs(indices), self._get_wds(indices)
        for w, g, (mom, prev), lr, wd in zip(weights, grads, states, lrs, wds):
            gg = self._grad(g, w, wd)
            d = gg + self.lamda * gg * gg * (w._data - prev._data)
            if mom is not None:
                mom._data.mul_(self.momentum).add_(d, alpha=-lr)
                upd = mom._data
            else:
                upd = -lr * d
            prev._data.copy_(w._data)
            w._data.add_(upd)


@register
class Adam(Optimizer):
    """Adam; bias correction folded into the step size (``optimizer/adam.py``)."""

    def __init__(self, learning_rate=0.001, beta1=0.9, beta2=0.999, epsilon=1e-8, lazy_update=False,
                 use_fused_step=True, **kwargs):
        super().__init__(learning_rate=learning_rate, use_fused_step=use_fused_step, **kwargs)
        self.beta1, self.beta2, self.epsilon, self.lazy_update = beta1, beta2, epsilon, lazy_update

    def create_state(self, index, weight):
        return (_zeros_like(weight), _zeros_like(weight))

    def step(self, indices, weights, grads, states):
        for index, w, g, (mean, var) in zip(indices, weights, grads, states):
            self._update_count(index)
            lr, wd = self._get_lr(index), self._get_wd(index)
            t = self._index_update_count[index]
            gg = self._grad(g, w, wd)
            lr *= math.sqrt(1. - self.beta2 ** t) / (1. - self.beta1 ** t)
            mean._data.mul_(self.beta1).add_(gg, alpha=1 - self.beta1)
            var._data.mul_(self.beta2).addcmul_(gg, gg, value=1 - self.beta2)
            w._data.addcdiv_(mean._data, var._data.sqrt().add_(self.epsilon), value=-lr)


@register
class AdamW(Optimizer):
    """Adam with decoupled weight decay (``optimizer/adamW.py``, ``src/operator/contrib/adamw.cc``)."""

    def __init__(self, learning_rate=0.001, beta1=0.9, beta2=0.999, epsilon=1e-6, correct_bias=True,
                 use_fused_step=True, **kwargs):
        super().__init__(learning_rate=learning_rate, use_fused_step=use_fused_step, **kwargs)
        self.beta1, self.beta2, self.epsilon, self.correct_bias = beta1, beta2, epsilon, correct_bias

    def create_state(self, index, weight):
        return (_zeros_like(weight), _zeros_like(weight))

    def step(self, indices, weights, grads, states):
        for index, w, g, (mean, var) in zip(indices, weights, grads, states):
            self._update_count(index)
            lr, wd = self._get_lr(index), self._get_wd(index)
            t = self._index_update_count[index]
            gg = self._grad(g)
            if self.correct_bias:
                lr *= math.sqrt(1. - self.beta2 ** t) / (1. - self.beta1 ** t)
            mean._data.mul_(self.beta1).add_(gg, alpha=1 - self.beta1)
            var._data.mul_(self.beta2).addcmul_(gg, gg, value=1 - self.beta2)
            w._data.addcdiv_(mean._data, var._data.sqrt().add_(self.epsilon), value=-lr)
            if wd > 0:
                w._data.mul_(1 - lr * wd)


@register
class Adamax(Optimizer):
    def __init__(self, learning_rate=0.002, beta1=0.9, beta2=0.999, use_fused_step=False, **kwargs):
        super().__init__(learning_rate=learning_rate, use_fused_step=use_fused_step, **kwargs)
        self.beta1, self.beta2 = beta1, beta2

    def create_state(self, index, weight):
        return (_zeros_like(weight), _zeros_like(weight))

    def step(self, indices, weights, grads, states):
        for index, w, g, (m, u) in zip(indices, weights, grads, states):
            self._update_count(index)
            lr, wd = self._get_lr(index), self._get_wd(index)
            t = self._index_update_count[index]
            lr /= (1. - self.beta1 ** t)
            gg = self._grad(g, w, wd)
            m._data.mul_(self.beta1).add_(gg, alpha=1 - self.beta1)
            u._data.copy_(torch.maximum(self.beta2 * u._data, gg.abs()))
            w._data.addcdiv_(m._data, u._data, value=-lr)


@register
class Nadam(Optimizer):
    def __init__(self, learning_rate=0.001, beta1=0.9, beta2=0.999, epsilon=1e-8, schedule_decay=0.004,
                 use_fused_step=False, **kwargs):
        super().__init__(learning_rate=learning_rate, use_fused_step=use_fused_step, **kwargs)
        self.beta1, self.beta2, self.epsilon, self.schedule_decay = beta1, beta2, epsilon, schedule_decay
        self.m_schedule = 1.

    def create_state(self, index, weight):
        return (_zeros_like(weight), _zeros_like(weight))

    def step(self, indices, weights, grads, states):
        for index, w, g, (m, v) in zip(indices, weights, grads, states):
            self._update_count(index)
            lr, wd = self._get_lr(index), self._get_wd(index)
            t = self._index_update_count[index]
            gg = self._grad(g, w, wd)
            mom_t = self.beta1 * (1. - 0.5 * (pow(0.96, t * self.schedule_decay)))
            mom_t1 = self.beta1 * (1. - 0.5 * (pow(0.96, (t + 1) * self.schedule_decay)))
            self.m_schedule = self.m_schedule * mom_t
            m_sched_next = self.m_schedule * mom_t1
            m._data.mul_(self.beta1).add_(gg, alpha=1 - self.beta1)
            v._data.mul_(self.beta2).addcmul_(gg, gg, value=1 - self.beta2)
            g_prime = gg / (1. - self.m_schedule)
            m_prime = m._data / (1. - m_sched_next)
            v_prime = v._data / (1. - pow(self.beta2, t))
            m_bar = (1. - mom_t) * g_prime + mom_t1 * m_prime
            w._data.sub_(lr * m_bar / (v_prime.sqrt() + self.epsilon))


@register
class AdaGrad(Optimizer):
    def __init__(self, learning_rate=0.01, epsilon=1e-6, use_fused_step=True, **kwargs):
        super().__init__(learning_rate=learning_rate, use_fused_step=use_fused_step, **kwargs)
        self.epsilon = epsilon

    def create_state(self, index, weight):
        return _zeros_like(weight)

    def step(self, indices, weights, grads, states):
        self._update_count(indices)
        lrs, wds = self._get_lrs(indices), self._get_wds(indices)
        for w, g, h, lr, wd in zip(weights, grads, states, lrs, wds):
            gg = self._grad(g, w, wd)
            h._data.addcmul_(gg, gg)
            w._data.sub_(lr * gg / (h._data.sqrt() + self.epsilon))


@register
class GroupAdaGrad(Optimizer):
    """AdaGrad with one accumulator per row (``optimizer/contrib.py``)."""

    def __init__(self, learning_rate=0.01, epsilon=1e-6, use_fused_step=True, **kwargs):
        super().__init__(learning_rate=learning_rate, use_fused_step=use_fused_step, **kwargs)
        self.epsilon = epsilon

    def create_state(self, index, weight):
        assert len(weight.shape) == 2
        return weight.__class__._from_tensor(torch.zeros(weight.shape[0], 1, dtype=weight._data.dtype,
                                                         device=weight._data.device), weight._ctx)

    def step(self, indices, weights, grads, states):
        self._update_count(indices)
        lrs = self._get_lrs(indices)
        for w, g, h, lr in zip(weights, grads, states, lrs):
            assert self._get_wd(0) == 0 or self.wd == 0, 'Weight decay is not supported for GroupAdaGrad'
            gg = self._grad(g)
            h._data.add_((gg * gg).mean(1, keepdim=True))
            w._data.sub_(lr * gg / (h._data.sqrt() + self.epsilon))


@register
class AdaDelta(Optimizer):
    def __init__(self, learning_rate=1.0, rho=0.9, epsilon=1e-6, use_fused_step=False, **kwargs):
        super().__init__(learning_rate=learning_rate, use_fused_step=use_fused_step, **kwargs)
        self.rho, self.epsilon = rho, epsilon

    def create_state(self, index, weight):
        return (_zeros_like(weight), _zeros_like(weight))

    def step(self, indices, weights, grads, states):
        self._update_count(indices)
        lrs, wds = self._get_lrs(indices), self._get_wds(indices)
        for w, g, (acc_g, acc_d), lr, wd in zip(weights, grads, states, lrs, wds):
            gg = self._grad(g, w, wd)
            acc_g._data.mul_(self.rho).addcmul_(gg, gg, value=1 - self.rho)
            delta = (acc_d._data + self.epsilon).sqrt() / (acc_g._data + self.epsilon).sqrt() * gg
            acc_d._data.mul_(self.rho).addcmul_(delta, delta, value=1 - self.rho)
            w._data.sub_(lr * delta)


@register
class AdaBelief(Optimizer):
    def __init__(self, learning_rate=0.001, beta1=0.9, beta2=0.999, epsilon=1e-6, correct_bias=True,
                 use_fused_step=True, **kwargs):
        super().__init__(learning_rate=learning_rate, use_fused_step=use_fused_step, **kwargs)
        self.beta1, self.beta2, self.epsilon, self.correct_bias = beta1, beta2, epsilon, correct_bias

    def create_state(self, index, weight):
        return (_zeros_like(weight), _zeros_like(weight))

    def step(self, indices, weights, grads, states):
        for index, w, g, (mean, var) in zip(indices, weights, grads, states):
            self._update_count(index)
            lr, wd = self._get_lr(index), self._get_wd(index)
            t = self._index_update_count[index]
            gg = self._grad(g, w, wd)
            if self.correct_bias:
                lr *= math.sqrt(1. - self.beta2 ** t) / (1. - self.beta1 ** t)
            mean._data.mul_(self.beta1).add_(gg, alpha=1 - self.beta1)
            diff = gg - mean._data
            var._data.mul_(self.beta2).addcmul_(diff, diff, value=1 - self.beta2).add_(self.epsilon)
            w._data.addcdiv_(mean._data, var._data.sqrt().add_(self.epsilon), value=-lr)


@register
class RMSProp(Optimizer):
    def __init__(self, learning_rate=0.001, rho=0.9, momentum=0.9, epsilon=1e-8, centered=False, clip_weights=None,
                 use_fused_step=True, **kwargs):
        super().__init__(learning_rate=learning_rate, use_fused_step=use_fused_step, **kwargs)
        self.rho, self.momentum, self.centered, self.epsilon, self.clip_weights = rho, momentum, centered, epsilon, clip_weights

    def create_state(self, index, weight):
        if self.centered:
            return (_zeros_like(weight), _zeros_like(weight), _zeros_like(weight))
        return _zeros_like(weight)

    def step(self, indices, weights, grads, states):
        self._update_count(indices)
        lrs, wds = self._get_lrs(indices), self._get_wds(indices)
        for w, g, s, lr, wd in zip(weights, grads, states, lrs, wds):
            gg = self._grad(g, w, wd)
            if not self.centered:
                s._data.mul_(self.rho).addcmul_(gg, gg, value=1 - self.rho)
                w._data.sub_(lr * gg / (s._data.sqrt() + self.epsilon))
            else:
                n, gm, delta = s
                n._data.mul_(self.rho).addcmul_(gg, gg, value=1 - self.rho)
                gm._data.mul_(self.rho).add_(gg, alpha=1 - self.rho)
                delta._data.mul_(self.momentum).sub_(lr * gg / (n._data - gm._data * gm._data + self.epsilon).sqrt())
                w._data.add_(delta._data)
            if self.clip_weights:
                w._data.clamp_(-self.clip_weights, self.clip_weights)


@register
class Ftrl(Optimizer):
    def __init__(self, learning_rate=0.1, lamda1=0.01, beta=1., use_fused_step=True, **kwargs):
        super().__init__(learning_rate=learning_rate, use_fused_step=use_fused_step, **kwargs)
        self.lamda1, self.beta = lamda1, beta

    def create_state(self, index, weight):
        return (_zeros_like(weight), _zeros_like(weight))

    def step(self, indices, weights, grads, states):
        self._update_count(indices)
        lrs, wds = self._get_lrs(indices), self._get_wds(indices)
        for w, g, (z, n), lr, wd in zip(weights, grads, states, lrs, wds):
            gg = self._grad(g)
            z._data.add_(gg - ((n._data + gg * gg).sqrt() - n._data.sqrt()) * w._data / lr)
            n._data.addcmul_(gg, gg)
            new_w = (torch.sign(z._data) * self.lamda1 - z._data) / ((self.beta + n._data.sqrt()) / lr + wd) * \
                (z._data.abs() > self.lamda1).to(w._data.dtype)
            w._data.copy_(new_w)


@register
class FTML(Optimizer):
    def __init__(self, learning_rate=0.0025, beta1=0.6, beta2=0.999, epsilon=1e-8, use_fused_step=True, **kwargs):
        super().__init__(learning_rate=learning_rate, use_fused_step=use_fused_step, **kwargs)
        self.beta1, self.beta2, self.epsilon = beta1, beta2, epsilon

    def create_state(self, index, weight):
        return (_zeros_like(weight), _zeros_like(weight), _zeros_like(weight))

    def step(self, indices, weights, grads, states):
        for index, w, g, (d, v, z) in zip(indices, weights, grads, states):
            self._update_count(index)
            lr, wd = self._get_lr(index), self._get_wd(index)
            t = self._index_update_count[index]
            gg = self._grad(g, w, wd)
            v._data.mul_(self.beta2).addcmul_(gg, gg, value=1 - self.beta2)
            d_t = (1. - self.beta1 ** t) / lr * ((v._data / (1. - self.beta2 ** t)).sqrt() + self.epsilon)
            sigma = d_t - self.beta1 * d._data
            z._data.mul_(self.beta1).add_((1. - self.beta1) * gg - sigma * w._data)
            d._data.copy_(d_t)
            w._data.copy_(-z._data / d_t)


@register
class LAMB(Optimizer):
    """Layer-wise adaptive moments (``optimizer/lamb.py``; phases in ``optimizer_op-inl.h:1736-1870``)."""

    def __init__(self, learning_rate=0.001, beta1=0.9, beta2=0.999, epsilon=1e-6, lower_bound=None, upper_bound=None,
                 bias_correction=True, aggregate_num=4, use_fused_step=True, **kwargs):
        assert aggregate_num <= 45, 'When use_fused_step is True, LAMB only supports aggregate_num <= 45'
        super().__init__(learning_rate=learning_rate, aggregate_num=aggregate_num, use_fused_step=use_fused_step, **kwargs)
        self.beta1, self.beta2, self.epsilon = beta1, beta2, epsilon
        self.lower_bound, self.upper_bound, self.bias_correction = lower_bound, upper_bound, bias_correction

    def create_state(self, index, weight):
        dt = torch.float32 if weight._data.dtype in (torch.float16, torch.bfloat16) else None
        return (_zeros_like(weight, dt), _zeros_like(weight, dt))

    def step(self, indices, weights, grads, states):
        for index, w, g, (mean, var) in zip(indices, weights, grads, states):
            self._update_count(index)
            lr, wd = self._get_lr(index), self._get_wd(index)
            t = self._index_update_count[index]
            gg = self._grad(g).to(mean._data.dtype)
            mean._data.mul_(self.beta1).add_(gg, alpha=1 - self.beta1)
            var._data.mul_(self.beta2).addcmul_(gg, gg, value=1 - self.beta2)
            if self.bias_correction:
                mh = mean._data / (1. - self.beta1 ** t)
                vh = var._data / (1. - self.beta2 ** t)
            else:
                mh, vh = mean._data, var._data
            u = mh / (vh.sqrt() + self.epsilon) + wd * w._data.to(mh.dtype)
            r1 = w._data.float().norm()
            if self.lower_bound is not None:
                r1 = r1.clamp(min=self.lower_bound)
            if self.upper_bound is not None:
                r1 = r1.clamp(max=self.upper_bound)
            r2 = u.float().norm()
            ratio = torch.where((r1 == 0) | (r2 == 0), torch.ones_like(r1), r1 / r2)
            w._data.sub_((lr * ratio * u).to(w._data.dtype))

    def _fused(self, indices, weights, grads, states, mp):
        self._update_count(indices)
        lrs, wds = self._get_lrs(indices), self._get_wds(indices)
        steps = [self._index_update_count[i] for i in indices]
        flat = []
        for i, (w, g, s) in enumerate(zip(weights, grads, states)):
            if mp:
                flat += [w, g, s[1][0], s[1][1], s[0]]
            else:
                flat += [w, g, s[0], s[1]]
        attrs = {'learning_rates': lrs, 'wds': wds, 'beta1': self.beta1, 'beta2': self.beta2, 'epsilon': self.epsilon,
                 'rescale_grad': self.rescale_grad, 'lower_bound': -1.0 if self.lower_bound is None else self.lower_bound,
                 'upper_bound': -1.0 if self.upper_bound is None else self.upper_bound,
                 'clip_gradient': -1.0 if self.clip_gradient is None else self.clip_gradient,
                 'bias_correction': self.bias_correction, 'step_count': steps, 'num_tensors': len(weights)}
        _reg.invoke('_multi_mp_lamb_update' if mp else '_multi_lamb_update', flat, attrs, out=list(weights))

    def fused_step(self, indices, weights, grads, states):
        self._fused(indices, weights, grads, states, False)

    def _fused_step_mp(self, indices, weights, grads, states):
        self._fused(indices, weights, grads, states, True)


@register
class LANS(LAMB):
    """LAMB with normalised gradients and Nesterov-style second trust ratio (``optimizer/lans.py``)."""

    def step(self, indices, weights, grads, states):
        from ..ops.optimizer_ops import _lans_step
        for index, w, g, (mean, var) in zip(indices, weights, grads, states):
            self._update_count(index)
            lr, wd = self._get_lr(index), self._get_wd(index)
            t = self._index_update_count[index]
            _lans_step(w._data, g._data, mean._data, var._data, lr, wd, self.beta1, self.beta2, self.epsilon, t,
                       self.rescale_grad, -1.0 if self.lower_bound is None else self.lower_bound,
                       -1.0 if self.upper_bound is None else self.upper_bound,
                       -1.0 if self.clip_gradient is None else self.clip_gradient)

    fused_step = step

    def _fused_step_mp(self, indices, weights, grads, states):
        self.step(indices, [s[0] for s in states], grads, [s[1] for s in states])
        for w, s in zip(weights, states):
            w._data.copy_(s[0]._data)


@register
class LARS(Optimizer):
    """Layer-wise adaptive rate scaling on top of momentum SGD (``optimizer/lars.py``)."""

    def __init__(self, learning_rate=0.1, momentum=0.0, eta=0.001, epsilon=1e-8, lazy_update=False,
                 use_fused_step=True, aggregate_num=None, **kwargs):
        super().__init__(learning_rate=learning_rate, use_fused_step=use_fused_step,
                         aggregate_num=aggregate_num or 4, **kwargs)
        self.momentum, self.eta, self.epsilon = momentum, eta, epsilon

    def create_state(self, index, weight):
        return _zeros_like(weight) if self.momentum != 0.0 else None

    def _is_excluded(self, index):
        name = self.idx2name.get(index, str(index)) if not isinstance(index, str) else index
        return name.endswith('gamma') or name.endswith('beta') or name.endswith('bias')

    def step(self, indices, weights, grads, states):
        self._update_count(indices)
        lrs, wds = self._get_lrs(indices), self._get_wds(indices)
        for index, w, g, s, lr, wd in zip(indices, weights, grads, states, lrs, wds):
            if not self._is_excluded(index):
                w_norm = w._data.float().norm()
                g_norm = g._data.float().norm() * self.rescale_grad
                ratio = torch.where((w_norm > 0) & (g_norm > 0), self.eta * w_norm / (g_norm + wd * w_norm + self.epsilon),
                                    torch.ones_like(w_norm))
                lr = lr * ratio
            gg = self._grad(g, w, wd)
            if s is not None:
                s._data.mul_(self.momentum).sub_(gg * lr)
                w._data.add_(s._data)
            else:
                w._data.sub_(gg * lr)

"""Automatic mixed precision (``python/mxnet/amp/amp.py``).

``init()`` turns on the cast policy: the reference monkey-patches every generated operator function
with casting wrappers driven by the lists; here every operator call already funnels through
``ops.registry.invoke`` (and ``Symbol._run``), so the policy is a single hook consulted there.
``init_trainer`` attaches a dynamic ``LossScaler``; ``scale_loss`` multiplies the loss and folds
``1/loss_scale`` into ``trainer._scale`` so unscaling rides on ``rescale_grad``
(``amp.py:291-299``); ``convert_symbol`` / ``convert_hybrid_block`` rewrite graphs with ``amp_cast``.
"""
import contextlib
import warnings

import torch

from .. import _state
from ..base import to_torch_dtype
from .lists import symbol_fp16, symbol_bf16
from .loss_scaler import LossScaler

__all__ = ['init', 'init_trainer', 'scale_loss', 'unscale', 'convert_model', 'convert_symbol', 'convert_hybrid_block',
           'list_lp16_ops', 'list_fp32_ops', 'list_lp16_fp32_ops', 'list_conditional_fp32_ops', 'list_widest_type_cast',
           'list_loss_output_functions', 'list_lp16_use_fp32_params']

_amp_initialized = False
_amp_loss_scale_initialized = False
_target = None
_sets = None
_ORDER = [torch.float16, torch.bfloat16, torch.float32, torch.float64]


def _lists(target_dtype):
    return symbol_bf16 if to_torch_dtype(target_dtype) == torch.bfloat16 else symbol_fp16


def _expand(names):
    """Include every alias of the listed operators."""
    from ..ops import registry as reg
    out = set()
    for n in names:
        out.add(n)
        if reg.has(n):
            op = reg.get(n)
            out.add(op.name)
            out.update(op.aliases)
    return out


def _hook(opname, tensors):
    lp, fp32, widest = _sets
    if opname in lp:
        return [t.to(_target) if isinstance(t, torch.Tensor) and t.is_floating_point() and t.dtype != _target else t
                for t in tensors]
    if opname in fp32:
        return [t.float() if isinstance(t, torch.Tensor) and t.dtype in (torch.float16, torch.bfloat16) else t
                for t in tensors]
    if opname in widest:
        fl = [t.dtype for t in tensors if isinstance(t, torch.Tensor) and t.is_floating_point()]
        if len(set(fl)) > 1:
            tgt = max(fl, key=_ORDER.index)
            return [t.to(tgt) if isinstance(t, torch.Tensor) and t.is_floating_point() else t for t in tensors]
    return tensors


from ..base import bfloat16   # noqa: E402,F401  (the dtype name scripts import from this module)


def init(target_dtype='float16', target_precision_ops=None, conditional_fp32_ops=None, fp32_ops=None, layout_optimization=False):
    """Turn on AMP for all subsequently executed operators."""
    global _amp_initialized, _target, _sets
    td = to_torch_dtype(target_dtype)
    assert td in (torch.float16, torch.bfloat16), 'AMP currently supports only float16 or bfloat16 as a target_dtype'
    if _amp_initialized:
        return
    lists = _lists(td)
    lp = list(target_precision_ops) if target_precision_ops is not None else \
        list(lists.BF16_FUNCS if td == torch.bfloat16 else lists.FP16_FUNCS)
    f32 = list(fp32_ops) if fp32_ops is not None else list(lists.FP32_FUNCS)
    _target = td
    _sets = (_expand(lp), _expand(f32), _expand(lists.WIDEST_TYPE_CASTS))
    _state.amp_hook = _hook
    _amp_initialized = True
    if layout_optimization:
        from ..symbol.layout import set_optimize_layout
        set_optimize_layout(True)


def _reset():
    """Turn AMP off again (tests)."""
    global _amp_initialized, _amp_loss_scale_initialized
    _state.amp_hook = None
    _amp_initialized = False
    _amp_loss_scale_initialized = False


def init_trainer(optimizer_or_trainer):
    """Attach a dynamic loss scaler to a Trainer."""
    global _amp_loss_scale_initialized
    from ..gluon.trainer import Trainer
    if not _amp_initialized:
        raise RuntimeError('AMP init function should be called before init_trainer')
    loss_scaler = LossScaler()
    _amp_loss_scale_initialized = True
    if isinstance(optimizer_or_trainer, Trainer):
        optimizer_or_trainer._amp_loss_scaler = loss_scaler
        optimizer_or_trainer._amp_original_scale = optimizer_or_trainer._scale
        if _target == torch.bfloat16:
            loss_scaler._loss_scale = 1.0
            loss_scaler._max_loss_scale = 1.0
        # bring up the optimizer path now when the parameters already exist, so that the loss scale can
        # live on the device from the first step on
        tr = optimizer_or_trainer
        ready = all(p._data is not None for p in tr._params)
        if ready and not tr._kv_initialized:
            tr._init_kvstore()
        if tr._fused is not None:
            tr._fused.attach_scaler(loss_scaler)
    else:
        raise TypeError('optimizer_or_trainer should be a Gluon Trainer instance, instead is %s' % type(optimizer_or_trainer))


@contextlib.contextmanager
def scale_loss(loss, optimizer_or_trainer):
    """``with amp.scale_loss(loss, trainer) as scaled: autograd.backward(scaled)``."""
    scaler = optimizer_or_trainer._amp_loss_scaler
    assert scaler is not None, 'Loss scaler is not initialized, did you forget to call amp.init_trainer()?'
    if scaler._device_state is not None:
        # the scale lives on the device (fused optimizer step): multiply by the device scalar, the
        # kernels divide it out again; the host never reads it, so there is no synchronisation here
        optimizer_or_trainer._scale = optimizer_or_trainer._amp_original_scale
        def scaled(l):
            # the copy of the scale that lives on the loss's own GPU (a single-process group keeps one per GPU)
            state = scaler._device_states.get(l._data.device, scaler._device_state)
            s_arr = l.__class__._from_tensor(state[0:1], l.context)
            return l * (s_arr.astype(l.dtype) if l.dtype != s_arr.dtype else s_arr)
        if isinstance(loss, (list, tuple)):
            yield [scaled(l) for l in loss]
        else:
            yield scaled(loss)
        return
    s = scaler.loss_scale
    optimizer_or_trainer._scale = optimizer_or_trainer._amp_original_scale / s
    if isinstance(loss, (list, tuple)):
        yield [l * s for l in loss]
    else:
        yield loss * s


def unscale(optimizer_or_trainer):
    """Divide the gradients by the loss scale now (before clipping them by hand)."""
    scaler = optimizer_or_trainer._amp_loss_scaler
    assert scaler is not None, 'Loss scaler is not initialized, did you forget to call amp.init_trainer()?'
    s = scaler.loss_scale
    for p in optimizer_or_trainer._params:
        if p.grad_req != 'null' and p._grad is not None:
            for g in p._grad.values():
                g._data.div_(s)
    optimizer_or_trainer._scale = optimizer_or_trainer._amp_original_scale
    # the next step must not divide by the scale again (the fused step does that division inside its reduce kernel); it
    # still checks for overflow and adapts the scale
    scaler._grads_unscaled = True


def convert_symbol(sym, input_dtypes=None, param_dtypes=None, target_dtype='float16', target_dtype_ops=None,
                   fp32_ops=None, conditional_fp32_ops=None, excluded_sym_names=None, data_names=None,
                   cast_params_offline=False, cast_optional_params=False):
    """Insert ``amp_cast`` / ``amp_multicast`` nodes according to the lists (``MXReducePrecisionSymbol``)."""
    from ..symbol import passes
    lists = _lists(target_dtype)
    td = to_torch_dtype(target_dtype)
    lp = target_dtype_ops if target_dtype_ops is not None else (lists.BF16_FUNCS if td == torch.bfloat16 else lists.FP16_FUNCS)
    f32 = fp32_ops if fp32_ops is not None else lists.FP32_FUNCS
    return passes.convert_precision(sym, 'bfloat16' if td == torch.bfloat16 else 'float16', _expand(lp), _expand(f32),
                                    _expand(lists.WIDEST_TYPE_CASTS), cast_optional_params, set(excluded_sym_names or ()))


def convert_model(sym, arg_params, aux_params, input_dtypes=None, target_dtype='float16', target_dtype_ops=None,
                  fp32_ops=None, conditional_fp32_ops=None, excluded_sym_names=None, cast_params_offline=False,
                  cast_optional_params=False):
    new_sym = convert_symbol(sym, input_dtypes, None, target_dtype, target_dtype_ops, fp32_ops, conditional_fp32_ops,
                             excluded_sym_names, None, cast_params_offline, cast_optional_params)
    return new_sym, arg_params, aux_params


def convert_hybrid_block(block, data_example=None, target_dtype='float16', target_dtype_ops=None, fp32_ops=None,
                         conditional_fp32_ops=None, excluded_sym_names=None, device=None, cast_params_offline=False,
                         cast_optional_params=False, ctx=None):
    """Return a ``SymbolBlock`` running the traced graph of ``block`` in mixed precision."""
    from ..gluon.block import SymbolBlock
    if block._cached_graph is None:
        if data_example is None:
            raise ValueError('run the block once or pass data_example so it can be traced')
        args = data_example if isinstance(data_example, (list, tuple)) else (data_example,)
        block(*args)
        block._trace(*args)
    inputs, sym = block._cached_graph
    new_sym = convert_symbol(sym, None, None, target_dtype, target_dtype_ops, fp32_ops, conditional_fp32_ops,
                             excluded_sym_names, None, cast_params_offline, cast_optional_params)
    params = {name: p for name, p in block.collect_params().items()}
    return SymbolBlock(new_sym, inputs, params)


def list_lp16_ops(target_dtype='float16'):
    l = _lists(target_dtype)
    return list(l.BF16_FUNCS if to_torch_dtype(target_dtype) == torch.bfloat16 else l.FP16_FUNCS)


def list_fp32_ops(target_dtype='float16'): return list(_lists(target_dtype).FP32_FUNCS)


def list_lp16_fp32_ops(target_dtype='float16'):
    l = _lists(target_dtype)
    return list(l.BF16_FP32_FUNCS if to_torch_dtype(target_dtype) == torch.bfloat16 else l.FP16_FP32_FUNCS)


def list_conditional_fp32_ops(target_dtype='float16'): return list(_lists(target_dtype).CONDITIONAL_FP32_FUNCS)
def list_widest_type_cast(target_dtype='float16'): return list(_lists(target_dtype).WIDEST_TYPE_CASTS)
def list_loss_output_functions(target_dtype='float16'): return list(_lists(target_dtype).LOSS_OUTPUT_FUNCTIONS)
def list_lp16_use_fp32_params(target_dtype='float16'): return ['BatchNorm', 'LayerNorm', 'GroupNorm', 'InstanceNorm']


def warn_if_model_exists():
    """Warn when ``amp.init()`` is called after a Block was already built: layers created earlier keep the operator
    functions they captured and are not patched."""
    import gc
    import warnings
    from ..gluon.block import Block
    for obj in gc.get_objects():
        try:
            if isinstance(obj, Block):
                warnings.warn('Block {} created in [{}] was not patched by AMP: create the network after amp.init()'.format(
                    type(obj).__name__, type(obj).__module__))
                return True
        except ReferenceError:
            continue
    return False

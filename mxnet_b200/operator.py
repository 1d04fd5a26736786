"""Custom operators written in Python (``python/mxnet/operator.py``: ``CustomOp`` / ``CustomOpProp`` /
``register``; native side ``src/operator/custom/custom.cc``).  A registered operator is invoked with
``mx.nd.Custom(*inputs, op_type='name', **kwargs)``; forward/backward run on the Python side and are
linked into the autograd tape as one node."""
import torch

from . import autograd
from .ndarray.ndarray import NDArray
from .ops import registry as _reg

__all__ = ['CustomOp', 'CustomOpProp', 'register', 'get_all_registered_operators', 'get_operator_arguments']

_custom_registry = {}


class CustomOp(object):
    def forward(self, is_train, req, in_data, out_data, aux):
        raise NotImplementedError

    def backward(self, req, out_grad, in_data, out_data, in_grad, aux):
        raise NotImplementedError

    def assign(self, dst, req, src):
        if req == 'null':
            return
        if req in ('write', 'inplace'):
            dst[:] = src
        elif req == 'add':
            dst[:] += src


class CustomOpProp(object):
    def __init__(self, need_top_grad=True):
        self.need_top_grad_ = need_top_grad

    def infer_shape(self, in_shape):
        return in_shape, (in_shape[0],) * len(self.list_outputs()), ()

    def infer_type(self, in_type):
        return in_type, [in_type[0]] * len(self.list_outputs()), [in_type[0]] * len(self.list_auxiliary_states())

    def list_outputs(self):
        return ['output']

    def list_arguments(self):
        return ['data']

    def list_auxiliary_states(self):
        return []

    def declare_backward_dependency(self, out_grad, in_data, out_data):
        deps = []
        if self.need_top_grad_:
            deps.extend(out_grad)
        deps.extend(in_data)
        deps.extend(out_data)
        return deps

    def create_operator(self, ctx, in_shapes, in_dtypes):
        return CustomOp()


def register(reg_name):
    def do_register(prop_cls):
        _custom_registry[reg_name] = prop_cls
        return prop_cls
    return do_register


def get_all_registered_operators():
    return _reg.list_ops()


def get_operator_arguments(op_name):
    op = _reg.get(op_name)
    from collections import namedtuple
    OperatorArguments = namedtuple('OperatorArguments', ['narg', 'names', 'types'])
    names = list(op.inputs) + list(op.defaults)
    return OperatorArguments(len(names), names, ['NDArray-or-Symbol'] * len(op.inputs) + ['any'] * len(op.defaults))


def _custom_fn(*tensors, op_type=None, **kwargs):
    prop = _custom_registry[op_type](**{k: str(v) for k, v in kwargs.items()})
    n_args = len(prop.list_arguments())
    in_t, aux_t = tensors[:n_args], tensors[n_args:]
    in_shapes = [tuple(t.shape) for t in in_t]
    _, out_shapes, _ = prop.infer_shape(list(in_shapes))
    _, out_types, _ = prop.infer_type([t.dtype for t in in_t])
    op = prop.create_operator(None, in_shapes, [t.dtype for t in in_t])
    from ._state import state
    is_train = state.training

    class _Fn(torch.autograd.Function):
        @staticmethod
        def forward(ctx, *ins):
            in_data = [NDArray._from_tensor(t.detach()) for t in ins]
            out_data = [NDArray._from_tensor(torch.zeros(s, dtype=d if isinstance(d, torch.dtype) else ins[0].dtype,
                                                         device=ins[0].device)) for s, d in zip(out_shapes, out_types)]
            aux = [NDArray._from_tensor(t) for t in aux_t]
            with autograd.pause():
                op.forward(is_train, ['write'] * len(out_data), in_data, out_data, aux)
            ctx.in_data, ctx.out_data, ctx.aux = in_data, out_data, aux
            outs = tuple(o._data for o in out_data)
            return outs if len(outs) > 1 else outs[0]

        @staticmethod
        def backward(ctx, *gouts):
            in_grad = [NDArray._from_tensor(torch.zeros_like(t._data)) for t in ctx.in_data]
            out_grad = [NDArray._from_tensor(g) for g in gouts]
            with autograd.pause():
                op.backward(['write'] * len(in_grad), out_grad, ctx.in_data, ctx.out_data, in_grad, ctx.aux)
            return tuple(g._data for g in in_grad)
    return _Fn.apply(*in_t)


_reg.register('Custom', inputs=('*data',), nout=lambda a: len(_custom_registry[a['op_type']](
    **{k: str(v) for k, v in a.items() if k != 'op_type'}).list_outputs()) if a.get('op_type') in _custom_registry else 1,
    defaults={'op_type': None})(_custom_fn)


def _install_frontends():
    from . import ndarray as nd, symbol as sym
    from .symbol.symbol import _op_frontend
    nd.Custom = _reg.make_frontend(_reg.get('Custom'), 'nd')
    sym.Custom = _op_frontend(_reg.get('Custom'))


_install_frontends()

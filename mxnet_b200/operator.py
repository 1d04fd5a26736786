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


# ---------------------------------------------------------------------------------------------------------
# legacy Python operators (PythonOp / NumpyOp / NDArrayOp of python/mxnet/operator.py): adapters onto CustomOp
# ---------------------------------------------------------------------------------------------------------
class PythonOp(object):
    """Base class of the deprecated Python operators: override ``forward``, ``backward``, ``infer_shape``,
    ``list_arguments``, ``list_outputs``; calling the object composes a Symbol node."""
    _ref_holder = []
    _counter = [0]

    def __init__(self, need_top_grad=True):
        self.info_ = None
        self.need_top_grad_ = need_top_grad

    def __call__(self, *args, **kwargs):
        return self.get_symbol(*args, **kwargs)

    def get_symbol(self, *args, **kwargs):
        raise NotImplementedError('Must override this')

    def forward(self, in_data, out_data):
        out_data[0][:] = in_data[0]

    def backward(self, out_grad, in_data, out_data, in_grad):
        in_grad[0][:] = 1.0

    def infer_shape(self, in_shape):
        return in_shape, [in_shape[0]]

    def list_outputs(self):
        return ['output']

    def list_arguments(self):
        return ['data']

    def need_top_grad(self):
        return self.need_top_grad_

    # -- shared by NumpyOp and NDArrayOp
    def _as_custom(self, convert, write_back):
        owner = self

        class _Op(CustomOp):
            def forward(self, is_train, req, in_data, out_data, aux):
                ins, outs = [convert(a) for a in in_data], [convert(a) for a in out_data]
                owner.forward(in_data=ins, out_data=outs)
                write_back(out_data, outs, req, self)

            def backward(self, req, out_grad, in_data, out_data, in_grad, aux):
                og, ins, outs, ig = ([convert(a) for a in group] for group in (out_grad, in_data, out_data, in_grad))
                owner.backward(out_grad=og, in_data=ins, out_data=outs, in_grad=ig)
                write_back(in_grad, ig, req, self)

        class _Prop(CustomOpProp):
            def __init__(self, **_kwargs):
                super().__init__(need_top_grad=owner.need_top_grad())

            def list_arguments(self):
                return owner.list_arguments()

            def list_outputs(self):
                return owner.list_outputs()

            def infer_shape(self, in_shape):
                ishape, oshape = owner.infer_shape([list(s) for s in in_shape])
                return ishape, oshape, []

            def create_operator(self, ctx, in_shapes, in_dtypes):
                return _Op()
        PythonOp._counter[0] += 1
        name = '_legacy_%s_%d' % (type(self).__name__.lower(), PythonOp._counter[0])
        register(name)(_Prop)
        PythonOp._ref_holder.append(self)
        return name

    def _compose(self, op_type, *args, **kwargs):
        from . import symbol as sym
        return sym.Custom(*args, op_type=op_type, **kwargs)


class NumpyOp(PythonOp):
    """Deprecated: forward / backward receive NumPy arrays (outputs and input gradients are written in place)."""

    def __init__(self, need_top_grad=True):
        super().__init__(need_top_grad)
        import warnings
        warnings.warn('NumpyOp has been deprecated. Please use CustomOp')

    def get_symbol(self, *args, **kwargs):
        def write_back(dst, arrays, req, op):
            for d, a, r in zip(dst, arrays, req):
                op.assign(d, r, NDArray._from_tensor(torch.from_numpy(a).to(d._data.device), d.context))
        op_type = self._as_custom(lambda a: a.asnumpy().copy(), write_back)
        return self._compose(op_type, *args, **kwargs)


class NDArrayOp(PythonOp):
    """Deprecated: forward / backward receive the framework's arrays and write into them."""

    def __init__(self, need_top_grad=True):
        super().__init__(need_top_grad)
        import warnings
        warnings.warn('NDArrayOp has been deprecated. Please use CustomOp')

    def get_symbol(self, *args, **kwargs):
        op_type = self._as_custom(lambda a: a, lambda dst, arrays, req, op: None)
        return self._compose(op_type, *args, **kwargs)

    def declare_backward_dependency(self, out_grad, in_data, out_data):
        deps = []
        if self.need_top_grad():
            deps.extend(out_grad)
        deps.extend(in_data)
        deps.extend(out_data)
        return deps


def get_all_registered_operators_grouped():
    """{operator name: [the name and all its aliases]} for every registered operator."""
    grouped = {}
    for name in _reg.list_ops():
        op = _reg.get(name)
        grouped.setdefault(op.name, [op.name])
        if name != op.name and name not in grouped[op.name]:
            grouped[op.name].append(name)
    return grouped


__all__ += ['PythonOp', 'NumpyOp', 'NDArrayOp', 'get_all_registered_operators_grouped']

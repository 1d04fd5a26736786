"""``mx.sym.Symbol``: static computation graphs, JSON-compatible with the reference.

Reference: nnvm graph JSON handled by ``src/c_api/c_api_symbolic.cc`` and
``src/nnvm/legacy_json_util.cc:46-200`` (upgrade of old files); Python class
``python/mxnet/symbol/symbol.py``.  File layout kept::

    {"nodes": [{"op": "null"|opname, "name": str, "attrs": {str: str}, "inputs": [[node, out, ver], ...]}, ...],
     "arg_nodes": [...], "node_row_ptr": [...], "heads": [[node, out, ver], ...],
     "attrs": {"mxnet_version": ["int", 20000]}}

Attribute values are strings in the file, formatted like dmlc parameters print them
(``"(3, 3)"``, ``"True"``, ``"None"``, bare enum names).  A Symbol is executed by walking the
nodes in topological order and calling the registered operator functions, so the same graph runs
imperatively, under autograd, or inside a CUDA-graph capture.
"""
from __future__ import annotations

import ast
import copy
import json

import numpy as _np
import torch

from .. import _state
from .. import env as _env
from ..attribute import AttrScope
from ..base import MXNetError, to_torch_dtype, dtype_name, to_numpy_dtype
from ..name import NameManager
from ..ops import registry as _reg

__all__ = ['Symbol', 'var', 'Variable', 'Group', 'load', 'load_json', 'fromjson', 'zeros', 'ones', 'full', 'arange']

_HIDDEN_KEYS = ('ctx_group', 'lr_mult', 'wd_mult', 'force_mirroring', 'mirror_stage', 'profiler_scope')


class _Node(object):
    __slots__ = ('op', 'name', 'attrs', 'inputs', 'nout', 'user_attrs')

    def __init__(self, op, name, attrs=None, inputs=None, nout=1, user_attrs=None):
        self.op = op                  # OpDef, or None for a variable
        self.name = name
        self.attrs = attrs or {}      # operator parameters as Python values
        self.inputs = inputs or []    # [(node, out_index)]
        self.nout = nout
        self.user_attrs = user_attrs or {}   # __shape__, __lr_mult__, ctx_group … (strings)


def _fmt_attr(v):
    """Python value → the string the reference writes for the same dmlc parameter value."""
    if isinstance(v, str):
        return v
    if isinstance(v, bool):
        return 'True' if v else 'False'
    if v is None:
        return 'None'
    if isinstance(v, torch.dtype):
        return dtype_name(v)
    if isinstance(v, type) and issubclass(v, _np.generic):
        return _np.dtype(v).name
    if isinstance(v, _np.dtype):
        return v.name
    if isinstance(v, (list, tuple)):
        inner = ', '.join(_fmt_attr(x) for x in v)
        if len(v) == 1 and isinstance(v, tuple):
            inner += ','
        return ('(%s)' if isinstance(v, tuple) else '[%s]') % inner
    if isinstance(v, float):
        return repr(v)
    if isinstance(v, _np.generic):
        return repr(v.item())
    if isinstance(v, slice):
        return 'slice(%s, %s, %s)' % (_fmt_attr(v.start), _fmt_attr(v.stop), _fmt_attr(v.step))
    if v is Ellipsis:
        return 'Ellipsis'
    if hasattr(v, 'device_type') and hasattr(v, 'device_id'):
        return '%s(%d)' % (v.device_type, v.device_id)
    if isinstance(v, torch.Tensor):
        return 'tensor(%s)' % json.dumps(v.tolist())
    return str(v)


def _eval_node(n):
    if isinstance(n, ast.Constant):
        return n.value
    if isinstance(n, ast.Tuple):
        return tuple(_eval_node(e) for e in n.elts)
    if isinstance(n, ast.List):
        return [_eval_node(e) for e in n.elts]
    if isinstance(n, ast.UnaryOp) and isinstance(n.op, (ast.USub, ast.UAdd)):
        v = _eval_node(n.operand)
        return -v if isinstance(n.op, ast.USub) else v
    if isinstance(n, ast.Name):
        if n.id in ('inf', 'Infinity'):
            return float('inf')
        if n.id == 'nan':
            return float('nan')
        if n.id == 'Ellipsis':
            return Ellipsis
        raise ValueError(n.id)
    if isinstance(n, ast.Call) and isinstance(n.func, ast.Name) and n.func.id == 'slice':
        return slice(*[_eval_node(a) for a in n.args])
    if isinstance(n, ast.Call) and isinstance(n.func, ast.Name) and n.func.id == 'tensor':
        return torch.as_tensor(_eval_node(n.args[0]))
    raise ValueError('unsupported literal')


def _parse_attr(s):
    """String from a JSON file → Python value (numbers, tuples, booleans, None; else the string)."""
    if not isinstance(s, str):
        return s
    try:
        return _eval_node(ast.parse(s.strip(), mode='eval').body)
    except (ValueError, SyntaxError, TypeError):
        return s


# Operators the backward-mirroring pass never recomputes: the contraction-heavy ones (recomputing them costs what the pass
# is meant to save), the ones with running state, and the sources of randomness.
_NO_MIRROR = frozenset(['Convolution', 'Deconvolution', 'FullyConnected', 'Concat', 'SoftmaxOutput', 'BatchNorm', 'SyncBatchNorm',
                        '_contrib_SyncBatchNorm', 'Dropout', 'RNN', 'Custom', 'dot', 'batch_dot', 'Embedding', '_FusedOp',
                        '_contrib_fused_self_attention', '_contrib_interleaved_matmul_selfatt_qk',
                        '_contrib_interleaved_matmul_selfatt_valatt', '_contrib_interleaved_matmul_encdec_qk',
                        '_contrib_interleaved_matmul_encdec_valatt', '_npi_matmul', '_npi_dot', '_npi_tensordot', '_npi_einsum',
                        '_foreach', '_while_loop', '_cond', 'CTCLoss', 'Correlation', '_contrib_DeformableConvolution'])


def _forced_mirror(node):
    v = node.user_attrs.get('force_mirroring', node.user_attrs.get('__force_mirroring__')) if node.op is not None else None
    return v is not None and str(v).lower() in ('1', 'true')


def _mirrorable(node, everything):
    """The reference's mirror predicate: with the switch on, every operator outside the exclusion list; without it, the
    operators marked ``force_mirroring``.  Operators with auxiliary or in-place inputs and random ones never qualify."""
    op = node.op
    if op.aux or op.mutate or op.name in _NO_MIRROR:
        return False
    low = op.name.lower()
    if 'random' in low or 'sample' in low or 'shuffle' in low or 'dropout' in low:
        return False
    return everything or _forced_mirror(node)


def _apply_node(node, ins):
    hook = _state.amp_hook
    if hook is not None and not _state.state.opt_constraints & 1:
        ins = hook(node.op.name, ins)
    res = node.op.fn(*ins, **node.attrs)
    return tuple(res) if isinstance(res, (tuple, list)) else (res,)


def _topo(outputs):
    order, seen = [], set()
    stack = [(n, False) for n, _ in reversed(outputs)]
    while stack:
        node, done = stack.pop()
        if done:
            order.append(node)
            continue
        if id(node) in seen:
            continue
        seen.add(id(node))
        stack.append((node, True))
        for inp, _ in reversed(node.inputs):
            if id(inp) not in seen:
                stack.append((inp, False))
    return order


class Symbol(object):
    """Symbolic graph handle: a list of output entries over shared nodes."""
    __slots__ = ('_outputs', '_fused')
    __array_priority__ = 1000.0

    def __init__(self, outputs):
        self._outputs = list(outputs)
        self._fused = None            # this graph after pointwise fusion (False: nothing to fuse), built on first GPU run

    # ------------------------------------------------------------------ introspection
    @property
    def name(self):
        if len(self._outputs) != 1:
            return None
        return self._outputs[0][0].name

    def _entry_name(self, node, idx):
        if node.op is None:
            return node.name
        if node.nout == 1:
            return node.name + '_output'
        return '%s_output%d' % (node.name, idx)

    def list_outputs(self):
        return [self._entry_name(n, i) for n, i in self._outputs]

    def _aux_nodes(self):
        aux = set()
        for node in _topo(self._outputs):
            if node.op is not None and node.op.aux:
                for nm, (inp, _) in zip(node.op.inputs, node.inputs):
                    if nm in node.op.aux and inp.op is None:
                        aux.add(id(inp))
        return aux

    def list_arguments(self):
        aux = self._aux_nodes()
        return [n.name for n in _topo(self._outputs) if n.op is None and id(n) not in aux]

    def list_auxiliary_states(self):
        aux = self._aux_nodes()
        return [n.name for n in _topo(self._outputs) if n.op is None and id(n) in aux]

    def list_inputs(self):
        return [n.name for n in _topo(self._outputs) if n.op is None]

    def get_internals(self):
        outs = []
        for n in _topo(self._outputs):
            for i in range(n.nout):
                outs.append((n, i))
        return Symbol(outs)

    def get_children(self):
        entries, seen = [], set()
        for node, _ in self._outputs:
            if id(node) not in seen:            # the heads of one multi-output operator share their inputs
                seen.add(id(node))
                entries.extend(node.inputs)
        return Symbol(entries) if entries else None

    def get_inputs(self):
        return Symbol([(n, 0) for n in _topo(self._outputs) if n.op is None])

    def __len__(self):
        return len(self._outputs)

    def __iter__(self):
        return (Symbol([o]) for o in self._outputs)

    def __getitem__(self, index):
        if isinstance(index, str):
            names = self.list_outputs()
            hits = [i for i, n in enumerate(names) if n == index]
            if not hits:
                raise ValueError('There is no output named "%s"' % index)
            if len(hits) > 1:
                raise ValueError('There are multiple outputs with name "%s"' % index)
            index = hits[0]
        if isinstance(index, slice):
            return Symbol(self._outputs[index])
        if len(self._outputs) == 1 and self._outputs[0][0].nout > 1 and self._outputs[0][0].op is not None:
            node = self._outputs[0][0]
            if index >= node.nout:
                raise IndexError
            return Symbol([(node, index)])
        return Symbol([self._outputs[index]])

    def attr(self, key):
        node = self._outputs[0][0]
        if key in node.user_attrs:
            return node.user_attrs[key]
        if key in node.attrs:
            return _fmt_attr(node.attrs[key])
        return None

    def list_attr(self, recursive=False):
        if recursive:
            raise DeprecationWarning('Symbol.list_attr with recursive=True has been deprecated; use attr_dict')
        node = self._outputs[0][0]
        d = {k: _fmt_attr(v) for k, v in node.attrs.items()}
        d.update(node.user_attrs)
        return d

    def attr_dict(self):
        out = {}
        for n in _topo(self._outputs):
            d = {k: _fmt_attr(v) for k, v in n.attrs.items()}
            d.update(n.user_attrs)
            if d:
                out[n.name] = d
        return out

    def _set_attr(self, **kwargs):
        node = self._outputs[0][0]
        for k, v in kwargs.items():
            if not isinstance(v, str):
                raise ValueError('Set Attr only accepts string values')
            if k == 'name':
                node.name = v
            else:
                node.user_attrs[k] = v

    def __copy__(self):
        return self.__deepcopy__(None)

    def __deepcopy__(self, memo):
        return load_json(self.tojson())

    def __repr__(self):
        if self.name is None:
            return '<Symbol group [%s]>' % ', '.join(n.name for n, _ in self._outputs)
        return '<Symbol %s>' % self.name

    # ------------------------------------------------------------------ composition
    def __call__(self, *args, **kwargs):
        s = load_json(self.tojson())
        s._compose(*args, **kwargs)
        return s

    def _compose(self, *args, **kwargs):
        kwargs.pop('name', None)
        self._fused = None
        if args and kwargs:
            raise TypeError('compose only accept input Symbols either as positional or keyword arguments, not both')
        variables = [n for n in _topo(self._outputs) if n.op is None]
        mapping = {}
        if args:
            for v, a in zip(variables, args):
                mapping[id(v)] = a._outputs[0]
        for k, a in kwargs.items():
            for v in variables:
                if v.name == k:
                    mapping[id(v)] = a._outputs[0]
        for n in _topo(self._outputs):
            n.inputs = [mapping.get(id(i), (i, k)) if i.op is None else (i, k) for i, k in n.inputs]
        self._outputs = [mapping.get(id(n), (n, k)) if n.op is None else (n, k) for n, k in self._outputs]

    def _binop(self, other, tt, ts, rts=None, reverse=False):
        if isinstance(other, Symbol):
            a, b = (other, self) if reverse else (self, other)
            return _make_op_symbol(_reg.get(tt), [a, b], {}, None)
        if isinstance(other, (int, float, _np.generic)):
            return _make_op_symbol(_reg.get(rts if reverse and rts else ts), [self], {'scalar': float(other)
                                   if not isinstance(other, int) else other}, None)
        return NotImplemented

    def __add__(self, o): return self._binop(o, 'broadcast_add' if _state.state.np_array else 'elemwise_add', '_plus_scalar')
    __radd__ = __add__
    def __sub__(self, o): return self._binop(o, 'broadcast_sub' if _state.state.np_array else 'elemwise_sub', '_minus_scalar')
    def __rsub__(self, o): return self._binop(o, 'elemwise_sub', '_minus_scalar', '_rminus_scalar', True)
    def __mul__(self, o): return self._binop(o, 'broadcast_mul' if _state.state.np_array else 'elemwise_mul', '_mul_scalar')
    __rmul__ = __mul__
    def __truediv__(self, o): return self._binop(o, 'broadcast_div' if _state.state.np_array else 'elemwise_div', '_div_scalar')
    def __rtruediv__(self, o): return self._binop(o, 'elemwise_div', '_div_scalar', '_rdiv_scalar', True)
    __div__, __rdiv__ = __truediv__, __rtruediv__
    def __mod__(self, o): return self._binop(o, 'broadcast_mod', '_mod_scalar')
    def __rmod__(self, o): return self._binop(o, 'broadcast_mod', '_mod_scalar', '_rmod_scalar', True)
    def __pow__(self, o): return self._binop(o, 'broadcast_power', '_power_scalar')
    def __rpow__(self, o): return self._binop(o, 'broadcast_power', '_power_scalar', '_rpower_scalar', True)
    def __neg__(self): return self.__mul__(-1.0)

    def __abs__(self):
        return _op_frontend(_reg.get('abs'))(self)
    def __eq__(self, o): return self._binop(o, 'broadcast_equal', '_equal_scalar')
    def __ne__(self, o): return self._binop(o, 'broadcast_not_equal', '_not_equal_scalar')
    def __gt__(self, o): return self._binop(o, 'broadcast_greater', '_greater_scalar')
    def __ge__(self, o): return self._binop(o, 'broadcast_greater_equal', '_greater_equal_scalar')
    def __lt__(self, o): return self._binop(o, 'broadcast_lesser', '_lesser_scalar')
    def __le__(self, o): return self._binop(o, 'broadcast_lesser_equal', '_lesser_equal_scalar')
    __hash__ = object.__hash__

    def __getattr__(self, name):
        # fluent operator methods: sym.reshape(...), sym.sum(...), …
        if name.startswith('_'):
            raise AttributeError(name)
        if _reg.has(name):
            op = _reg.get(name)

            def method(*args, **kwargs):
                return _op_frontend(op)(self, *args, **kwargs)
            return method
        if name == 'split_v2':
            def split_v2(indices_or_sections, axis=0, squeeze_axis=False):
                from .. import symbol as _sym_mod
                return _sym_mod.split_v2(self, indices_or_sections, axis, squeeze_axis)
            return split_v2
        raise AttributeError(name)

    # ------------------------------------------------------------------ serialisation
    def tojson(self, remove_amp_cast=True):
        nodes = _topo(self._outputs)
        index = {id(n): i for i, n in enumerate(nodes)}
        jnodes, arg_nodes, row_ptr = [], [], [0]
        for i, n in enumerate(nodes):
            entry = {'op': 'null' if n.op is None else n.op.name, 'name': n.name}
            attrs = {k: _fmt_attr(v) for k, v in n.attrs.items()
                     if not (n.op is not None and k in n.op.defaults and n.op.defaults[k] == v and v is None)
                     and not isinstance(v, Symbol)}
            subgraphs = [v for k, v in sorted(n.attrs.items()) if isinstance(v, Symbol)]      # control-flow bodies
            if subgraphs:
                entry['subgraphs'] = [json.loads(g.tojson(remove_amp_cast)) for g in subgraphs]
            attrs.update(n.user_attrs)
            if attrs:
                entry['attrs'] = attrs
            entry['inputs'] = [[index[id(inp)], k, 0] for inp, k in n.inputs]
            jnodes.append(entry)
            if n.op is None:
                arg_nodes.append(i)
            row_ptr.append(row_ptr[-1] + n.nout)
        heads = [[index[id(n)], k, 0] for n, k in self._outputs]
        return json.dumps({'nodes': jnodes, 'arg_nodes': arg_nodes, 'node_row_ptr': row_ptr, 'heads': heads,
                           'attrs': {'mxnet_version': ['int', 20000]}}, indent=2)

    def save(self, fname, remove_amp_cast=True):
        with open(fname, 'w') as f:
            f.write(self.tojson(remove_amp_cast))

    # ------------------------------------------------------------------ execution / inference
    def _place(self, default_ctx, group2ctx):
        """Device of every node for model-parallel execution (the reference's PlaceDevice pass,
        src/executor/graph_executor.cc AssignContext): a node whose ``ctx_group`` attribute names a key of ``group2ctx``
        runs on that context; a node without one takes the device of its first placed input, else of its first placed
        consumer, else the default.  Returns {id(node): Context}; values cross contexts with a copy at the consumer."""
        devices = {}
        for g, c in (group2ctx or {}).items():
            devices[g] = c[0] if isinstance(c, (list, tuple)) else c
        order = _topo(self._outputs)
        placed = {}
        for n in order:
            g = n.user_attrs.get('ctx_group', n.user_attrs.get('__ctx_group__'))
            if g is not None and g in devices:
                placed[id(n)] = devices[g]
        for n in order:                                   # forward: follow the first placed input
            if id(n) not in placed:
                for i, _ in n.inputs:
                    if id(i) in placed:
                        placed[id(n)] = placed[id(i)]
                        break
        for n in reversed(order):                         # backward: follow a placed consumer
            if id(n) in placed:
                for i, _ in n.inputs:
                    placed.setdefault(id(i), placed[id(n)])
        for n in order:
            placed.setdefault(id(n), default_ctx)
        return placed

    def _run(self, feed, training=None, placement=None, stats=None):
        """Evaluate the graph.  ``feed``: {variable name: tensor}.  Returns list of tensors.  On a GPU the graph runs
        with its elementwise groups fused into generated kernels (``MXNET_USE_FUSION``).  With ``placement`` (from
        :meth:`_place`) every operator runs on its assigned device: inputs that live elsewhere are copied there first (the
        ``_CrossDeviceCopy`` nodes of the reference; the copies are differentiable, so gradients flow back across devices),
        and ``stats['copies']`` counts them."""
        graph = self
        if placement is not None:
            return self._run_placed(feed, placement, stats)
        if self._fused is not False and _env.get('MXNET_USE_FUSION') and any(
                isinstance(t, torch.Tensor) and t.is_cuda for t in feed.values()):
            if self._fused is None:
                from .fusion import fuse_pointwise
                fused = fuse_pointwise(self)
                self._fused = fused if fused is not self else False
            graph = self._fused or self
        if torch.is_grad_enabled() and (_env.get('MXNET_MEMORY_OPT') or _env.get('MXNET_BACKWARD_DO_MIRROR') or
                                        any(_forced_mirror(n) for n in _topo(graph._outputs))):
            return graph._run_mirrored(feed, stats)
        values = {}
        for node in _topo(graph._outputs):
            if node.op is None:
                if node.name not in feed:
                    raise MXNetError('missing input %s' % node.name)
                values[id(node)] = (feed[node.name],)
                continue
            ins = [values[id(i)][k] for i, k in node.inputs]
            values[id(node)] = _apply_node(node, ins)
        return [values[id(n)][k] for n, k in graph._outputs]

    def _run_mirrored(self, feed, stats=None):
        """Evaluate the graph with backward mirroring (reference: src/nnvm/gradient.cc, the gradient pass with a
        ``mirror_fun``; switches ``MXNET_BACKWARD_DO_MIRROR`` / ``MXNET_MEMORY_OPT`` and the node attribute
        ``force_mirroring``).  Maximal runs of consecutive mirrorable operators (cheap, stateless, deterministic: everything
        except convolutions, dense products, normalisation with running statistics, random and in-place operators) keep
        only their inputs: their intermediate results are dropped after the forward pass and recomputed when the backward
        pass reaches the run.  ``stats['mirrored_nodes']`` / ``stats['mirror_segments']`` report what was mirrored."""
        from torch.utils.checkpoint import checkpoint
        order = _topo(self._outputs)
        everything = bool(_env.get('MXNET_MEMORY_OPT') or _env.get('MXNET_BACKWARD_DO_MIRROR'))
        needed_later = {}                               # id(node) -> position of its last consumer (graph outputs: infinity)
        for pos, node in enumerate(order):
            for inp, _ in node.inputs:
                needed_later[id(inp)] = pos
        for n, _ in self._outputs:
            needed_later[id(n)] = len(order)
        values = {}
        mirrored = segments = 0
        pos = 0
        while pos < len(order):
            node = order[pos]
            if node.op is None:
                if node.name not in feed:
                    raise MXNetError('missing input %s' % node.name)
                values[id(node)] = (feed[node.name],)
                pos += 1
                continue
            end = pos
            while end < len(order) and order[end].op is not None and _mirrorable(order[end], everything):
                end += 1
            if end - pos < 2:                           # a run of one operator has nothing to drop
                ins = [values[id(i)][k] for i, k in node.inputs]
                values[id(node)] = _apply_node(node, ins)
                pos += 1
                continue
            seg = order[pos:end]
            inside = {id(n) for n in seg}
            ext, ext_index = [], {}
            for n in seg:
                for inp, k in n.inputs:
                    if id(inp) not in inside and (id(inp), k) not in ext_index:
                        ext_index[(id(inp), k)] = len(ext)
                        ext.append(values[id(inp)][k])
            exported = [n for n in seg if needed_later.get(id(n), -1) >= end]

            counts = []

            def run_segment(*tensors, seg=seg, inside=inside, ext_index=ext_index, exported=exported, counts=counts):
                local = {}
                for n in seg:
                    ins = [local[id(i)][k] if id(i) in inside else tensors[ext_index[(id(i), k)]] for i, k in n.inputs]
                    local[id(n)] = _apply_node(n, ins)
                counts[:] = [len(local[id(n)]) for n in exported]
                return tuple(t for n in exported for t in local[id(n)])
            if any(isinstance(t, torch.Tensor) and t.requires_grad for t in ext):
                flat = checkpoint(run_segment, *ext, use_reentrant=False, preserve_rng_state=False)
                mirrored += len(seg)
                segments += 1
            else:
                flat = run_segment(*ext)
            at = 0
            for n, cnt in zip(exported, counts):
                values[id(n)] = tuple(flat[at:at + cnt])
                at += cnt
            pos = end
        if stats is not None:
            stats['mirrored_nodes'] = mirrored
            stats['mirror_segments'] = segments
        return [values[id(n)][k] for n, k in self._outputs]

    def _run_placed(self, feed, placement, stats=None):
        values = {}
        where = {}
        copies = 0
        for node in _topo(self._outputs):
            if node.op is None:
                if node.name not in feed:
                    raise MXNetError('missing input %s' % node.name)
                values[id(node)] = (feed[node.name],)
                where[id(node)] = placement[id(node)]
                continue
            ctx = placement[id(node)]
            dev = ctx.torch_device
            where[id(node)] = ctx
            ins = []
            for i, k in node.inputs:
                t = values[id(i)][k]
                if isinstance(t, torch.Tensor) and where[id(i)] != ctx:
                    copies += 1                            # a _CrossDeviceCopy of the reference
                    if t.device != dev:
                        t = t.to(dev)
                ins.append(t)
            hook = _state.amp_hook
            if hook is not None and not _state.state.opt_constraints & 1:
                ins = hook(node.op.name, ins)
            if dev.type == 'cuda':
                with torch.cuda.device(dev):
                    res = node.op.fn(*ins, **node.attrs)
            else:
                res = node.op.fn(*ins, **node.attrs)
            values[id(node)] = tuple(res) if isinstance(res, (tuple, list)) else (res,)
        if stats is not None:
            stats['copies'] = copies
        return [values[id(n)][k] for n, k in self._outputs]

    def _infer(self, shapes, dtypes, partial=False):
        feed, unknown = {}, []
        variables = [n for n in _topo(self._outputs) if n.op is None]
        for v in variables:
            shp = shapes.get(v.name)
            if shp is None and '__shape__' in v.user_attrs:
                shp = _parse_attr(v.user_attrs['__shape__'])
            dt = dtypes.get(v.name)
            if dt is None and '__dtype__' in v.user_attrs:
                dt = _parse_attr(v.user_attrs['__dtype__'])
                if isinstance(dt, int):
                    from ..base import flag_to_torch
                    dt = flag_to_torch(dt)
            if shp is None or any(s in (0, -1) for s in shp) and not _state.state.np_shape and 0 in shp:
                unknown.append(v)
            feed[v.name] = (tuple(shp) if shp is not None else None, to_torch_dtype(dt) if dt is not None else None)
        return _shape_infer_graph(self, feed, partial)

    def infer_shape(self, *args, **kwargs):
        res = self._infer_shape_impl(False, *args, **kwargs)
        return res

    def infer_shape_partial(self, *args, **kwargs):
        return self._infer_shape_impl(True, *args, **kwargs)

    def _infer_shape_impl(self, partial, *args, **kwargs):
        shapes = dict(kwargs)
        if args:
            for name, s in zip(self.list_arguments(), args):
                if s is not None:
                    shapes[name] = s
        info = _shape_infer_graph(self, {k: (tuple(v), None) for k, v in shapes.items()}, partial)
        if info is None:
            return None, None, None
        arg_names, aux_names = self.list_arguments(), self.list_auxiliary_states()
        return ([info['vars'].get(n) for n in arg_names], info['outs'], [info['vars'].get(n) for n in aux_names])

    def infer_type(self, *args, **kwargs):
        dtypes = dict(kwargs)
        if args:
            for name, t in zip(self.list_arguments(), args):
                if t is not None:
                    dtypes[name] = t
        arg_names, aux_names = self.list_arguments(), self.list_auxiliary_states()
        default = None
        for v in dtypes.values():
            default = v
            break
        default = default or _np.float32
        arg_t = [_np.dtype(dtypes.get(n, default)).type for n in arg_names]
        out_t = [_np.dtype(default).type for _ in self._outputs]
        aux_t = [_np.dtype(default).type for _ in aux_names]
        return arg_t, out_t, aux_t

    def infer_type_partial(self, *args, **kwargs):
        return self.infer_type(*args, **kwargs)

    def eval(self, ctx=None, **kwargs):
        from ..ndarray.ndarray import NDArray
        feed = {k: v._data for k, v in kwargs.items()}
        outs = self._run(feed)
        cls = type(next(iter(kwargs.values()))) if kwargs else NDArray
        return [cls._from_tensor(o) for o in outs]

    def _bind(self, ctx, args, args_grad=None, grad_req='write', aux_states=None, group2ctx=None, shared_exec=None):
        from ..executor import Executor
        return Executor(self, ctx, args, args_grad, grad_req, aux_states, group2ctx=group2ctx)

    bind = _bind

    def simple_bind(self, ctx, grad_req='write', type_dict=None, stype_dict=None, group2ctx=None,
                    shared_arg_names=None, shared_exec=None, shared_buffer=None, **kwargs):
        from .. import ndarray as nd
        arg_shapes, _, aux_shapes = self.infer_shape(**kwargs)
        if arg_shapes is None or any(s is None for s in arg_shapes):
            raise MXNetError('cannot infer shapes for simple_bind')
        type_dict = type_dict or {}
        # arguments and their gradients live on the context of their group (model parallelism), else on `ctx`
        where = {}
        if group2ctx:
            placed = self._place(ctx, group2ctx)
            for n in _topo(self._outputs):
                if n.op is None:
                    where[n.name] = placed[id(n)]
        args = {n: nd.zeros(s, ctx=where.get(n, ctx), dtype=type_dict.get(n, 'float32'))
                for n, s in zip(self.list_arguments(), arg_shapes)}
        grads = {n: nd.zeros(s, ctx=where.get(n, ctx), dtype=type_dict.get(n, 'float32'))
                 for n, s in zip(self.list_arguments(), arg_shapes)} if grad_req != 'null' else None
        aux = {n: nd.zeros(s, ctx=where.get(n, ctx)) for n, s in zip(self.list_auxiliary_states(), aux_shapes)}
        return self._bind(ctx, args, grads, grad_req, aux, group2ctx=group2ctx)

    _simple_bind = simple_bind

    def optimize_for(self, backend, args=None, aux=None, ctx=None, shape_dict=None, type_dict=None, stype_dict=None,
                     skip_infer=False, **kwargs):
        """Graph partitioning hook (``MXOptimizeForBackend``).  Backends registered with
        :func:`mxnet_b200.symbol.passes.register_backend` rewrite the graph; unknown names raise."""
        from . import passes
        return passes.optimize_for(self, backend, args, aux, **kwargs)

    def as_np_ndarray(self):
        return self

    def as_nd_ndarray(self):
        return self

    def remove_amp_cast(self):
        from . import passes
        return passes.remove_amp_cast(self)

    def get_backend_symbol(self, backend):
        return self.optimize_for(backend)

    def gradient(self, wrt):
        raise MXNetError('Symbol.gradient is not supported; bind the symbol and call backward')

    def debug_str(self):
        lines = []
        for n in _topo(self._outputs):
            if n.op is None:
                lines.append('Variable:%s' % n.name)
            else:
                lines.append('--------------------\nOp:%s, Name=%s\nInputs:' % (n.op.name, n.name))
                for j, (i, k) in enumerate(n.inputs):
                    lines.append('\targ[%d]=%s(%d)' % (j, i.name, k))
                if n.attrs:
                    lines.append('Attrs:')
                    for k, v in n.attrs.items():
                        lines.append('\t%s=%s' % (k, _fmt_attr(v)))
        return '\n'.join(lines)


# ----------------------------------------------------------------------------------------------
# shape/type inference by abstract evaluation on the 'meta' device
# ----------------------------------------------------------------------------------------------
_PARAM_SHAPE_RULES = {}


def _rule(opname):
    def deco(fn):
        _PARAM_SHAPE_RULES[opname] = fn
        return fn
    return deco


def _same_shape_rule(node, in_shapes):
    """Operators whose operands all have one shape (``elemwise_*``, ``add_n``): an unknown operand takes the known shape."""
    known = [s for s in in_shapes if s is not None]
    if not known:
        return {}
    return {pos: known[0] for pos, s in enumerate(in_shapes) if s is None}


for _n in ('elemwise_add', 'elemwise_sub', 'elemwise_mul', 'elemwise_div', 'add_n'):
    if _reg.has(_n):
        _PARAM_SHAPE_RULES[_reg.get(_n).name] = _same_shape_rule



@_rule('FullyConnected')
def _fc_rule(node, ins):
    data = ins[0]
    if data is None:
        return {}
    nh = node.attrs.get('num_hidden')
    flatten = node.attrs.get('flatten', True)
    k = int(_np.prod(data[1:])) if flatten else data[-1]
    return {1: (nh, k), 2: (nh,)}


@_rule('Convolution')
def _conv_rule(node, ins):
    data = ins[0]
    if data is None:
        return {}
    layout = node.attrs.get('layout')
    kernel = tuple(node.attrs.get('kernel'))
    nf, ng = node.attrs.get('num_filter'), node.attrs.get('num_group', 1)
    if layout in ('NWC', 'NHWC', 'NDHWC'):
        return {1: (nf,) + kernel + (data[-1] // ng,), 2: (nf,)}
    return {1: (nf, data[1] // ng) + kernel, 2: (nf,)}


@_rule('Deconvolution')
def _deconv_rule(node, ins):
    data = ins[0]
    if data is None:
        return {}
    kernel = tuple(node.attrs.get('kernel'))
    nf, ng = node.attrs.get('num_filter'), node.attrs.get('num_group', 1)
    return {1: (data[1], nf // ng) + kernel, 2: (nf,)}


def _channel_rule(node, ins):
    data = ins[0]
    if data is None:
        return {}
    axis = node.attrs.get('axis', 1 if node.op.name != 'LayerNorm' else -1)
    c = data[axis]
    return {i: (c,) for i in range(1, len(node.op.inputs))}


for _n in ('BatchNorm', 'LayerNorm', 'InstanceNorm', 'SyncBatchNorm'):
    _PARAM_SHAPE_RULES[_n] = _channel_rule


@_rule('GroupNorm')
def _gn_rule(node, ins):
    return {} if ins[0] is None else {1: (ins[0][1],), 2: (ins[0][1],)}


@_rule('Embedding')
def _emb_rule(node, ins):
    return {1: (node.attrs.get('input_dim'), node.attrs.get('output_dim'))}


@_rule('LeakyReLU')
def _prelu_rule(node, ins):
    if node.attrs.get('act_type') == 'prelu' and ins[0] is not None:
        return {1: (ins[0][1],) if len(ins[0]) > 1 else (1,)}
    return {}


@_rule('RNN')
def _rnn_rule(node, ins):
    data = ins[0]
    if data is None:
        return {}
    from ..ops.nn import rnn_param_size
    a = node.attrs
    d = 2 if a.get('bidirectional') else 1
    L, H = a.get('num_layers', 1), a.get('state_size')
    P = a.get('projection_size') or H
    out = {1: (rnn_param_size(a.get('mode', 'lstm'), L, data[2], H, a.get('bidirectional', False), a.get('projection_size')),),
           2: (L * d, data[1], P)}
    if a.get('mode', 'lstm') == 'lstm':
        out[3] = (L * d, data[1], H)
    return out


for _n in ('SoftmaxOutput', 'LinearRegressionOutput', 'LogisticRegressionOutput', 'MAERegressionOutput', 'SVMOutput'):
    def _label_rule(node, ins, _name=_n):
        if ins[0] is None:
            return {}
        if _name == 'SoftmaxOutput':
            if node.attrs.get('multi_output'):
                return {1: (ins[0][0],) + tuple(ins[0][2:])}
            return {1: (ins[0][0],)}
        if _name == 'SVMOutput':
            return {1: (ins[0][0],)}
        return {1: tuple(ins[0])}
    _PARAM_SHAPE_RULES[_n] = _label_rule


def _shape_infer_graph(sym, feed, partial=False):
    """Forward abstract evaluation; parameter shapes of NN layers are back-filled from the data
    shape with per-operator rules (the job of ``FInferShape`` in the reference)."""
    nodes = _topo(sym._outputs)
    var_shapes, var_dtypes = {}, {}
    for n in nodes:
        if n.op is None:
            shp, dt = feed.get(n.name, (None, None))
            if shp is None and '__shape__' in n.user_attrs:
                shp = _parse_attr(n.user_attrs['__shape__'])
                if shp is not None and (len(shp) == 0 or any(s <= 0 for s in shp)) and not _state.state.np_shape:
                    shp = None
            if dt is None and '__dtype__' in n.user_attrs:
                d = _parse_attr(n.user_attrs['__dtype__'])
                if isinstance(d, int):
                    from ..base import flag_to_torch
                    dt = flag_to_torch(d) if d >= 0 else None
                elif d is not None:
                    dt = to_torch_dtype(d)
            var_shapes[id(n)] = tuple(shp) if shp is not None else None
            var_dtypes[id(n)] = dt
    values = {}
    ok = True
    deferred = []
    with torch.no_grad():
        for n in nodes:
            if n.op is None:
                s = var_shapes[id(n)]
                values[id(n)] = (torch.empty(s, dtype=var_dtypes[id(n)] or torch.float32, device='meta'),) if s is not None else (None,)
                continue
            in_shapes = [tuple(values[id(i)][k].shape) if values[id(i)][k] is not None else None for i, k in n.inputs]
            rule = _PARAM_SHAPE_RULES.get(n.op.name)
            if rule is not None and any(s is None for s in in_shapes):
                filled = rule(n, in_shapes)
                for pos, shp in filled.items():
                    if pos < len(n.inputs) and in_shapes[pos] is None:
                        inp, k = n.inputs[pos]
                        if inp.op is None:
                            var_shapes[id(inp)] = tuple(shp)
                            dt = var_dtypes[id(inp)] or (values[id(n.inputs[0][0])][n.inputs[0][1]].dtype
                                                          if values[id(n.inputs[0][0])][n.inputs[0][1]] is not None else torch.float32)
                            if n.op.name in ('Embedding',) or (n.op.name == 'SoftmaxOutput' and pos == 1):
                                dt = var_dtypes[id(inp)] or torch.float32
                            values[id(inp)] = (torch.empty(tuple(shp), dtype=dt, device='meta'),)
                        elif inp.op.name in ('_layout_transpose', 'transpose') and inp.attrs.get('axes') and \
                                inp.inputs[0][0].op is None and values[id(inp.inputs[0][0])][0] is None:
                            # a parameter that reaches the layer through a transpose (the layout pass puts one on every
                            # convolution weight): the variable has the inverse permutation of the shape the layer wants
                            src = inp.inputs[0][0]
                            axes = tuple(inp.attrs['axes'])
                            vshape = [0] * len(axes)
                            for pos_out, ax in enumerate(axes):
                                vshape[ax] = shp[pos_out]
                            var_shapes[id(src)] = tuple(vshape)
                            first = values[id(n.inputs[0][0])][n.inputs[0][1]]
                            dt = var_dtypes[id(src)] or (first.dtype if first is not None else torch.float32)
                            values[id(src)] = (torch.empty(tuple(vshape), dtype=dt, device='meta'),)
                            values[id(inp)] = (values[id(src)][0].permute(axes),)
            ins = [values[id(i)][k] for i, k in n.inputs]
            if any(v is None for v in ins):
                if n.op.name in ('_layout_transpose', 'transpose') and n.inputs[0][0].op is None:
                    deferred.append(n)         # its consumer's rule may still give the variable a shape
                else:
                    ok = False
                values[id(n)] = (None,) * n.nout
                continue
            try:
                prev = _state.state.training
                res = n.op.fn(*ins, **n.attrs)
            except Exception:  # pylint: disable=broad-except
                try:   # operators that need real data (python-side loops): evaluate on zeros
                    cpu_ins = [torch.zeros(v.shape, dtype=v.dtype) for v in ins]
                    res = n.op.fn(*cpu_ins, **n.attrs)
                    res = tuple(torch.empty(r.shape, dtype=r.dtype, device='meta') for r in
                                (res if isinstance(res, (tuple, list)) else (res,)))
                except Exception as e:  # pylint: disable=broad-except
                    if partial:
                        ok = False
                        values[id(n)] = (None,) * n.nout
                        continue
                    raise MXNetError('Error in operator %s: %s' % (n.name, e))
            values[id(n)] = tuple(res) if isinstance(res, (tuple, list)) else (res,)
    if any(values[id(n)][0] is None for n in deferred):
        ok = False
    if not ok and not partial:
        return None
    vars_out = {n.name: var_shapes[id(n)] for n in nodes if n.op is None}
    outs = [tuple(values[id(n)][k].shape) if values[id(n)][k] is not None else None for n, k in sym._outputs]
    dts = {n.name: (values[id(n)][0].dtype if values[id(n)][0] is not None else None) for n in nodes if n.op is None}
    return {'vars': vars_out, 'outs': outs, 'dtypes': dts,
            'out_dtypes': [values[id(n)][k].dtype if values[id(n)][k] is not None else None for n, k in sym._outputs]}


# ----------------------------------------------------------------------------------------------
# construction helpers
# ----------------------------------------------------------------------------------------------
def var(name, attr=None, shape=None, lr_mult=None, wd_mult=None, dtype=None, init=None, stype=None, **kwargs):
    """Create a variable symbol (``mx.sym.var`` / ``Variable``)."""
    if not isinstance(name, str):
        raise TypeError('Expect a string for variable `name`')
    attrs = AttrScope.current().get(attr)
    attrs = dict(attrs) if attrs else {}
    if shape is not None:
        attrs['__shape__'] = str(tuple(shape))
    if lr_mult is not None:
        attrs['__lr_mult__'] = str(lr_mult)
    if wd_mult is not None:
        attrs['__wd_mult__'] = str(wd_mult)
    if dtype is not None:
        from ..base import dtype_flag
        attrs['__dtype__'] = str(dtype_flag(dtype))
    if init is not None:
        attrs['__init__'] = init if isinstance(init, str) else init.dumps()
    if stype is not None:
        attrs['__storage_type__'] = str({'default': 0, 'row_sparse': 1, 'csr': 2}[stype])
    for k, v in kwargs.items():
        if k.startswith('__') and k.endswith('__'):
            attrs[k] = str(v)
        else:
            raise ValueError('Attribute name=%s is not supported. Additional attributes must start and end with '
                             'double underscores, e.g, __yourattr__' % k)
    return Symbol([(_Node(None, name, user_attrs=attrs), 0)])


Variable = var


def Group(symbols):
    outs = []
    for s in symbols:
        outs.extend(s._outputs)
    return Symbol(outs)


def _make_op_symbol(op, sym_inputs, attrs, name, user_attrs=None, resolved=False):
    if not resolved:      # `resolved`: the caller already passed the name through the NameManager
        hint = op.name.lower().lstrip('_')
        name = NameManager.current().get(name, hint)
    inputs = []
    for s in sym_inputs:
        if s is None:
            continue
        if len(s._outputs) != 1:
            if op.variadic:
                inputs.extend(s._outputs)
                continue
            raise MXNetError('operator %s got a grouped symbol as one input' % op.name)
        inputs.append(s._outputs[0])
    ua = AttrScope.current().get(user_attrs)
    node = _Node(op, name, dict(attrs), inputs, op.num_outputs(attrs) or 1, dict(ua) if ua else {})
    return Symbol([(node, i) for i in range(node.nout)]) if node.nout > 1 else Symbol([(node, 0)])


def _op_frontend(op):
    """Symbol-composition function of an operator; missing array inputs become auto-named variables
    (``fc1_weight``, ``bn0_moving_mean`` …) exactly like the reference's generated functions."""
    in_names = op.inputs

    def fn(*args, **kwargs):
        name = kwargs.pop('name', None)
        attr = kwargs.pop('attr', None)
        sym_kwargs = {k: v for k, v in kwargs.items() if isinstance(v, Symbol)}
        attrs = {k: v for k, v in kwargs.items() if not isinstance(v, Symbol)}
        attrs.pop('out', None)
        user_attrs = {k: attrs.pop(k) for k in list(attrs) if k.startswith('__') and k.endswith('__')}
        if attr:
            user_attrs.update(attr)
        pos = [a for a in args if isinstance(a, Symbol)]
        extra = [a for a in args if not isinstance(a, Symbol)]
        if op.variadic:
            syms = []
            for a in args:
                if isinstance(a, (list, tuple)):
                    syms.extend(a)
                elif isinstance(a, Symbol):
                    syms.append(a)
            syms.extend(sym_kwargs.values())
            if 'num_args' in op.defaults:
                attrs.setdefault('num_args', len(syms))
            return _make_op_symbol(op, syms, attrs, name, user_attrs)
        for k, v in zip([k for k in op.defaults if k not in attrs], extra):
            attrs[k] = v
        hint = op.name.lower().lstrip('_')
        name = NameManager.current().get(name, hint)
        syms = []
        for i, nm in enumerate(in_names):
            if i < len(pos):
                syms.append(pos[i])
            elif nm in sym_kwargs:
                syms.append(sym_kwargs[nm])
            else:
                syms.append(None)
        # optional inputs switched off by attributes are not materialised
        no_bias = attrs.get('no_bias', op.defaults.get('no_bias', False))
        out_syms = []
        for nm, s in zip(in_names, syms):
            if s is None:
                if nm == 'bias' and no_bias:
                    continue
                if nm in ('gamma',) and op.name == 'LeakyReLU' and attrs.get('act_type', 'leaky') != 'prelu':
                    continue
                if nm in ('length', 'mask', 'sequence_length', 'data_lengths', 'label_lengths', 'like', 'state_cell',
                          'weights', 'bins', 'obj_t', 'values', 'rhs', 'residual') and nm not in ('rhs',):
                    if nm == 'state_cell' and attrs.get('mode', 'lstm') == 'lstm':
                        pass
                    else:
                        continue
                # a missing data input becomes the free variable ``<name>_data`` that composition fills later
                # (``net(fc3_data=other)``), as every missing input does in the reference
                s = var('%s_%s' % (name, nm))
            out_syms.append(s)
        return _make_op_symbol(op, out_syms, attrs, name, user_attrs, resolved=True)
    fn.__name__ = op.name
    fn.__doc__ = op.doc
    return fn


def load_json(json_str):
    """Build a Symbol from JSON, upgrading legacy layouts (``param``/``attr`` keys, missing aux inputs)."""
    g = json.loads(json_str)
    jnodes = g['nodes']
    nodes = []
    for jn in jnodes:
        raw = {}
        for key in ('param', 'attr', 'attrs'):
            if key in jn and isinstance(jn[key], dict):
                raw.update(jn[key])
        opname = jn['op']
        if opname == 'null':
            nodes.append(_Node(None, jn['name'], user_attrs={k: v for k, v in raw.items()}))
            continue
        if not _reg.has(opname):
            raise MXNetError('Operator %s in the symbol file is not registered' % opname)
        op = _reg.get(opname)
        attrs, user = {}, {}
        for k, v in raw.items():
            if k.startswith('__') or k in _HIDDEN_KEYS:
                user[k if k.startswith('__') else '__%s__' % k] = v
            else:
                attrs[k] = _parse_attr(v)
        inputs = [(nodes[i[0]], i[1]) for i in jn['inputs']]
        for k, sg in enumerate(jn.get('subgraphs', ())):
            attrs['__subgraph__%d' % k] = load_json(json.dumps(sg))
        node = _Node(op, jn['name'], attrs, inputs, 1, user)
        node.nout = op.num_outputs(attrs) or 1
        # files written before auxiliary states became explicit inputs
        if not op.variadic and op.aux and len(inputs) < len(op.inputs):
            have = len(inputs)
            for nm in op.inputs[have:]:
                if nm in op.aux:
                    node.inputs.append((_Node(None, '%s_%s' % (jn['name'], nm)), 0))
        nodes.append(node)
    heads = g.get('heads', [[len(nodes) - 1, 0, 0]])
    return Symbol([(nodes[h[0]], h[1]) for h in heads])


fromjson = load_json


def load(fname):
    with open(fname) as f:
        return load_json(f.read())


def zeros(shape, dtype=None, **kwargs):
    return _make_op_symbol(_reg.get('_zeros'), [], {'shape': tuple(shape) if not isinstance(shape, int) else (shape,),
                                                     'dtype': dtype or 'float32'}, kwargs.get('name'))


def ones(shape, dtype=None, **kwargs):
    return _make_op_symbol(_reg.get('_ones'), [], {'shape': tuple(shape) if not isinstance(shape, int) else (shape,),
                                                    'dtype': dtype or 'float32'}, kwargs.get('name'))


def full(shape, val, dtype=None, **kwargs):
    return _make_op_symbol(_reg.get('_full'), [], {'shape': tuple(shape) if not isinstance(shape, int) else (shape,),
                                                    'dtype': dtype or 'float32', 'value': val}, kwargs.get('name'))


def arange(start, stop=None, step=1.0, repeat=1, infer_range=False, name=None, dtype=None):
    return _make_op_symbol(_reg.get('_arange'), [], {'start': start, 'stop': stop, 'step': step, 'repeat': repeat,
                                                      'dtype': dtype or 'float32'}, name)


# ---- Symbol methods that complete the NDArray-like surface (python/mxnet/symbol/symbol.py) ----------------------
from ..base import NotImplementedForSymbol          # noqa: E402  (one class for ``mx.base`` and ``mx.sym``)


def _symbol_astype(self, dtype, name=None):
    """A Symbol of the same values cast to ``dtype``."""
    return _op_frontend(_reg.get('Cast'))(self, dtype=dtype_name(to_torch_dtype(dtype)), name=name)


_DYNAMIC_SHAPE_OPS = ('_contrib_boolean_mask', '_npi_nonzero', '_npi_unique', '_npx_nonzero', '_contrib_dynamic_reshape',
                      '_npi_boolean_mask', '_npi_advanced_indexing', '_npi_delete', '_npi_insert_tensor')


def _symbol_has_dynamic_shape_op(self):
    """Whether the graph contains an operator whose output shape depends on input values."""
    return any(n.op is not None and (n.op.name in _DYNAMIC_SHAPE_OPS or any(a in _DYNAMIC_SHAPE_OPS for a in n.op.aliases))
               for n in _topo(self._outputs))


def _only_ndarray(name):
    def method(self, *args, **kwargs):
        raise NotImplementedForSymbol(method, None, *args)
    method.__name__ = name
    return method


Symbol.astype = _symbol_astype
Symbol.has_dynamic_shape_op = _symbol_has_dynamic_shape_op
for _n in ('as_in_context', 'as_in_ctx', 'asnumpy', 'asscalar', 'backward', 'copy', 'detach', 'wait_to_read'):
    if _n not in Symbol.__dict__:
        setattr(Symbol, _n, _only_ndarray(_n))

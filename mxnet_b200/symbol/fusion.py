"""Pointwise fusion: connected groups of elementwise operators of a Symbol become one ``_FusedOp`` node whose CUDA
kernel is generated from per-operator expression templates and compiled at run time with NVRTC for the running
architecture (the role of ``src/imperative/pointwise_fusion_pass.cc:61-352`` and ``src/operator/fusion/fused_op.cu``
with the templates of ``fused_op-inl.h`` in the reference; switch ``MXNET_USE_FUSION``).

Differences in design:

* The pass needs no shapes.  A fused node decides per call: when every input is a contiguous floating CUDA tensor that
  either has the output's shape, holds one element, or spans the last axis (a bias), the generated kernel runs; any
  other call evaluates the group's operators one by one, so fusing never changes what a graph accepts.
* Backward is a second generated kernel that re-computes the group's intermediates in registers from the saved *inputs*
  and applies the chain rule in reverse order, so a fused group keeps no intermediate tensor alive for autograd.
* All arithmetic is in fp32 whatever the storage type; loads and stores move four elements per thread as one vector
  when sizes and addresses allow.
"""
import math

import torch

from .. import env as _env
from ..base import MXNetError, to_torch_dtype
from ..ops import registry as _reg
from .symbol import Symbol, _Node, _topo

__all__ = ['fuse_pointwise', 'FusedGroup', 'kernel_source', 'stats']

stats = {'groups': 0, 'kernel_calls': 0, 'fallback_calls': 0, 'compiled': 0}


# ------------------------------------------------------------------------------------------------------------
# expression templates.  forward(x, attrs) -> C expression; backward(g, x, y, attrs) -> one expression per input
# (None: no gradient flows).  ``x`` is the list of input variable names, ``y`` the output variable name.
# ------------------------------------------------------------------------------------------------------------
def _lit(v):
    v = float(v)
    if math.isinf(v):
        return '(-INFINITY)' if v < 0 else 'INFINITY'
    if math.isnan(v):
        return 'NAN'
    return '%.9gf' % v if ('e' in '%.9g' % v or '.' in '%.9g' % v) else '%.9g.f' % v


_UNARY = {
    'relu': ('fmaxf({x}, 0.f)', '({x} > 0.f ? {g} : 0.f)'),
    'sigmoid': ('(1.f / (1.f + __expf(-{x})))', '({g} * {y} * (1.f - {y}))'),
    'tanh': ('tanhf({x})', '({g} * (1.f - {y} * {y}))'),
    'exp': ('__expf({x})', '({g} * {y})'),
    'log': ('__logf({x})', '({g} / {x})'),
    'log2': ('log2f({x})', '({g} / ({x} * 0.693147181f))'),
    'log10': ('log10f({x})', '({g} / ({x} * 2.30258509f))'),
    'log1p': ('log1pf({x})', '({g} / (1.f + {x}))'),
    'expm1': ('expm1f({x})', '({g} * ({y} + 1.f))'),
    'sqrt': ('sqrtf({x})', '({g} * 0.5f / {y})'),
    'rsqrt': ('rsqrtf({x})', '(-0.5f * {g} * {y} / {x})'),
    'cbrt': ('cbrtf({x})', '({g} / (3.f * {y} * {y}))'),
    'square': ('({x} * {x})', '(2.f * {g} * {x})'),
    'abs': ('fabsf({x})', '({x} > 0.f ? {g} : ({x} < 0.f ? -{g} : 0.f))'),
    'sign': ('({x} > 0.f ? 1.f : ({x} < 0.f ? -1.f : 0.f))', None),
    'negative': ('(-{x})', '(-{g})'),
    'reciprocal': ('(1.f / {x})', '(-{g} * {y} * {y})'),
    'erf': ('erff({x})', '({g} * 1.12837917f * __expf(-{x} * {x}))'),
    'sin': ('sinf({x})', '({g} * cosf({x}))'),
    'cos': ('cosf({x})', '(-{g} * sinf({x}))'),
    'tan': ('tanf({x})', '({g} * (1.f + {y} * {y}))'),
    'sinh': ('sinhf({x})', '({g} * coshf({x}))'),
    'cosh': ('coshf({x})', '({g} * sinhf({x}))'),
    'arcsin': ('asinf({x})', '({g} * rsqrtf(1.f - {x} * {x}))'),
    'arccos': ('acosf({x})', '(-{g} * rsqrtf(1.f - {x} * {x}))'),
    'arctan': ('atanf({x})', '({g} / (1.f + {x} * {x}))'),
    'arcsinh': ('asinhf({x})', '({g} * rsqrtf({x} * {x} + 1.f))'),
    'arccosh': ('acoshf({x})', '({g} * rsqrtf({x} * {x} - 1.f))'),
    'arctanh': ('atanhf({x})', '({g} / (1.f - {x} * {x}))'),
    'softsign': ('({x} / (1.f + fabsf({x})))', '({g} / ((1.f + fabsf({x})) * (1.f + fabsf({x}))))'),
    'log_sigmoid': ('(fminf({x}, 0.f) - log1pf(__expf(-fabsf({x}))))', '({g} / (1.f + __expf({x})))'),
    'mish': ('({x} * tanhf(fmaxf({x}, 0.f) + log1pf(__expf(-fabsf({x})))))',
             '({g} * mxb_mish_grad({x}))'),
    'softrelu': ('(fmaxf({x}, 0.f) + log1pf(__expf(-fabsf({x}))))', '({g} / (1.f + __expf(-{x})))'),
    'gelu': ('(0.5f * {x} * (1.f + mxb_erf_fast({x} * 0.707106781f)))',
             '({g} * (0.5f * (1.f + mxb_erf_fast({x} * 0.707106781f)) + {x} * 0.398942280f * __expf(-0.5f * {x} * {x})))'),
    'floor': ('floorf({x})', None), 'ceil': ('ceilf({x})', None), 'trunc': ('truncf({x})', None),
    'rint': ('rintf({x})', None), 'fix': ('truncf({x})', None),
    'degrees': ('({x} * 57.2957795f)', '({g} * 57.2957795f)'),
    'radians': ('({x} * 0.0174532925f)', '({g} * 0.0174532925f)'),
    'identity': ('{x}', '{g}'),
    'stop': ('{x}', None),
}

_PRELUDE_FUNCS = '''
// Abramowitz & Stegun 7.1.26: absolute error below 7e-7 in fp32, about half the instructions of erff
__device__ __forceinline__ float mxb_erf_fast(float x) {
  const float ax = fabsf(x);
  const float t = __fdividef(1.f, fmaf(0.3275911f, ax, 1.f));
  float p = fmaf(1.061405429f, t, -1.453152027f);
  p = fmaf(p, t, 1.421413741f);
  p = fmaf(p, t, -0.284496736f);
  p = fmaf(p, t, 0.254829592f);
  return copysignf(1.f - p * t * __expf(-ax * ax), x);
}
__device__ __forceinline__ float mxb_mish_grad(float x) {
  const float sp = fmaxf(x, 0.f) + log1pf(__expf(-fabsf(x)));
  const float t = tanhf(sp);
  return t + x * (1.f - t * t) / (1.f + __expf(-x));
}
'''


def _unary(kind):
    f, b = _UNARY[kind]
    return (lambda x, a: f.format(x=x[0]),
            lambda g, x, y, a: [b.format(g=g, x=x[0], y=y) if b is not None else None])


def _binary(fwd, ga, gb):
    return (lambda x, a: fwd.format(a=x[0], b=x[1]),
            lambda g, x, y, a: [ga.format(g=g, a=x[0], b=x[1], y=y) if ga else None,
                                gb.format(g=g, a=x[0], b=x[1], y=y) if gb else None])


def _scalar(fwd, grad):
    return (lambda x, a: fwd.format(x=x[0], s=_lit(a.get('scalar', 0.0))),
            lambda g, x, y, a: [grad.format(g=g, x=x[0], y=y, s=_lit(a.get('scalar', 0.0))) if grad else None])


def _activation(x, a):
    kind = a.get('act_type', 'relu')
    if kind not in ('relu', 'sigmoid', 'tanh', 'softrelu', 'softsign', 'log_sigmoid', 'mish'):
        return None
    return kind


def _leaky_kind(a):
    kind = a.get('act_type', 'leaky')
    return kind if kind in ('leaky', 'elu', 'selu', 'gelu') else None


def _leaky_fwd(x, a):
    kind, s = _leaky_kind(a), _lit(a.get('slope', 0.25))
    v = x[0]
    if kind == 'leaky':
        return '({x} > 0.f ? {x} : {s} * {x})'.format(x=v, s=s)
    if kind == 'elu':
        return '({x} > 0.f ? {x} : {s} * expm1f({x}))'.format(x=v, s=s)
    if kind == 'selu':
        return '(1.05070099f * ({x} > 0.f ? {x} : 1.67326324f * expm1f({x})))'.format(x=v)
    return _UNARY['gelu'][0].format(x=v)


def _leaky_bwd(g, x, y, a):
    kind, s = _leaky_kind(a), _lit(a.get('slope', 0.25))
    v = x[0]
    if kind == 'leaky':
        return ['({x} > 0.f ? {g} : {s} * {g})'.format(x=v, g=g, s=s)]
    if kind == 'elu':
        return ['({x} > 0.f ? {g} : {g} * {s} * __expf({x}))'.format(x=v, g=g, s=s)]
    if kind == 'selu':
        return ['({g} * 1.05070099f * ({x} > 0.f ? 1.f : 1.67326324f * __expf({x})))'.format(x=v, g=g)]
    return [_UNARY['gelu'][1].format(x=v, g=g, y=y)]


def _clip_fwd(x, a):
    e = x[0]
    if a.get('a_min') is not None:
        e = 'fmaxf(%s, %s)' % (e, _lit(a['a_min']))
    if a.get('a_max') is not None:
        e = 'fminf(%s, %s)' % (e, _lit(a['a_max']))
    return e


def _clip_bwd(g, x, y, a):
    conds = []
    if a.get('a_min') is not None:
        conds.append('%s >= %s' % (x[0], _lit(a['a_min'])))
    if a.get('a_max') is not None:
        conds.append('%s <= %s' % (x[0], _lit(a['a_max'])))
    return ['(%s ? %s : 0.f)' % (' && '.join(conds), g) if conds else g]


def _build_templates():
    """{canonical operator name: (forward, backward, accepts(node) -> bool)}"""
    t = {}

    def put(names, fwd_bwd, accepts=None):
        for n in names if isinstance(names, (list, tuple)) else [names]:
            if _reg.has(n):
                t[_reg.get(n).name] = (fwd_bwd[0], fwd_bwd[1], accepts)

    for kind in ('relu', 'sigmoid', 'tanh', 'exp', 'log', 'log2', 'log10', 'log1p', 'expm1', 'sqrt', 'rsqrt', 'cbrt', 'square',
                 'abs', 'sign', 'negative', 'reciprocal', 'erf', 'sin', 'cos', 'tan', 'sinh', 'cosh', 'arcsin', 'arccos',
                 'arctan', 'arcsinh', 'arccosh', 'arctanh', 'softsign', 'log_sigmoid', 'mish', 'floor', 'ceil', 'trunc',
                 'rint', 'fix', 'degrees', 'radians'):
        put(kind, _unary(kind))
    put(['identity', '_copy'], _unary('identity'))
    put(['BlockGrad', 'stop_gradient'], _unary('stop'))
    put('Activation', (lambda x, a: _UNARY[_activation(x, a)][0].format(x=x[0]),
                       lambda g, x, y, a: [_UNARY[_activation(x, a)][1].format(g=g, x=x[0], y=y)]),
        lambda n: _activation(None, n.attrs) is not None)
    put('LeakyReLU', (_leaky_fwd, _leaky_bwd), lambda n: len(n.inputs) == 1 and _leaky_kind(n.attrs) is not None)
    put('clip', (_clip_fwd, _clip_bwd))
    put(['Cast', 'amp_cast'], _unary('identity'),
        lambda n: to_torch_dtype(n.attrs.get('dtype', 'float32')) in (torch.float16, torch.bfloat16, torch.float32))

    put(['broadcast_add', '_npi_add'], _binary('({a} + {b})', '{g}', '{g}'))
    put(['broadcast_sub', '_npi_subtract'], _binary('({a} - {b})', '{g}', '(-{g})'))
    put(['broadcast_mul', '_npi_multiply'], _binary('({a} * {b})', '({g} * {b})', '({g} * {a})'))
    put(['broadcast_div', '_npi_true_divide'], _binary('({a} / {b})', '({g} / {b})', '(-{g} * {y} / {b})'))
    put(['broadcast_maximum', '_npi_maximum'], _binary('fmaxf({a}, {b})', '({a} >= {b} ? {g} : 0.f)', '({a} >= {b} ? 0.f : {g})'))
    put(['broadcast_minimum', '_npi_minimum'], _binary('fminf({a}, {b})', '({a} <= {b} ? {g} : 0.f)', '({a} <= {b} ? 0.f : {g})'))
    put(['broadcast_power', '_npi_power'], _binary('powf({a}, {b})', '({g} * {b} * powf({a}, {b} - 1.f))', '({g} * {y} * __logf({a}))'))
    put(['_hypot'], _binary('hypotf({a}, {b})', '({g} * {a} / {y})', '({g} * {b} / {y})'))

    put(['_add_scalar', '_npi_add_scalar'], _scalar('({x} + {s})', '{g}'))
    put(['_sub_scalar', '_npi_subtract_scalar'], _scalar('({x} - {s})', '{g}'))
    put(['_rsub_scalar', '_npi_rsubtract_scalar'], _scalar('({s} - {x})', '(-{g})'))
    put(['_mul_scalar', '_npi_multiply_scalar'], _scalar('({x} * {s})', '({g} * {s})'))
    put(['_div_scalar', '_npi_true_divide_scalar'], _scalar('({x} / {s})', '({g} / {s})'))
    put(['_rdiv_scalar', '_npi_rtrue_divide_scalar'], _scalar('({s} / {x})', '(-{g} * {y} / {x})'))
    put(['_power_scalar', '_npi_power_scalar'], _scalar('powf({x}, {s})', '({g} * {s} * powf({x}, {s} - 1.f))'))
    put(['_rpower_scalar', '_npi_rpower_scalar'], _scalar('powf({s}, {x})', '({g} * {y} * __logf({s}))'))
    put(['_maximum_scalar', '_npi_maximum_scalar'], _scalar('fmaxf({x}, {s})', '({x} >= {s} ? {g} : 0.f)'))
    put(['_minimum_scalar', '_npi_minimum_scalar'], _scalar('fminf({x}, {s})', '({x} <= {s} ? {g} : 0.f)'))
    return t


_templates = None


def templates():
    global _templates
    if _templates is None:
        _templates = _build_templates()
    return _templates


def fusable(node):
    if node.op is None or node.nout != 1:
        return False
    t = templates().get(node.op.name)
    if t is None or any(i is None for i in node.inputs):
        return False
    return t[2] is None or bool(t[2](node))


# ------------------------------------------------------------------------------------------------------------
# the pass
# ------------------------------------------------------------------------------------------------------------
_MAX_INPUTS = 24
_MAX_NODES = 96


def _find_groups(nodes):
    """Partition the fusable nodes into connected groups such that contracting every group keeps the graph acyclic.
    Returns {id(node): group index} for nodes in groups of two or more."""
    index = {id(n): i for i, n in enumerate(nodes)}
    root = list(range(len(nodes)))               # union-find parent; only fusable nodes ever get merged
    members = {i: [i] for i in range(len(nodes))}

    def find(i):
        while root[i] != i:
            root[i] = root[root[i]]
            i = root[i]
        return i

    consumers = [[] for _ in nodes]
    for i, n in enumerate(nodes):
        for inp, _k in n.inputs:
            consumers[index[id(inp)]].append(i)
    ok = [fusable(n) for n in nodes]

    def path_through_outside(src, dst, limit):
        """Is there a path from group ``src`` to group ``dst`` whose first step leaves ``src``?  Groups move as one
        node.  ``limit``: no node after it (in topological order) can lie on such a path."""
        stack, seen = [], {src}
        for m in members[src]:
            for c in consumers[m]:
                g = find(c)
                if g not in seen and c <= limit:
                    if g == dst:
                        continue                  # a direct edge src -> dst is what the merge contracts
                    seen.add(g)
                    stack.append(g)
        while stack:
            g = stack.pop()
            for m in members[g]:
                for c in consumers[m]:
                    gc = find(c)
                    if gc == dst:
                        return True
                    if gc not in seen and c <= limit:
                        seen.add(gc)
                        stack.append(gc)
        return False

    for i, n in enumerate(nodes):
        if not ok[i]:
            continue
        for inp, _k in n.inputs:
            j = index[id(inp)]
            if not ok[j]:
                continue
            gj, gi = find(j), find(i)
            if gj == gi or len(members[gj]) + len(members[gi]) > _MAX_NODES:
                continue
            if path_through_outside(gj, gi, i) or path_through_outside(gi, gj, i):
                continue
            if len(members[gj]) < len(members[gi]):
                gj, gi = gi, gj
            root[gi] = gj
            members[gj].extend(members.pop(gi))
    out = {}
    for i in range(len(nodes)):
        if ok[i] and len(members[find(i)]) >= 2:
            out[id(nodes[i])] = find(i)
    return out


def fuse_pointwise(sym):
    """Return a Symbol computing the same outputs with every group of two or more connected elementwise operators
    replaced by one ``_FusedOp`` node."""
    nodes = _topo(sym._outputs)
    membership = _find_groups(nodes)
    if not membership:
        return sym
    heads = {(id(n), k) for n, k in sym._outputs}
    used_outside = set()                          # entries of group members read by a node outside their group
    for n in nodes:
        for inp, k in n.inputs:
            if id(inp) in membership and membership.get(id(n)) != membership[id(inp)]:
                used_outside.add((id(inp), k))
    by_group = {}
    for n in nodes:
        g = membership.get(id(n))
        if g is not None:
            by_group.setdefault(g, []).append(n)

    # units of the contracted graph in an order in which every unit follows the units it reads
    def unit(n):
        g = membership.get(id(n))
        return ('g', g) if g is not None else ('n', id(n))

    unit_nodes, deps = {}, {}
    for n in nodes:
        u = unit(n)
        unit_nodes.setdefault(u, []).append(n)
        d = deps.setdefault(u, set())
        for inp, _k in n.inputs:
            ui = unit(inp)
            if ui != u:
                d.add(ui)
    order, state = [], {}
    for start in unit_nodes:
        if start in state:
            continue
        stack = [(start, iter(deps[start]))]
        state[start] = 1
        while stack:
            u, it = stack[-1]
            advanced = False
            for v in it:
                if v not in state:
                    state[v] = 1
                    stack.append((v, iter(deps[v])))
                    advanced = True
                    break
                if state[v] == 1:
                    raise MXNetError('pointwise fusion produced a cycle')     # the grouping rules exclude this
            if not advanced:
                state[u] = 2
                order.append(u)
                stack.pop()

    op = _reg.get('_FusedOp')
    mapping = {}                                  # id(old node) -> list of new entries per output

    def copy_node(n):
        nn = _Node(n.op, n.name, dict(n.attrs), [mapping[id(i)][k] for i, k in n.inputs], n.nout, dict(n.user_attrs))
        mapping[id(n)] = [(nn, i) for i in range(n.nout)]

    for u in order:
        if u[0] == 'n':
            n = unit_nodes[u][0]
            if n.op is None:
                mapping[id(n)] = [(n, 0)]
            else:
                copy_node(n)
            continue
        group_nodes = by_group[u[1]]
        member_ids = {id(m) for m in group_nodes}
        ext, ext_pos = [], {}
        for m in group_nodes:
            for inp, k in m.inputs:
                if id(inp) not in member_ids and (id(inp), k) not in ext_pos:
                    ext_pos[(id(inp), k)] = len(ext)
                    ext.append((inp, k))
        outs = [m for m in group_nodes if (id(m), 0) in used_outside or (id(m), 0) in heads]
        if len(ext) > _MAX_INPUTS or not outs:
            for m in group_nodes:                 # too many inputs: keep the members as they are
                copy_node(m)
            continue
        fg = FusedGroup(group_nodes, ext_pos, outs)
        label = '_'.join(dict.fromkeys(m.op.name.lstrip('_') for m in group_nodes))[:60]
        node = _Node(op, 'fused_%s_%d' % (label, u[1]), {'group': fg}, [mapping[id(inp)][k] for inp, k in ext], len(outs))
        stats['groups'] += 1
        pos = {id(m): i for i, m in enumerate(outs)}
        for m in group_nodes:
            mapping[id(m)] = [(node, pos[id(m)])] if id(m) in pos else [None]
    return Symbol([mapping[id(n)][k] for n, k in sym._outputs])


# ------------------------------------------------------------------------------------------------------------
# code generation
# ------------------------------------------------------------------------------------------------------------
_CTYPE = {torch.float32: 'float', torch.float16: '__half', torch.bfloat16: '__nv_bfloat16'}
FULL, ONE, LAST = 0, 1, 2                         # how an input maps onto the output's elements

_PRELUDE = '''#include <cuda_fp16.h>
#include <cuda_bf16.h>
template <typename T, int N> struct __align__(sizeof(T) * N) Vec { T v[N]; };
__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
''' + _PRELUDE_FUNCS


def kernel_source(group, in_dtypes, modes, out_dtypes, vec, backward=False, need_grad=None):
    """CUDA source of the forward (or backward) kernel of ``group`` for one call signature.

    Forward arguments:  n (vectors), c (vectors along the last axis), inputs..., outputs...
    Backward arguments: n, c, inputs..., output gradients..., input gradients for every input with need_grad
    (inputs that are broadcast receive a full-size fp32 gradient that the caller reduces)."""
    nin, nout = len(in_dtypes), len(out_dtypes)
    need_grad = list(need_grad or [False] * nin)
    args = ['const long long n', 'const long long c']
    args += ['const %s* __restrict__ in%d' % (_CTYPE[t], i) for i, t in enumerate(in_dtypes)]
    if backward:
        args += ['const %s* __restrict__ og%d' % (_CTYPE[t], i) for i, t in enumerate(out_dtypes)]
        gtypes = [(_CTYPE[t] if modes[i] == FULL else 'float') for i, t in enumerate(in_dtypes)]
        args += ['%s* __restrict__ ig%d' % (gtypes[i], i) for i in range(nin) if need_grad[i]]
    else:
        args += ['%s* __restrict__ out%d' % (_CTYPE[t], i) for i, t in enumerate(out_dtypes)]
    L = [_PRELUDE, 'extern "C" __global__ void __launch_bounds__(256) %s(%s) {' % ('fused_bwd' if backward else 'fused_fwd',
                                                                                 ', '.join(args)),
         '  constexpr int V = %d;' % vec,
         '  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < n; i += gridDim.x * 256LL) {']
    for i, t in enumerate(in_dtypes):
        ct = _CTYPE[t]
        if modes[i] == FULL:
            L.append('    const Vec<%s, V> a%d = reinterpret_cast<const Vec<%s, V>*>(in%d)[i];' % (ct, i, ct, i))
        elif modes[i] == LAST:
            L.append('    const Vec<%s, V> a%d = reinterpret_cast<const Vec<%s, V>*>(in%d)[i %% c];' % (ct, i, ct, i))
        else:
            L.append('    const float s%d = to_f(in%d[0]);' % (i, i))
    if backward:
        for i, t in enumerate(out_dtypes):
            L.append('    const Vec<%s, V> b%d = reinterpret_cast<const Vec<%s, V>*>(og%d)[i];' % (_CTYPE[t], i, _CTYPE[t], i))
        for i in range(nin):
            if need_grad[i]:
                L.append('    Vec<%s, V> r%d;' % (gtypes[i], i))
    else:
        for i, t in enumerate(out_dtypes):
            L.append('    Vec<%s, V> r%d;' % (_CTYPE[t], i))
    L.append('#pragma unroll')
    L.append('    for (int e = 0; e < V; ++e) {')
    for i in range(nin):
        L.append('      const float x%d = %s;' % (i, ('s%d' % i) if modes[i] == ONE else 'to_f(a%d.v[e])' % i))
    tmpl = templates()
    names = {}                                    # id(member) -> variable of its value

    def operand(entry):
        inp, k = entry
        if id(inp) in names:
            return names[id(inp)]
        return 'x%d' % group.ext_pos[(id(inp), k)]

    for j, m in enumerate(group.nodes):
        fwd = tmpl[m.op.name][0]
        L.append('      const float t%d = %s;' % (j, fwd([operand(e) for e in m.inputs], m.attrs)))
        names[id(m)] = 't%d' % j
    if not backward:
        for i, m in enumerate(group.outputs):
            L.append('      r%d.v[e] = from_f<%s>(%s);' % (i, _CTYPE[out_dtypes[i]], names[id(m)]))
    else:
        out_index = {id(m): i for i, m in enumerate(group.outputs)}
        for j, m in enumerate(group.nodes):
            seed = 'to_f(b%d.v[e])' % out_index[id(m)] if id(m) in out_index else '0.f'
            L.append('      float g%d = %s;' % (j, seed))
        for i in range(nin):
            L.append('      float d%d = 0.f;' % i)
        node_pos = {id(m): j for j, m in enumerate(group.nodes)}
        for j in range(len(group.nodes) - 1, -1, -1):
            m = group.nodes[j]
            bwd = tmpl[m.op.name][1]
            parts = bwd('g%d' % j, [operand(e) for e in m.inputs], 't%d' % j, m.attrs)
            for (inp, k), expr in zip(m.inputs, parts):
                if expr is None:
                    continue
                if id(inp) in node_pos:
                    L.append('      g%d += %s;' % (node_pos[id(inp)], expr))
                else:
                    L.append('      d%d += %s;' % (group.ext_pos[(id(inp), k)], expr))
        for i in range(nin):
            if need_grad[i]:
                L.append('      r%d.v[e] = from_f<%s>(d%d);' % (i, gtypes[i], i))
    L.append('    }')
    if backward:
        for i in range(nin):
            if need_grad[i]:
                L.append('    reinterpret_cast<Vec<%s, V>*>(ig%d)[i] = r%d;' % (gtypes[i], i, i))
    else:
        for i, t in enumerate(out_dtypes):
            L.append('    reinterpret_cast<Vec<%s, V>*>(out%d)[i] = r%d;' % (_CTYPE[t], i, i))
    L += ['  }', '}']
    return '\n'.join(L) + '\n'


_include_dir = None


def _cuda_include():
    global _include_dir
    if _include_dir is None:
        import os
        cands = [os.environ.get('CUDA_HOME'), os.environ.get('CUDA_PATH'), '/usr/local/cuda']
        try:
            from torch.utils.cpp_extension import CUDA_HOME
            cands.insert(0, CUDA_HOME)
        except Exception:   # pylint: disable=broad-except
            pass
        for c in cands:
            if c and os.path.exists(os.path.join(c, 'include', 'cuda_fp16.h')):
                _include_dir = os.path.join(c, 'include')
                break
        else:
            raise MXNetError('pointwise fusion needs the CUDA headers (cuda_fp16.h); set CUDA_HOME')
    return _include_dir


def compile_cubin(source, arch='sm_100a'):
    """NVRTC: CUDA source -> cubin bytes for ``arch`` (no device needed)."""
    try:
        from cuda.bindings import nvrtc
    except Exception:   # pylint: disable=broad-except
        from cuda import nvrtc
    err, prog = nvrtc.nvrtcCreateProgram(source.encode(), b'mxb_fused.cu', 0, [], [])
    opts = [('--gpu-architecture=' + arch).encode(), ('-I' + _cuda_include()).encode(), b'-std=c++17']
    err, = nvrtc.nvrtcCompileProgram(prog, len(opts), opts)
    if int(err) != 0:
        _, n = nvrtc.nvrtcGetProgramLogSize(prog)
        log = b' ' * n
        nvrtc.nvrtcGetProgramLog(prog, log)
        raise MXNetError('NVRTC failed on a fused kernel:\n%s\n--- source ---\n%s' % (log.decode(errors='replace'), source))
    _, n = nvrtc.nvrtcGetCUBINSize(prog)
    cubin = b' ' * n
    nvrtc.nvrtcGetCUBIN(prog, cubin)
    nvrtc.nvrtcDestroyProgram(prog)
    stats['compiled'] += 1
    return cubin


_kernels = {}                                     # (device, source, name) -> (module, function), per process


def _driver():
    try:
        from cuda.bindings import driver as cu
    except Exception:   # pylint: disable=broad-except
        from cuda import cuda as cu
    return cu


def _ensure_context(index):
    """Make the device's primary context current on this thread for driver-API calls.  The tensor library binds it
    through the runtime API on the threads it computes on, but a thread that has only run cached allocations so far
    (an autograd worker) may have none."""
    cu = _driver()
    err, ctx = cu.cuCtxGetCurrent()
    if int(err) == 0 and ctx is not None and int(ctx) != 0:
        return
    torch.cuda.current_stream(index)              # initialises the runtime and the primary context
    err, dev = cu.cuDeviceGet(index)
    err, pctx = cu.cuDevicePrimaryCtxRetain(dev)
    if int(err) != 0:
        raise MXNetError('cuDevicePrimaryCtxRetain failed: %s' % err)
    err, = cu.cuCtxSetCurrent(pctx)
    if int(err) != 0:
        raise MXNetError('cuCtxSetCurrent failed: %s' % err)


def _get_function(source, name, index=0):
    hit = _kernels.get((index, source, name))
    if hit is not None:
        return hit[1]
    cu = _driver()
    major, minor = torch.cuda.get_device_capability(index)
    cubin = compile_cubin(source, 'sm_%d%d%s' % (major, minor, 'a' if major >= 9 else ''))
    _ensure_context(index)
    err, module = cu.cuModuleLoadData(cubin)
    if int(err) != 0:
        raise MXNetError('cuModuleLoadData failed on a fused kernel: %s' % err)
    err, fn = cu.cuModuleGetFunction(module, name.encode())
    if int(err) != 0:
        raise MXNetError('kernel %s not found in its module: %s' % (name, err))
    _kernels[(index, source, name)] = (module, fn)
    return fn


def _launch(fn, n_vec, c_vec, pointers, device):
    import ctypes
    cu = _driver()
    _ensure_context(device.index or 0)
    holders = [ctypes.c_longlong(n_vec), ctypes.c_longlong(c_vec)] + [ctypes.c_void_p(p) for p in pointers]
    arr = (ctypes.c_void_p * len(holders))(*[ctypes.addressof(h) for h in holders])
    blocks = max(1, min((n_vec + 255) // 256, 148 * 8))
    stream = torch.cuda.current_stream(device).cuda_stream
    err, = cu.cuLaunchKernel(fn, blocks, 1, 1, 256, 1, 1, 0, stream, ctypes.addressof(arr), 0)
    if int(err) != 0:
        raise MXNetError('launch of a fused kernel failed: %s' % err)


# ------------------------------------------------------------------------------------------------------------
# run time
# ------------------------------------------------------------------------------------------------------------
class FusedGroup(object):
    """The operators of one fused node.  ``nodes``: members in topological order; ``ext_pos``: {(id(producer), output
    index): position among the fused node's inputs}; ``outputs``: members whose value leaves the group."""

    def __init__(self, nodes, ext_pos, outputs):
        self.nodes, self.ext_pos, self.outputs = list(nodes), dict(ext_pos), list(outputs)
        self.nin = len(ext_pos)
        self._meta = {}                           # (dtypes, shapes) -> (out dtypes, out shapes)

    def __repr__(self):
        return '<FusedGroup %s>' % '+'.join(n.op.name for n in self.nodes)

    # -- operator by operator (also the abstract evaluation for shapes and types)
    def interpret(self, tensors):
        values = {}
        for m in self.nodes:
            ins = [values[id(i)] if id(i) in values else tensors[self.ext_pos[(id(i), k)]] for i, k in m.inputs]
            values[id(m)] = m.op.fn(*ins, **m.attrs)
        return tuple(values[id(m)] for m in self.outputs)

    def _signature(self, tensors):
        key = (tuple(t.dtype for t in tensors), tuple(tuple(t.shape) for t in tensors))
        hit = self._meta.get(key)
        if hit is None:
            with torch.no_grad():
                outs = self.interpret([torch.empty(t.shape, dtype=t.dtype, device='meta') for t in tensors])
            hit = (tuple(o.dtype for o in outs), tuple(tuple(o.shape) for o in outs))
            if len(self._meta) < 64:
                self._meta[key] = hit
        return hit

    def plan(self, tensors):
        """(modes, out dtypes, out shape, vector width) when the generated kernel can take this call, else None."""
        if not tensors or not all(isinstance(t, torch.Tensor) for t in tensors):
            return None
        dev = tensors[0].device
        if dev.type != 'cuda' or any(t.device != dev or t.dtype not in _CTYPE or not t.is_contiguous() for t in tensors):
            return None
        try:
            out_dtypes, out_shapes = self._signature(tensors)
        except Exception:   # pylint: disable=broad-except
            return None
        shape = out_shapes[0]
        if any(s != shape for s in out_shapes) or any(t not in _CTYPE for t in out_dtypes):
            return None
        n = 1
        for s in shape:
            n *= s
        if n == 0 or not shape:
            return None
        modes = []
        for t in tensors:
            if tuple(t.shape) == shape:
                modes.append(FULL)
            elif t.numel() == 1:
                modes.append(ONE)
            elif t.numel() == shape[-1] and t.shape[-1] == shape[-1]:
                modes.append(LAST)
            else:
                return None
        if FULL not in modes:
            return None
        moving = [t for t, m in zip(tensors, modes) if m != ONE]
        widths = ([8] if any(t.element_size() == 2 for t in moving) or any(d.itemsize == 2 for d in out_dtypes) else []) + [4]
        vec = 1
        for v in widths:                          # 16-byte accesses for the narrowest type when sizes and addresses allow
            if n % v == 0 and (LAST not in modes or shape[-1] % v == 0) and \
                    all(t.data_ptr() % (v * t.element_size()) == 0 for t in moving):
                vec = v
                break
        return tuple(modes), out_dtypes, shape, vec

    def run_forward(self, tensors, plan):
        modes, out_dtypes, shape, vec = plan
        src = kernel_source(self, [t.dtype for t in tensors], modes, out_dtypes, vec)
        fn = _get_function(src, 'fused_fwd', tensors[0].device.index or 0)
        dev = tensors[0].device
        outs = [torch.empty(shape, dtype=d, device=dev) for d in out_dtypes]
        n = outs[0].numel()
        _launch(fn, n // vec, max(shape[-1] // vec, 1), [t.data_ptr() for t in tensors] + [o.data_ptr() for o in outs], dev)
        stats['kernel_calls'] += 1
        return outs

    def run_backward(self, tensors, plan, ograds, need_grad):
        modes, out_dtypes, shape, vec = plan
        dev = tensors[0].device
        if vec > 1 and any(g.data_ptr() % (vec * g.element_size()) for g in ograds):
            vec = 1
        src = kernel_source(self, [t.dtype for t in tensors], modes, out_dtypes, vec, True, need_grad)
        fn = _get_function(src, 'fused_bwd', tensors[0].device.index or 0)
        grads = [torch.empty(shape, dtype=(t.dtype if m == FULL else torch.float32), device=dev) if ng else None
                 for t, m, ng in zip(tensors, modes, need_grad)]
        n = ograds[0].numel()
        _launch(fn, n // vec, max(shape[-1] // vec, 1),
                [t.data_ptr() for t in tensors] + [g.data_ptr() for g in ograds] + [g.data_ptr() for g in grads if g is not None],
                dev)
        stats['kernel_calls'] += 1
        res = []
        for t, m, g in zip(tensors, modes, grads):
            if g is None or m == FULL:
                res.append(g)
            elif m == ONE:
                res.append(g.sum().to(t.dtype).reshape(t.shape))
            else:
                res.append(g.reshape(-1, shape[-1]).sum(0).to(t.dtype).reshape(t.shape))
        return res

    def __call__(self, *tensors):
        plan = self.plan(tensors) if _env.get('MXNET_USE_FUSION') else None
        if plan is None:
            stats['fallback_calls'] += 1
            res = self.interpret(tensors)
        elif torch.is_grad_enabled() and any(t.requires_grad for t in tensors):
            res = _FusedFunction.apply(self, plan, *tensors)
        else:
            res = tuple(self.run_forward(tensors, plan))
        return res[0] if len(res) == 1 else tuple(res)


class _FusedFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, group, plan, *tensors):
        outs = group.run_forward(tensors, plan)
        ctx.group, ctx.plan = group, plan
        ctx.save_for_backward(*tensors)
        return tuple(outs)

    @staticmethod
    def backward(ctx, *ograds):
        tensors = ctx.saved_tensors
        shape, out_dtypes = ctx.plan[2], ctx.plan[1]
        og = [(g.contiguous() if g is not None else torch.zeros(shape, dtype=d, device=tensors[0].device))
              for g, d in zip(ograds, out_dtypes)]
        need = list(ctx.needs_input_grad[2:])
        grads = ctx.group.run_backward(tensors, ctx.plan, og, need)
        return (None, None) + tuple(grads)


def _fused_op(*tensors, group=None):
    if group is None:
        raise MXNetError('_FusedOp nodes are created by the pointwise fusion pass only')
    return group(*tensors)


_reg.register('_FusedOp', inputs=('*data',), nout=lambda attrs: len(attrs['group'].outputs))(_fused_op)

"""Testing helpers (``python/mxnet/test_utils.py``): dtype-aware comparisons, finite-difference gradient
checks, symbolic forward/backward checks, cross-device consistency, optimizer comparison, RNG tests."""
import contextlib
import numbers
import os

import numpy as np

from . import autograd, env
from .device import Device, cpu, gpu, current_device, num_gpus
from .ndarray.ndarray import NDArray

_DEFAULT_RTOL = {np.dtype(np.float16): 1e-2, np.dtype(np.float32): 1e-4, np.dtype(np.float64): 1e-5,
                 np.dtype(np.bool_): 0, np.dtype(np.int8): 0, np.dtype(np.uint8): 0, np.dtype(np.int32): 0,
                 np.dtype(np.int64): 0}
_DEFAULT_ATOL = {np.dtype(np.float16): 1e-1, np.dtype(np.float32): 1e-3, np.dtype(np.float64): 1e-20,
                 np.dtype(np.bool_): 0, np.dtype(np.int8): 0, np.dtype(np.uint8): 0, np.dtype(np.int32): 0,
                 np.dtype(np.int64): 0}
_default_device = [None]


def default_device():
    return _default_device[0] or current_device()


default_context = default_device


def set_default_device(dev):
    from . import device
    _default_device[0] = dev
    device.set_default_device(dev)


set_default_context = set_default_device


def default_dtype():
    return np.float32


def default_rtols():
    return dict(_DEFAULT_RTOL)


def default_atols():
    return dict(_DEFAULT_ATOL)


def get_rtol(rtol=None, dtype=np.dtype(np.float64)):
    return _DEFAULT_RTOL.get(np.dtype(dtype), 1e-5) if rtol is None else rtol


def get_atol(atol=None, dtype=np.dtype(np.float64)):
    return _DEFAULT_ATOL.get(np.dtype(dtype), 1e-20) if atol is None else atol


def get_tolerance(dat, tol, default_tol):
    if isinstance(tol, numbers.Number):
        return tol
    dtype = np.dtype(dat.dtype) if hasattr(dat, 'dtype') and not isinstance(dat.dtype, str) else np.dtype(np.float32)
    return default_tol.get(dtype, 1e-5)


def _as_np(a):
    if isinstance(a, NDArray):
        return a.asnumpy()
    return np.asarray(a)


def effective_dtype(dat):
    return np.dtype(dat.dtype) if not isinstance(dat.dtype, str) else np.dtype(np.float32)


def get_tols(x, y, rtol, atol):
    x, y = _as_np(x), _as_np(y)
    dts = [np.dtype(x.dtype), np.dtype(y.dtype)]
    rt = max(_DEFAULT_RTOL.get(d, 1e-5) for d in dts) if rtol is None else rtol
    at = max(_DEFAULT_ATOL.get(d, 1e-20) for d in dts) if atol is None else atol
    return rt, at


def same(a, b):
    return np.array_equal(_as_np(a), _as_np(b))


def almost_equal(a, b, rtol=None, atol=None, equal_nan=False, use_broadcast=True):
    rtol, atol = get_tols(a, b, rtol, atol)
    return np.allclose(_as_np(a).astype(np.float64), _as_np(b).astype(np.float64), rtol=rtol, atol=atol, equal_nan=equal_nan)


def find_max_violation(a, b, rtol=None, atol=None):
    rtol, atol = get_tols(a, b, rtol, atol)
    a, b = _as_np(a).astype(np.float64), _as_np(b).astype(np.float64)
    diff = np.abs(a - b)
    tol = atol + rtol * np.abs(b)
    violation = diff / (tol + 1e-20)
    loc = np.argmax(violation)
    idx = np.unravel_index(loc, violation.shape)
    return idx, np.max(violation)


def assert_almost_equal(a, b, rtol=None, atol=None, names=('a', 'b'), equal_nan=False, use_broadcast=True,
                        mismatches=(10, 10)):
    """Compare two arrays with tolerances picked from the less precise dtype (``test_utils.py:653``)."""
    if almost_equal(a, b, rtol, atol, equal_nan):
        return
    rtol, atol = get_tols(a, b, rtol, atol)
    an, bn = _as_np(a), _as_np(b)
    if an.shape != bn.shape and not use_broadcast:
        raise AssertionError('shape mismatch %s vs %s' % (an.shape, bn.shape))
    index, rel = find_max_violation(an, bn, rtol, atol)
    raise AssertionError('Items are not equal:\nError %f exceeds tolerance rtol=%e, atol=%e (mismatch at least at %s: '
                         '%s vs %s)\n %s: %s\n %s: %s' % (rel, rtol, atol, str(index), an[index] if an.shape else an,
                                                           bn[index] if bn.shape else bn, names[0],
                                                           np.array2string(an, threshold=20), names[1],
                                                           np.array2string(bn, threshold=20)))


def assert_allclose(a, b, rtol=1e-07, atol=0, equal_nan=True):
    assert_almost_equal(a, b, rtol, atol, equal_nan=equal_nan)


def assert_almost_equal_with_err(a, b, rtol=None, atol=None, etol=None, names=('a', 'b'), equal_nan=False, mismatches=(10, 10)):
    etol = etol or 0.0
    rtol, atol = get_tols(a, b, rtol, atol)
    an, bn = _as_np(a).astype(np.float64), _as_np(b).astype(np.float64)
    bad = ~np.isclose(an, bn, rtol=rtol, atol=atol, equal_nan=equal_nan)
    if bad.mean() > etol:
        assert_almost_equal(a, b, rtol, atol, names, equal_nan)


def assert_exception(f, exception_type, *args, **kwargs):
    try:
        f(*args, **kwargs)
        assert False
    except exception_type:
        return


def random_arrays(*shapes):
    arrays = [np.array(np.random.randn(), dtype=default_dtype()) if len(s) == 0 else
              np.random.randn(*s).astype(default_dtype()) for s in shapes]
    return arrays[0] if len(arrays) == 1 else arrays


def random_uniform_arrays(*shapes, **kwargs):
    low, high, dtype = kwargs.pop('low', 0.0), kwargs.pop('high', 1.0), kwargs.pop('dtype', default_dtype())
    arrays = [np.random.uniform(low, high, size=s).astype(dtype) for s in shapes]
    return arrays[0] if len(arrays) == 1 else arrays


def random_sample(population, k):
    import random
    assert 0 <= k <= len(population)
    pop = list(population)
    random.shuffle(pop)
    return pop[0:k]


def rand_shape_2d(dim0=10, dim1=10, allow_zero_size=False):
    low = 0 if allow_zero_size else 1
    return np.random.randint(low, dim0 + 1), np.random.randint(low, dim1 + 1)


def rand_shape_3d(dim0=10, dim1=10, dim2=10, allow_zero_size=False):
    low = 0 if allow_zero_size else 1
    return np.random.randint(low, dim0 + 1), np.random.randint(low, dim1 + 1), np.random.randint(low, dim2 + 1)


def rand_shape_nd(num_dim, dim=10, allow_zero_size=False):
    low = 0 if allow_zero_size else 1
    return tuple(np.random.randint(low, dim + 1, size=num_dim))


def rand_ndarray(shape, stype='default', density=None, dtype=None, ctx=None, **kwargs):
    from . import ndarray as nd
    a = np.random.uniform(-1, 1, size=shape).astype(dtype or 'float32')
    if stype != 'default':
        density = 0.5 if density is None else density
        mask = np.random.rand(shape[0]) < density if stype == 'row_sparse' else np.random.rand(*shape) < density
        a = a * (mask.reshape((-1,) + (1,) * (len(shape) - 1)) if stype == 'row_sparse' else mask)
        return nd.array(a, ctx=ctx, dtype=a.dtype).tostype(stype)
    return nd.array(a, ctx=ctx, dtype=a.dtype)


def np_reduce(dat, axis, keepdims, numpy_reduce_func):
    if isinstance(axis, int):
        axis = [axis]
    else:
        axis = list(axis) if axis is not None else range(len(dat.shape))
    ret = dat
    for i in reversed(sorted(axis)):
        ret = numpy_reduce_func(ret, axis=i)
    if keepdims:
        keepdims_shape = list(dat.shape)
        for i in axis:
            keepdims_shape[i] = 1
        ret = ret.reshape(tuple(keepdims_shape))
    return ret


def numeric_grad(f, inputs, eps=1e-4):
    """Central finite differences of a scalar-valued ``f(*inputs)`` w.r.t. every numpy input."""
    grads = []
    for i, x in enumerate(inputs):
        g = np.zeros_like(x, dtype=np.float64)
        flat = x.reshape(-1)
        gf = g.reshape(-1)
        for j in range(flat.size):
            old = flat[j]
            flat[j] = old + eps
            fp = f(*inputs)
            flat[j] = old - eps
            fm = f(*inputs)
            flat[j] = old
            gf[j] = (fp - fm) / (2 * eps)
        grads.append(g)
    return grads


def check_numeric_gradient(fn, inputs, numeric_eps=1e-3, rtol=1e-2, atol=1e-4, grad_nodes=None, dtype=np.float64, ctx=None):
    """Compare autograd gradients of ``sum(fn(*inputs) * proj)`` with finite differences
    (``test_utils.py:1038``).  ``fn`` maps arrays to one array; inputs are numpy arrays or NDArrays.
    A Symbol may be given instead of a callable together with a list/dict of inputs."""
    from . import ndarray as nd
    from .symbol import Symbol
    if isinstance(fn, Symbol):
        sym = fn
        names = sym.list_arguments()
        if isinstance(inputs, dict):
            inputs = [inputs[n] for n in names]

        def fn(*arrs):   # pylint: disable=function-redefined
            outs = sym._run({n: a._data for n, a in zip(names, arrs)})
            return arrs[0].__class__._from_tensor(outs[0])
    ctx = ctx or default_device()
    np_inputs = [_as_np(x).astype(dtype) for x in inputs]
    arrays = [nd.array(x, ctx=ctx, dtype=dtype) for x in np_inputs]
    for a in arrays:
        a.attach_grad()
    with autograd.record():
        out = fn(*arrays)
    proj = np.random.uniform(0.5, 1.5, size=out.shape).astype(dtype)
    out.backward(nd.array(proj, ctx=ctx, dtype=dtype))
    sym_grads = [a.grad.asnumpy() for a in arrays]

    def scalar(*xs):
        with autograd.pause():
            o = fn(*[nd.array(x, ctx=ctx, dtype=dtype) for x in xs])
        return float((o.asnumpy().astype(np.float64) * proj).sum())
    num_grads = numeric_grad(scalar, [x.copy() for x in np_inputs], numeric_eps)
    for i, (sg, ng) in enumerate(zip(sym_grads, num_grads)):
        if grad_nodes is not None and i not in grad_nodes:
            continue
        assert_almost_equal(sg, ng, rtol, atol, ('autograd[%d]' % i, 'numeric[%d]' % i))


def check_symbolic_forward(sym, location, expected, rtol=None, atol=None, aux_states=None, ctx=None, equal_nan=False, dtype=np.float32):
    from . import ndarray as nd
    ctx = ctx or default_device()
    names = sym.list_arguments()
    if isinstance(location, (list, tuple)):
        location = dict(zip(names, location))
    args = {k: nd.array(_as_np(v), ctx=ctx, dtype=dtype) for k, v in location.items()}
    aux = {}
    if aux_states is not None:
        aux_names = sym.list_auxiliary_states()
        if isinstance(aux_states, (list, tuple)):
            aux_states = dict(zip(aux_names, aux_states))
        aux = {k: nd.array(_as_np(v), ctx=ctx, dtype=dtype) for k, v in aux_states.items()}
    ex = sym._bind(ctx, args, aux_states=aux)
    outs = ex.forward(is_train=False)
    if isinstance(expected, dict):
        expected = [expected[k] for k in sym.list_outputs()]
    for o, e in zip(outs, expected):
        assert_almost_equal(o, e, rtol, atol, ('FORWARD', 'EXPECTED'), equal_nan)
    return outs


def check_symbolic_backward(sym, location, out_grads, expected, rtol=None, atol=None, aux_states=None, grad_req='write',
                            ctx=None, grad_stypes=None, equal_nan=False, dtype=np.float32):
    from . import ndarray as nd
    ctx = ctx or default_device()
    names = sym.list_arguments()
    if isinstance(location, (list, tuple)):
        location = dict(zip(names, location))
    if isinstance(expected, (list, tuple)):
        expected = dict(zip(names, expected))
    args = {k: nd.array(_as_np(v), ctx=ctx, dtype=dtype) for k, v in location.items()}
    grads = {k: nd.zeros(v.shape, ctx=ctx, dtype=dtype) for k, v in args.items()}
    aux = {}
    if aux_states is not None:
        aux_names = sym.list_auxiliary_states()
        if isinstance(aux_states, (list, tuple)):
            aux_states = dict(zip(aux_names, aux_states))
        aux = {k: nd.array(_as_np(v), ctx=ctx, dtype=dtype) for k, v in aux_states.items()}
    ex = sym._bind(ctx, args, grads, grad_req, aux)
    ex.forward(is_train=True)
    if isinstance(out_grads, (list, tuple)):
        out_grads = [nd.array(_as_np(g), ctx=ctx, dtype=dtype) for g in out_grads]
    ex.backward(out_grads)
    for k, e in expected.items():
        assert_almost_equal(grads[k], e, rtol, atol, ('BACKWARD_%s' % k, 'EXPECTED_%s' % k), equal_nan)
    return grads


def check_consistency(sym, ctx_list, scale=1.0, grad_req='write', arg_params=None, aux_params=None, rtol=None, atol=None,
                      raise_on_err=True, ground_truth=None, equal_nan=False, use_uniform=False, rand_type=np.float64):
    """Run the same symbol on several (device, dtype) configurations and compare forward and backward
    against the most precise one (``test_utils.py:1485``)."""
    from . import ndarray as nd
    assert len(ctx_list) > 1
    if isinstance(sym, (list, tuple)):
        syms = list(sym)
    else:
        syms = [sym] * len(ctx_list)
    arg_names = syms[0].list_arguments()
    results = []
    base_args = None
    for s, cfg in zip(syms, ctx_list):
        cfg = dict(cfg)
        ctx = cfg.pop('ctx')
        type_dict = cfg.pop('type_dict', {})
        shapes = {k: v for k, v in cfg.items()}
        arg_shapes, _, aux_shapes = s.infer_shape(**shapes)
        if base_args is None:
            base_args = {n: (np.random.uniform(-scale, scale, size=sh) if use_uniform else
                             np.random.normal(size=sh) * scale).astype(rand_type) for n, sh in zip(arg_names, arg_shapes)}
            if arg_params:
                base_args.update({k: _as_np(v) for k, v in arg_params.items()})
            base_aux = {n: np.ones(sh) if 'var' in n else np.zeros(sh) for n, sh in zip(s.list_auxiliary_states(), aux_shapes)}
            if aux_params:
                base_aux.update({k: _as_np(v) for k, v in aux_params.items()})
        args = {n: nd.array(base_args[n], ctx=ctx, dtype=type_dict.get(n, np.float32)) for n in arg_names}
        grads = {n: nd.zeros(a.shape, ctx=ctx, dtype=a.dtype) for n, a in args.items()}
        aux = {n: nd.array(v, ctx=ctx, dtype=np.float32) for n, v in base_aux.items()}
        ex = s._bind(ctx, args, grads, grad_req, aux)
        outs = ex.forward(is_train=grad_req != 'null')
        if grad_req != 'null':
            ex.backward([nd.array(np.ones(o.shape), ctx=ctx, dtype=o.dtype) for o in outs])
        dts = [np.dtype(a.dtype) for a in args.values()]
        results.append((min(dts, key=lambda d: d.itemsize), [o.asnumpy() for o in outs], {k: g.asnumpy() for k, g in grads.items()}))
    gt_idx = int(np.argmax([r[0].itemsize for r in results]))
    gt = results[gt_idx]
    for i, (dt, outs, grads) in enumerate(results):
        if i == gt_idx:
            continue
        rt = rtol if rtol is not None else max(_DEFAULT_RTOL[dt], _DEFAULT_RTOL[gt[0]])
        at = atol if atol is not None else max(_DEFAULT_ATOL[dt], _DEFAULT_ATOL[gt[0]])
        for o, g in zip(outs, gt[1]):
            assert_almost_equal(o, g, rt, at, ('ctx%d' % i, 'ground truth'), equal_nan)
        if grad_req != 'null':
            for k in grads:
                assert_almost_equal(grads[k], gt[2][k], rt, at, ('grad %s ctx%d' % (k, i), 'ground truth'), equal_nan)
    return [r[1] for r in results]


def compare_optimizer(opt1, opt2, shapes, dtype, w_stype='default', g_stype='default', rtol=1e-4, atol=1e-5,
                      compare_states=True, ntensors=1, ctx=None):
    """Apply two optimizers to identical weights/gradients and compare results (``test_utils.py:2240``)."""
    from . import ndarray as nd
    ctx = ctx or default_device()
    if not isinstance(shapes, list):
        shapes = [shapes] * ntensors if isinstance(shapes, tuple) else shapes
    w1, w2, g1, g2, s1, s2 = [], [], [], [], [], []
    for i, shape in enumerate(shapes):
        w = np.random.uniform(-1, 1, size=shape).astype(dtype)
        g = np.random.uniform(-1, 1, size=shape).astype(dtype)
        w1.append(nd.array(w, ctx=ctx, dtype=dtype)); w2.append(nd.array(w, ctx=ctx, dtype=dtype))
        g1.append(nd.array(g, ctx=ctx, dtype=dtype)); g2.append(nd.array(g, ctx=ctx, dtype=dtype))
        s1.append(opt1.create_state_multi_precision(i, w1[-1]))
        s2.append(opt2.create_state_multi_precision(i, w2[-1]))
    idx = list(range(len(shapes)))
    opt1.update_multi_precision(idx, w1, g1, s1)
    opt2.update_multi_precision(idx, w2, g2, s2)

    def cmp_state(a, b):
        if a is None and b is None:
            return
        if isinstance(a, (tuple, list)):
            for x, y in zip(a, b):
                cmp_state(x, y)
        elif isinstance(a, NDArray):
            assert_almost_equal(a, b, rtol, atol)
    if compare_states:
        for a, b in zip(s1, s2):
            cmp_state(a, b)
    for a, b in zip(w1, w2):
        assert_almost_equal(a, b, rtol, atol)


def check_gluon_hybridize_consistency(net_builder, data_l, numpy_func=None, test_grad=True, rtol=1e-4, atol=1e-4):
    """Same network imperative vs hybridized: outputs (and gradients) must agree (``test_utils.py:2492``)."""
    import tempfile
    saved_out, saved_grad = None, None
    with tempfile.TemporaryDirectory() as d:
        params_file = os.path.join(d, 'net.params')
        for hybridize in (False, True):
            net = net_builder()
            if hybridize:
                net.load_parameters(params_file)
                net.hybridize()
            else:
                net.initialize()
            ins = [x.copy() for x in data_l]
            if test_grad:
                for x in ins:
                    x.attach_grad()
            with autograd.record():
                out = net(*ins)
            if not hybridize:
                net.save_parameters(params_file)
            if test_grad:
                out.backward()
            o = out.asnumpy()
            g = [x.grad.asnumpy() for x in ins] if test_grad else None
            if saved_out is None:
                saved_out, saved_grad = o, g
            else:
                assert_almost_equal(o, saved_out, rtol, atol)
                if test_grad:
                    for a, b in zip(g, saved_grad):
                        assert_almost_equal(a, b, rtol, atol)
    if numpy_func is not None:
        assert_almost_equal(saved_out, numpy_func(*[x.asnumpy() for x in data_l]), rtol, atol)


def chi_square_check(generator, buckets, probs, nsamples=1000000):
    """Chi-square goodness of fit of samples against bucket probabilities (``test_utils.py:2102``)."""
    import scipy.stats as ss
    samples = np.asarray(generator(nsamples)).reshape(-1)
    continuous = isinstance(buckets[0], (tuple, list))
    expected = np.asarray(probs) * samples.size
    obs = np.zeros(len(buckets))
    if continuous:
        for i, (lo, hi) in enumerate(buckets):
            obs[i] = ((samples >= lo) & (samples < hi)).sum()
    else:
        for i, b in enumerate(buckets):
            obs[i] = (samples == b).sum()
    _, p = ss.chisquare(f_obs=obs, f_exp=expected * obs.sum() / expected.sum())
    return p, obs, expected


def verify_generator(generator, buckets, probs, nsamples=1000000, nrepeat=5, success_rate=0.2, alpha=0.05):
    cs_ret_l = [chi_square_check(generator, buckets, probs, nsamples)[0] for _ in range(nrepeat)]
    success_num = (np.array(cs_ret_l) > alpha).sum()
    if success_num < nrepeat * success_rate:
        raise AssertionError('Generator test fails, Chi-square p=%s, obs/expected mismatch' % str(cs_ret_l))
    return cs_ret_l


def gen_buckets_probs_with_ppf(ppf, nbuckets):
    probs = [1.0 / nbuckets for _ in range(nbuckets)]
    buckets = [(ppf(i / float(nbuckets)), ppf((i + 1) / float(nbuckets))) for i in range(nbuckets)]
    return buckets, probs


class DummyIter(object):
    """Repeat the first batch of an iterator forever (``test_utils.py:1939``)."""

    def __init__(self, real_iter):
        self.real_iter = real_iter
        self.provide_data, self.provide_label = real_iter.provide_data, real_iter.provide_label
        self.batch_size = real_iter.batch_size
        self.the_batch = next(real_iter)

    def __iter__(self):
        return self

    def next(self):
        return self.the_batch

    __next__ = next


@contextlib.contextmanager
def environment(*args):
    """``with environment('MXNET_X', '1'):`` or ``with environment({'A': '1', 'B': None}):``."""
    if len(args) == 2:
        kv = {args[0]: args[1]}
    else:
        kv = dict(args[0])
    with env.scope(**kv):
        yield


def list_gpus():
    return list(range(num_gpus()))


def is_cd_run():
    return os.environ.get('CD_JOB', 0) == '1'


def has_tvm_ops():
    return False


def is_op_runnable():
    return True


def get_mnist(path=None):
    raise RuntimeError('MNIST files are not bundled; place the idx files under MXNET_HOME/datasets/mnist')


def new_matrix_with_real_eigvals_2d(n):
    shape = (n, n)
    q = np.ones(shape)
    while 1:
        d = np.random.uniform(-1., 1., shape)
        if np.linalg.matrix_rank(d) == n:
            break
    d = np.diag(np.random.uniform(-1., 1., (n,)))
    q = np.random.uniform(-1., 1., shape)
    while np.linalg.matrix_rank(q) != n:
        q = np.random.uniform(-1., 1., shape)
    return np.matmul(np.matmul(q.T, d), np.linalg.inv(q.T))


def new_sym_matrix_with_real_eigvals_2d(n):
    a = np.random.uniform(-1., 1., (n, n))
    return (a + a.T) / 2


# ---------------------------------------------------------------------------------------------------------
# further helpers of python/mxnet/test_utils.py
# ---------------------------------------------------------------------------------------------------------
def default_numeric_eps():
    """Step of the finite differences of ``check_numeric_gradient`` per dtype."""
    return {np.dtype(np.float16): 1.0 / 2 ** 6, np.dtype(np.float32): 1.0 / 2 ** 9, np.dtype(np.float64): 1.0 / 2 ** 14}


def get_etol(etol=None):
    """Allowed fraction of mismatching elements (0 when not given)."""
    return 0 if etol is None else etol


def shuffle_csr_column_indices(csr):
    """Shuffle the column indices inside every row of a scipy CSR matrix (unordered rows are still a valid matrix)."""
    for i in range(len(csr.indptr) - 1):
        lo, hi = csr.indptr[i], csr.indptr[i + 1]
        part = np.array(csr.indices[lo:hi])
        np.random.shuffle(part)
        csr.indices[lo:hi] = part


def assign_each(the_input, function):
    """``function`` applied to every element, as float64 (a plain copy when ``function`` is None)."""
    if function is None:
        return np.array(the_input)
    return np.vectorize(function, otypes=[np.float64])(np.asarray(the_input))


def assign_each2(input1, input2, function):
    if function is None:
        return np.array(input1)
    assert input1.shape == input2.shape
    return np.vectorize(function, otypes=[np.float64])(np.asarray(input1), np.asarray(input2))


def create_2d_np_tensor(rows, columns, dtype=np.int64):
    """(rows, columns) NumPy-semantics array whose row r is filled with r."""
    from . import numpy as mxnp
    return mxnp.broadcast_to(mxnp.arange(0, rows, dtype=dtype).reshape(rows, 1), (rows, columns))


def create_2d_tensor(rows, columns, dtype=np.int64):
    from . import ndarray as nd
    return nd.broadcast_to(nd.arange(0, rows, dtype=dtype).reshape((rows, 1)), shape=(rows, columns))


def create_vector(size, dtype=np.int64):
    from . import ndarray as nd
    return nd.arange(0, size, dtype=dtype)


def rand_sparse_ndarray(shape, stype, density=None, dtype=None, distribution=None, data_init=None, rsp_indices=None,
                        modifier_func=None, shuffle_csr_indices=False, ctx=None):
    """A random sparse array and its parts: (array, (data, indices)) for ``row_sparse``, (array, (indptr, indices, data))
    for ``csr``.  ``distribution='powerlaw'`` makes row i hold about twice the non-zeros of row i - 1 (csr only)."""
    from . import ndarray as nd
    ctx = ctx or default_device()
    density = np.random.rand() if density is None else density
    dtype = np.dtype(dtype or 'float32')
    distribution = distribution or 'uniform'
    if stype == 'row_sparse':
        assert distribution == 'uniform', 'Distribution %s not supported for row_sparse' % distribution
        if rsp_indices is not None:
            indices = np.asarray(sorted(rsp_indices), dtype=np.int64)
        else:
            indices = np.nonzero(np.random.rand(shape[0]) < density)[0].astype(np.int64)
        if indices.size == 0:
            arr = nd.zeros(shape, ctx=ctx, dtype=dtype).tostype('row_sparse')
            return arr, (np.zeros((0,) + tuple(shape[1:]), dtype=dtype), indices)
        vals = np.random.uniform(-1, 1, (indices.size,) + tuple(shape[1:])).astype(dtype)
        if data_init is not None:
            vals.fill(data_init)
        if modifier_func is not None:
            vals = assign_each(vals, modifier_func).astype(dtype)
        dense = np.zeros(shape, dtype=dtype)
        dense[indices] = vals
        return nd.array(dense, ctx=ctx, dtype=dtype).tostype('row_sparse'), (vals, indices)
    if stype == 'csr':
        assert len(shape) == 2
        import scipy.sparse as sp
        if distribution == 'uniform':
            mat = sp.random(shape[0], shape[1], density=density, format='csr', dtype=np.float64)
        elif distribution == 'powerlaw':
            dense = np.zeros(shape)
            budget = max(int(density * shape[0] * shape[1]), 1)
            per_row = 1
            for r in range(shape[0]):
                n = min(per_row, shape[1], budget)
                if n <= 0:
                    break
                dense[r, np.random.choice(shape[1], n, replace=False)] = np.random.rand(n) + 0.1
                budget -= n
                per_row *= 2
            mat = sp.csr_matrix(dense)
        else:
            raise AssertionError('Distribution not supported: %s' % distribution)
        if data_init is not None:
            mat.data.fill(data_init)
        if modifier_func is not None:
            mat.data = assign_each(mat.data, modifier_func)
        if shuffle_csr_indices:
            shuffle_csr_column_indices(mat)
        arr = nd.sparse.csr_matrix((mat.data.astype(dtype), mat.indices.astype(np.int64), mat.indptr.astype(np.int64)), shape=shape,
                                   ctx=ctx, dtype=dtype)
        return arr, (mat.indptr, mat.indices, mat.data.astype(dtype))
    raise AssertionError('unknown storage type %s' % stype)


def create_sparse_array(shape, stype, data_init=None, rsp_indices=None, dtype=None, modifier_func=None, density=.5,
                        shuffle_csr_indices=False):
    """A sparse array of the given storage type with optional fixed fill value / row set."""
    if stype == 'row_sparse':
        arr, _ = rand_sparse_ndarray(shape, stype, density=density, data_init=data_init, rsp_indices=rsp_indices, dtype=dtype,
                                     modifier_func=modifier_func)
    elif stype == 'csr':
        arr, _ = rand_sparse_ndarray(shape, stype, density=density, data_init=data_init, dtype=dtype, modifier_func=modifier_func,
                                     shuffle_csr_indices=shuffle_csr_indices)
    else:
        raise AssertionError('Unknown storage type: %s' % stype)
    return arr


def create_sparse_array_zd(shape, stype, density, data_init=None, rsp_indices=None, dtype=None, modifier_func=None,
                           shuffle_csr_indices=False):
    """``create_sparse_array`` that also accepts density 0 (an all-zero array of the storage type)."""
    if stype == 'row_sparse' and density == 0.0 and rsp_indices is None:
        rsp_indices = []
    if density == 0.0:
        from . import ndarray as nd
        return nd.zeros(shape, dtype=dtype or 'float32').tostype(stype)
    return create_sparse_array(shape, stype, data_init=data_init, rsp_indices=rsp_indices, dtype=dtype, modifier_func=modifier_func,
                               density=density, shuffle_csr_indices=shuffle_csr_indices)


def rand_coord_2d(x_low, x_high, y_low, y_high):
    return np.random.randint(x_low, x_high, dtype=np.int64), np.random.randint(y_low, y_high, dtype=np.int64)


def checkShapes(a, b):   # pylint: disable=invalid-name
    if a.shape != b.shape:
        raise AssertionError('a.shape = %s and b.shape = %s are not equal' % (a.shape, b.shape))


def locationError(a, b, index, names, maxError=False):   # pylint: disable=invalid-name
    """One line naming where two arrays differ (most)."""
    return 'Location of %serror: %s, %s=%.8f, %s=%.8f' % ('maximum ' if maxError else '', str(index), names[0], a[index], names[1],
                                                           b[index])


def assert_almost_equal_ignore_nan(a, b, rtol=None, atol=None, names=('a', 'b')):
    """``assert_almost_equal`` where positions holding NaN in either array are not compared."""
    a = np.copy(a.asnumpy() if isinstance(a, NDArray) else a)
    b = np.copy(b.asnumpy() if isinstance(b, NDArray) else b)
    nan = np.logical_or(np.isnan(a), np.isnan(b))
    a[nan] = 0
    b[nan] = 0
    assert_almost_equal(a, b, rtol, atol, names)


def check_speed(sym, location=None, ctx=None, N=20, grad_req=None, typ='whole', **kwargs):   # pylint: disable=invalid-name
    """Seconds per iteration of a bound Symbol: forward + backward (``typ='whole'``) or forward only; shapes come from
    ``location`` or from keyword arguments."""
    import time
    from . import ndarray as nd
    ctx = ctx or default_device()
    grad_req = grad_req or 'write'
    if location is None:
        arg_shapes, _, _ = sym.infer_shape(**kwargs)
        location = {n: np.random.normal(size=s, scale=1.0) for n, s in zip(sym.list_arguments(), arg_shapes)}
    args = {k: nd.array(v, ctx=ctx, dtype=getattr(v, 'dtype', 'float32')) for k, v in location.items()}
    grads = {k: nd.zeros(v.shape, ctx=ctx, dtype=v.dtype) for k, v in args.items()} if typ == 'whole' else None
    exe = sym._bind(ctx, args, args_grad=grads, grad_req=grad_req if typ == 'whole' else 'null')
    if typ not in ('whole', 'forward'):
        raise ValueError('typ can only be "whole" or "forward".')

    def step():
        outs = exe.forward(is_train=typ == 'whole')
        if typ == 'whole':
            exe.backward(out_grads=[nd.ones(o.shape, ctx=ctx, dtype=o.dtype) for o in outs])
    step()
    nd.waitall()
    tic = time.time()
    for _ in range(N):
        step()
    nd.waitall()
    return (time.time() - tic) / N


def download(url, fname=None, dirname=None, overwrite=False, retries=5):
    """``gluon.utils.download`` with the argument order of the test helper."""
    from .gluon.utils import download as _download
    path = fname if dirname is None else os.path.join(dirname, fname or url.split('/')[-1])
    return _download(url, path=path, overwrite=overwrite, retries=retries)


def _need_files(directory, names, what):
    missing = [n for n in names if not os.path.exists(os.path.join(directory, n))]
    if missing:
        raise IOError('%s: %s not found under %s and this build does not fetch data sets; place the files there'
                      % (what, ', '.join(missing), directory))


def get_mnist_ubyte(path='data'):
    """The four idx files of MNIST must be present under ``path`` (no download here)."""
    _need_files(path, ['train-images-idx3-ubyte', 'train-labels-idx1-ubyte', 't10k-images-idx3-ubyte', 't10k-labels-idx1-ubyte'],
                'get_mnist_ubyte')


def get_cifar10(path='data'):
    _need_files(os.path.join(path, 'cifar'), ['train.rec', 'test.rec'], 'get_cifar10')


def get_bz2_data(data_dir, data_name, url, data_origin_name):
    """Unpack ``data_origin_name`` (a .bz2 file already in ``data_dir``) to ``data_name`` unless that exists."""
    import bz2
    target = os.path.join(data_dir, data_name)
    if os.path.exists(target):
        return
    src = os.path.join(data_dir, data_origin_name)
    _need_files(data_dir, [data_origin_name], 'get_bz2_data')
    with bz2.BZ2File(src) as fin, open(target, 'wb') as fout:
        fout.write(fin.read())


def get_mnist_iterator(batch_size, input_shape, num_parts=1, part_index=0, path='data'):
    """Training and validation ``MNISTIter`` over the idx files under ``path``."""
    from . import io as mxio
    get_mnist_ubyte(path)
    flat = len(input_shape) != 3
    common = dict(input_shape=input_shape, batch_size=batch_size, flat=flat, num_parts=num_parts, part_index=part_index)
    train = mxio.MNISTIter(image=os.path.join(path, 'train-images-idx3-ubyte'), label=os.path.join(path, 'train-labels-idx1-ubyte'),
                           shuffle=True, **common)
    val = mxio.MNISTIter(image=os.path.join(path, 't10k-images-idx3-ubyte'), label=os.path.join(path, 't10k-labels-idx1-ubyte'),
                         **common)
    return train, val


def same_array(array1, array2):
    """Whether two arrays share memory: a write through one must show in the other."""
    array1[:] += 1
    if not same(array1.asnumpy(), array2.asnumpy()):
        array1[:] -= 1
        return False
    array1[:] -= 1
    return same(array1.asnumpy(), array2.asnumpy())


@contextlib.contextmanager
def discard_stderr():
    """Send everything written to the process's stderr descriptor to the null device inside the block."""
    import sys
    with open(os.devnull, 'w') as sink:
        try:
            fd = sys.stderr.fileno()
            saved = os.dup(fd)
        except (AttributeError, OSError, ValueError):
            yield                                # stderr is not a real file (captured by a test runner)
            return
        try:
            os.dup2(sink.fileno(), fd)
            yield
        finally:
            os.dup2(saved, fd)
            os.close(saved)


def mean_check(generator, mu, sigma, nsamples=1000000):
    """Sample mean of ``generator(nsamples)`` within mu +- 3 sigma / sqrt(n)."""
    sample_mean = np.asarray(generator(nsamples)).mean()
    return (sample_mean > mu - 3 * sigma / np.sqrt(nsamples)) and (sample_mean < mu + 3 * sigma / np.sqrt(nsamples))


def var_check(generator, sigma, nsamples=1000000):
    """Sample variance of ``generator(nsamples)`` within sigma^2 +- 3 sqrt(2 sigma^4 / (n - 1))."""
    sample_var = np.asarray(generator(nsamples)).var(ddof=1)
    half = 3 * np.sqrt(2 * sigma ** 4 / (nsamples - 1))
    return (sample_var > sigma ** 2 - half) and (sample_var < sigma ** 2 + half)


def get_im2rec_path(home_env='MXNET_HOME'):
    """Path of the im2rec tool (``mxnet_b200/tools/im2rec.py``; ``$MXNET_HOME/tools/im2rec.py`` when that is set)."""
    if home_env in os.environ:
        cand = os.path.join(os.environ[home_env], 'tools', 'im2rec.py')
        if os.path.isfile(cand):
            return cand
    cand = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'tools', 'im2rec.py')
    if os.path.isfile(cand):
        return cand
    raise IOError('Could not find path to tools/im2rec.py')


def compare_ndarray_tuple(t1, t2, rtol=None, atol=None):
    """Compare (nested tuples of) arrays element-wise; None entries are skipped."""
    if t1 is None or t2 is None:
        return
    if isinstance(t1, (tuple, list)):
        for s1, s2 in zip(t1, t2):
            compare_ndarray_tuple(s1, s2, rtol, atol)
    else:
        assert_almost_equal(t1, t2, rtol=rtol, atol=atol)


def compare_optimizer_noise_seeded(opt1, opt2, shapes, dtype, noise_seed, w_stype='default', g_stype='default', rtol=1e-4,
                                   atol=1e-5, compare_states=True):
    """``compare_optimizer`` for optimizers that draw noise in their update (SGLD): the generator is seeded with
    ``noise_seed`` before each of the two updates so both see the same draws."""
    from . import ndarray as nd
    from . import random as mxrandom
    ctx = default_device()
    w1, w2, g1, g2, s1, s2 = [], [], [], [], [], []
    for i, shape in enumerate(shapes):
        w = np.random.uniform(-1, 1, size=shape).astype(dtype)
        g = np.random.uniform(-1, 1, size=shape).astype(dtype)
        w1.append(nd.array(w, ctx=ctx, dtype=dtype)); w2.append(nd.array(w, ctx=ctx, dtype=dtype))   # noqa: E702
        g1.append(nd.array(g, ctx=ctx, dtype=dtype)); g2.append(nd.array(g, ctx=ctx, dtype=dtype))   # noqa: E702
        s1.append(opt1.create_state_multi_precision(i, w1[-1]))
        s2.append(opt2.create_state_multi_precision(i, w2[-1]))
    if compare_states:
        compare_ndarray_tuple(tuple(s1), tuple(s2))
    idx = list(range(len(shapes)))
    mxrandom.seed(noise_seed)
    opt1.update_multi_precision(idx, w1, g1, s1)
    mxrandom.seed(noise_seed)
    opt2.update_multi_precision(idx, w2, g2, s2)
    if compare_states:
        compare_ndarray_tuple(tuple(s1), tuple(s2), rtol=rtol, atol=atol)
    for a, b in zip(w1, w2):
        assert_almost_equal(a, b, rtol=rtol, atol=atol)


def same_symbol_structure(sym1, sym2):
    """Whether the two graphs have the same operator at every node position."""
    import json
    n1, n2 = json.loads(sym1.tojson())['nodes'], json.loads(sym2.tojson())['nodes']
    return all(a['op'] == b['op'] for a, b in zip(n1, n2))


def collapse_sum_like(a, shape):
    """Sum ``a`` over the axes along which an array of ``shape`` was broadcast to give ``a`` (the gradient of a
    broadcast)."""
    assert len(a.shape) >= len(shape)
    if np.prod(shape) == 0 or a.size == 0:
        return np.zeros(shape, dtype=a.dtype)
    diff = len(a.shape) - len(shape)
    axes = [i for i in range(len(a.shape)) if i < diff or shape[i - diff] != a.shape[i]]
    return np.sum(a, axis=tuple(axes)).reshape(shape)


def new_matrix_with_real_eigvals_nd(shape):
    """Random batch of square matrices with real eigenvalues (D P D^-1 form)."""
    n = int(np.prod(shape[:-2])) if len(shape) > 2 else 1
    return np.array([new_matrix_with_real_eigvals_2d(shape[-1]) for _ in range(n)]).reshape(shape)


def new_matrix_with_real_eigvals_2d(n):
    """One n x n matrix with real eigenvalues: Q diag(d) Q^-1 with a random invertible Q."""
    shape = (n, n)
    q = np.ones(shape)
    while 1:
        q = np.random.uniform(-1, 1, shape)
        if np.linalg.cond(q, 2) < 3:
            break
    d = np.diag(np.random.uniform(-1.0, 1.0, shape[-1]))
    return q.dot(d).dot(np.linalg.inv(q))


def new_orthonormal_matrix_2d(n):
    """A random n x n orthonormal matrix (Q of a QR factorisation)."""
    x = np.random.randn(n, n)
    x_trans = x.T
    sym_mat = np.matmul(x_trans, x)
    return np.linalg.qr(sym_mat)[0]


def new_sym_matrix_with_real_eigvals_2d(n):
    """Symmetric n x n matrix Q diag(d) Q^T."""
    q = new_orthonormal_matrix_2d(n)
    d = np.diag(np.random.uniform(-1.0, 1.0, n))
    return q.dot(d).dot(q.T)


def new_sym_matrix_with_real_eigvals_nd(shape):
    n = int(np.prod(shape[:-2])) if len(shape) > 2 else 1
    return np.array([new_sym_matrix_with_real_eigvals_2d(shape[-1]) for _ in range(n)]).reshape(shape)


# ---- names the reference's test_utils re-exports or defines beside its checks ------------------------------------------
from .util import get_cuda_compute_capability, get_rtc_compile_opts, getenv, setenv, use_np, use_np_default_dtype   # noqa: E402,F401
from .runtime import Features   # noqa: E402,F401
from .symbol import Symbol   # noqa: E402,F401


def get_max_supported_compute_capability():
    """Highest compute capability the toolkit used for run-time compilation can target (``major * 10 + minor``)."""
    return 100


def get_dtype_name(dtype):
    """``'float32'`` for ``np.float32`` / ``'float32'`` / ``np.dtype('float32')``."""
    import numpy as _np
    return _np.dtype(dtype).name


def np_symbol(sym):
    """The same graph under NumPy semantics (``Symbol.as_np_ndarray``)."""
    return sym.as_np_ndarray()


# Scripts written against the reference do ``from mxnet.test_utils import *`` and then use ``mx``, ``nd``, ``np`` (NumPy), ``sym``
# that the reference module happens to import at its top; the same names are provided here.
import sys as _sys   # noqa: E402
mx = _sys.modules[__name__.rsplit('.', 1)[0]]   # the package itself
from . import ndarray as nd, symbol as sym   # noqa: E402,F401
from .ndarray import array   # noqa: E402,F401
from .symbol import Symbol   # noqa: E402,F401,F811
import numpy.testing as npt, numpy.random as rnd   # noqa: E402,F401

"""Registry-wide operator sweep: every registered operator name is invoked on generated inputs and checked.

The reference checks operators one by one against NumPy with ``check_numeric_gradient`` / ``check_consistency``
(python/mxnet/test_utils.py:1038, 1485; tests/python/unittest/test_operator.py, test_numpy_op.py).  This module does the
same for the whole registry at once:

* inputs come from a per-operator entry of ``SPECS`` (shapes and attributes the operator needs) or, without one, from a list
  of generic candidates (unary / binary float tensors, an NCHW batch, square matrices, integer and boolean tensors);
* every operator must run, give the same result when run again (random operators excepted), match NumPy where a NumPy
  function of the same name exists (``_npi_*`` names), and its autograd gradient must agree with central differences in
  float64 where the operator is differentiable at the sampled point;
* ``EXCLUDED`` lists the names that cannot be called in isolation, each with its reason; the last test asserts that at least
  95 % of all names are exercised.

The GPU variant re-runs the same cases on ``cuda:0`` and compares with the CPU result.
"""
import re
import warnings

import numpy as np
import pytest
import torch

import mxnet_b200 as mx  # noqa: F401  (registers the operators)
from mxnet_b200.ops import registry

import inspect

from _sweep_specs import SPECS, EXCLUDED, NO_GRADCHECK, NO_NUMPY, RANDOM_PATTERN, GRAD_INPUTS, NO_DEVICE_COMPARE

warnings.filterwarnings('ignore')


def _f(*shape, lo=0.1, hi=0.9, dtype=torch.float32, gen=None):
    return torch.rand(*shape, generator=gen, dtype=torch.float64).mul(hi - lo).add(lo).to(dtype)


def generic_candidates(n, gen):
    """Input lists tried in order for an operator without a spec."""
    out = [[_f(3, 4, gen=gen) for _ in range(n)],
           [_f(3, 4, lo=1.1, hi=2.1, gen=gen) for _ in range(n)],
           [_f(2, 3, 8, 8, gen=gen) for _ in range(n)],
           [_f(4, 4, gen=gen) for _ in range(n)],
           [torch.randint(0, 3, (3, 4), generator=gen) for _ in range(n)],
           [_f(3, 4, gen=gen)] + [torch.randint(0, 3, (3, 4), generator=gen) for _ in range(n - 1)],
           [_f(3, 4, gen=gen)] + [torch.randint(0, 3, (3,), generator=gen) for _ in range(n - 1)],
           [_f(6, gen=gen) for _ in range(n)],
           [_f(3, 4, gen=gen) > 0.5 for _ in range(n)]]
    return out


def _unique_ops():
    seen, out = {}, []
    for name in registry.list_ops():
        op = registry.get(name)
        if id(op) not in seen:
            seen[id(op)] = [name]
            out.append((name, op))
        else:
            seen[id(op)].append(name)
    return out, seen


_OPS, _NAMES = _unique_ops()


def _names_of(op):
    return _NAMES[id(op)]


def _spec_for(op):
    for n in _names_of(op):
        if n in SPECS:
            return SPECS[n]
    return None


def _excluded(op):
    for n in _names_of(op):
        if n in EXCLUDED:
            return EXCLUDED[n]
    return None


def _seed(name):
    import zlib
    return zlib.crc32(name.encode()) % (2 ** 31)


def make_case(name, op):
    """(tensors, attrs) on which the operator runs, or raises the first error when nothing works."""
    gen = torch.Generator().manual_seed(_seed(name))
    spec = _spec_for(op)
    if spec is not None:
        tensors, attrs = spec(gen)
        return list(tensors), dict(attrs)
    n = max(1, len(op.inputs))
    counts = [2, 3, 1] if op.variadic else list(range(n, 0, -1))
    attrs = {}
    try:
        if 'scalar' in inspect.signature(op.fn).parameters:
            attrs = {'scalar': 2.0}                      # the default 0 puts division-like operators on their pole
    except (TypeError, ValueError):
        pass
    first = None
    for k in counts:
        for cand in generic_candidates(k, gen):
            try:
                with torch.no_grad():
                    res = _flat(op.fn(*[c.clone() for c in cand], **attrs))
                if any(r.is_floating_point() and not bool(torch.isfinite(r).all()) for r in res):
                    raise ValueError('non-finite output: outside the domain of the operator')
                return cand, attrs
            except Exception as e:   # pylint: disable=broad-except
                first = first or e
    raise AssertionError('no generated input runs %s%s: %s: %s' % (name, op.inputs, type(first).__name__, first))


def _flat(res):
    if isinstance(res, torch.Tensor):
        return [res]
    if isinstance(res, (tuple, list)):
        return [r for r in res if isinstance(r, torch.Tensor)]
    return []


def _is_random(op):
    return any(re.search(RANDOM_PATTERN, n) for n in _names_of(op))


def _numpy_counterpart(op):
    for n in _names_of(op):
        if n in NO_NUMPY:
            return None
    for n in _names_of(op):
        m = re.match(r'^_np[i]?_(\w+)$', n)
        if m and hasattr(np, m.group(1)) and callable(getattr(np, m.group(1))):
            return getattr(np, m.group(1))
    return None


def _close(a, b, rtol=1e-4, atol=1e-5):
    a, b = np.asarray(a), np.asarray(b)
    if a.shape != b.shape:
        return False
    if a.dtype == bool or b.dtype == bool:
        return bool((a.astype(bool) == b.astype(bool)).all())
    return bool(np.allclose(a.astype('float64'), b.astype('float64'), rtol=rtol, atol=atol, equal_nan=True))


def check_gradient(name, op, tensors, attrs):
    """Autograd against central differences in float64, on a random projection of the outputs, at three coordinates of
    every floating-point input.  Returns None (checked), or a string saying why the check does not apply."""
    which = None
    for n in _names_of(op):
        which = GRAD_INPUTS.get(n, which)
    if not tensors or not all(t.is_floating_point() for i, t in enumerate(tensors) if which is None or i in which):
        return 'non-float inputs'
    xs = [t.detach().double().clone().requires_grad_(which is None or i in which) if t.is_floating_point() else t.clone()
          for i, t in enumerate(tensors)]
    try:
        every = _flat(op.fn(*xs, **attrs))
        used = [k for k, o in enumerate(every) if o.is_floating_point() and o.requires_grad]
        outs = [every[k] for k in used]
    except Exception as e:   # pylint: disable=broad-except
        return 'float64 unsupported: %s' % type(e).__name__
    if not outs:
        return 'no differentiable output'
    gen = torch.Generator().manual_seed(_seed(name) + 1)
    ws = [torch.rand(o.shape, generator=gen, dtype=torch.float64) + 0.5 for o in outs]
    loss = sum((o * w).sum() for o, w in zip(outs, ws))
    diff = [i for i, x in enumerate(xs) if x.requires_grad]
    try:
        grads = dict(zip(diff, torch.autograd.grad(loss, [xs[i] for i in diff], allow_unused=True)))
    except RuntimeError as e:
        return 'no derivative: %s' % str(e)[:60]

    def f(vals):
        with torch.no_grad():
            every_ = _flat(op.fn(*vals, **attrs))
            return float(sum((every_[k].double() * w).sum() for k, w in zip(used, ws)))

    def mismatch(eps, rtol, atol):
        for i in diff:
            x, g = xs[i], grads[i]
            for j in torch.randperm(x.numel(), generator=torch.Generator().manual_seed(_seed(name) + 2 + i))[:3].tolist():
                hi = [v.detach().clone() for v in xs]
                lo = [v.detach().clone() for v in xs]
                hi[i].reshape(-1)[j] += eps
                lo[i].reshape(-1)[j] -= eps
                num = (f(hi) - f(lo)) / (2 * eps)
                ana = 0.0 if g is None else float(g.reshape(-1)[j])
                if not abs(num - ana) <= atol + rtol * max(abs(num), abs(ana)):
                    return '%s: d/d input %d [%d]: autograd %.8g, finite difference %.8g (step %g)' % (name, i, j, ana, num, eps)
        return None
    # strict first; an operator that computes in fp32 internally only supports a coarse difference quotient, which still
    # tells a wrong gradient (a missing factor, a wrong sign) from a right one
    first = mismatch(1e-6, 1e-3, 1e-4)
    if first is not None:
        second = mismatch(1e-2, 5e-2, 5e-3)
        assert second is None, first + ' / ' + second
    return None


def run_checks(name, op, device='cpu'):
    tensors, attrs = make_case(name, op)
    with torch.no_grad():
        res = _flat(op.fn(*[t.clone() for t in tensors], **attrs))
        again = _flat(op.fn(*[t.clone() for t in tensors], **attrs))
    assert len(res) == len(again)
    if not _is_random(op):
        for a, b in zip(res, again):
            assert a.shape == b.shape and a.dtype == b.dtype
            assert _close(a.cpu().numpy(), b.cpu().numpy(), 0, 0), '%s is not deterministic' % name
    fn_np = _numpy_counterpart(op)
    if fn_np is not None and not attrs and not _is_random(op):
        try:
            expect = fn_np(*[t.numpy() for t in tensors])
        except Exception:   # pylint: disable=broad-except
            expect = None
        if isinstance(expect, np.ndarray) and len(res) == 1 and expect.shape == tuple(res[0].shape):
            assert _close(res[0].numpy(), expect, 1e-4, 1e-5), '%s differs from numpy.%s' % (name, fn_np.__name__)
    if not _is_random(op) and not any(n in NO_GRADCHECK for n in _names_of(op)):
        check_gradient(name, op, tensors, attrs)
    if device != 'cpu':
        with torch.no_grad():
            dres = _flat(op.fn(*[t.clone().to(device) for t in tensors], **attrs))
        assert len(dres) == len(res)
        if not _is_random(op) and not any(n in NO_DEVICE_COMPARE for n in _names_of(op)):
            for a, b in zip(res, dres):
                assert _close(a.numpy(), b.cpu().numpy(), 2e-3, 2e-4), '%s: GPU result differs from CPU' % name
    return True


_CASES = [(n, op) for n, op in _OPS if _excluded(op) is None]


@pytest.mark.parametrize('name', [n for n, _ in _CASES])
def test_operator(name):
    run_checks(name, registry.get(name))


@pytest.mark.gpu
@pytest.mark.parametrize('name', [n for n, _ in _CASES])
def test_operator_gpu_matches_cpu(name):
    run_checks(name, registry.get(name), device='cuda:0')


def test_sweep_covers_the_registry():
    """At least 95 % of all registered names (aliases included) are exercised; the rest are listed with a reason."""
    total = len(registry.list_ops())
    covered = sum(len(_names_of(op)) for _, op in _CASES)
    assert covered >= 0.95 * total, '%d of %d names' % (covered, total)
    for n, why in EXCLUDED.items():
        assert registry.has(n) and why

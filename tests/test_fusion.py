"""Pointwise fusion pass: grouping, acyclicity, equivalence of the fused graph, generated CUDA source (compiled with
NVRTC for sm_100a without a device), and on a GPU the generated kernels against the unfused graph."""
import numpy as np
import pytest
import torch

import mxnet_b200 as mx
from mxnet_b200 import nd, autograd
from mxnet_b200.symbol import fusion
from mxnet_b200.symbol.symbol import _topo


def _ops(sym):
    return [n.op.name for n in _topo(sym._outputs) if n.op is not None]


def _graph():
    x, b, y = mx.sym.var('x'), mx.sym.var('b'), mx.sym.var('y')
    h = mx.sym.LeakyReLU(mx.sym.broadcast_add(x, b), act_type='gelu')
    o = h * 2.0 + mx.sym.tanh(y)
    z = mx.sym.FullyConnected(o, num_hidden=8, name='fc')
    w = mx.sym.sigmoid(z) * mx.sym.exp(-z)
    return mx.sym.Group([w, o])


def _feed(rng, dtype=torch.float32, device='cpu'):
    f = {'x': rng.randn(6, 16), 'b': rng.randn(16), 'y': rng.randn(6, 16), 'fc_weight': rng.randn(8, 16) * 0.2,
         'fc_bias': rng.randn(8)}
    return {k: torch.tensor(v, dtype=dtype, device=device) for k, v in f.items()}


def test_groups_are_contracted_and_results_unchanged():
    s = _graph()
    f = fusion.fuse_pointwise(s)
    assert _ops(f) == ['_FusedOp', 'FullyConnected', '_FusedOp']
    assert f.list_arguments() == s.list_arguments()
    feed = _feed(np.random.RandomState(0))
    for a, b in zip(s._run(feed), f._run(feed)):
        torch.testing.assert_close(a, b)
    # gradients flow through the operator-by-operator evaluation of a group
    feed = {k: v.requires_grad_(True) for k, v in feed.items()}
    outs = f._run(feed)
    (outs[0].sum() + outs[1].sum()).backward()
    assert all(v.grad is not None for v in feed.values())


def test_no_cycle_through_an_outside_node():
    # a -> (exp) -> FC -> (+) and a -> (exp) -> (+): exp and + may not fuse around the FullyConnected between them
    a = mx.sym.var('a')
    e = mx.sym.exp(a)
    t = mx.sym.tanh(e)
    fc = mx.sym.FullyConnected(t, num_hidden=4, no_bias=True, name='fc')
    out = mx.sym.relu(fc + 1.0) + mx.sym.sum(t)
    f = fusion.fuse_pointwise(out)
    ops = _ops(f)
    assert ops.count('_FusedOp') == 2 and 'FullyConnected' in ops
    feed = {'a': torch.randn(3, 4), 'fc_weight': torch.randn(4, 4)}
    torch.testing.assert_close(out._run(feed)[0], f._run(feed)[0])
    # a diamond inside one group is fine; a path that leaves and re-enters is not
    d = mx.sym.var('d')
    p = mx.sym.sigmoid(d)
    q = mx.sym.dot(p, p)                     # outside node fed by the group
    r = p * q                                # would close a cycle if p and r were fused
    g = fusion.fuse_pointwise(mx.sym.tanh(r))
    feed = {'d': torch.randn(4, 4)}
    torch.testing.assert_close(mx.sym.tanh(r)._run(feed)[0], g._run(feed)[0])


def test_single_operators_and_unknown_operators_stay():
    x = mx.sym.var('x')
    s = mx.sym.softmax(mx.sym.relu(x))
    assert fusion.fuse_pointwise(s) is s
    s = mx.sym.LeakyReLU(mx.sym.relu(x), act_type='prelu', gamma=mx.sym.var('g'))
    assert '_FusedOp' not in _ops(fusion.fuse_pointwise(s))


@pytest.mark.parametrize('backward', [False, True])
def test_generated_source_compiles_for_sm100a(backward):
    pytest.importorskip('cuda')
    s = _graph()
    f = fusion.fuse_pointwise(s)
    groups = [n.attrs['group'] for n in _topo(f._outputs) if n.op is not None and n.op.name == '_FusedOp']
    g = groups[0]
    assert g.nin == 3 and len(g.outputs) == 1
    for vec in (1, 4, 8):
        src = fusion.kernel_source(g, [torch.float16, torch.bfloat16, torch.float32], (fusion.FULL, fusion.LAST, fusion.ONE),
                                   (torch.float16,), vec, backward, [True, True, False])
        assert ('fused_bwd' if backward else 'fused_fwd') in src
        assert len(fusion.compile_cubin(src)) > 1000


def test_every_template_compiles_and_matches_the_operator_on_the_host():
    """Each template's forward expression, evaluated through the generated source's arithmetic restated in Python
    is out of reach without a device; what can be checked here is that every template yields source NVRTC accepts."""
    pytest.importorskip('cuda')
    x, y = mx.sym.var('x'), mx.sym.var('y')
    from mxnet_b200.ops import registry
    outs = []
    for name, (fwd, bwd, accepts) in sorted(fusion.templates().items()):
        op = registry.get(name)
        if name in ('Activation',):
            for act in ('relu', 'sigmoid', 'tanh', 'softrelu', 'softsign', 'log_sigmoid', 'mish'):
                outs.append(mx.sym.Activation(x, act_type=act))
        elif name == 'LeakyReLU':
            for act in ('leaky', 'elu', 'selu', 'gelu'):
                outs.append(mx.sym.LeakyReLU(x, act_type=act, slope=0.1))
        elif name == 'clip':
            outs.append(mx.sym.clip(x, a_min=-1.0, a_max=2.0))
        elif name in ('Cast', 'amp_cast'):
            outs.append(getattr(mx.sym, name)(x, dtype='float16'))
        elif len(op.inputs) == 2:
            outs.append(getattr(mx.sym.op, name)(x, y))
        elif 'scalar' in name:
            outs.append(getattr(mx.sym.op, name)(x, scalar=1.5))
        else:
            outs.append(getattr(mx.sym.op, name)(x))
    assert len(outs) > 70
    total = outs[0]
    for o in outs[1:]:
        total = total + mx.sym.Cast(o, dtype='float32')
    f = fusion.fuse_pointwise(total)
    groups = [n.attrs['group'] for n in _topo(f._outputs) if n.op is not None and n.op.name == '_FusedOp']
    assert sum(len(g.nodes) for g in groups) >= len(outs)
    for g in groups:
        for backward in (False, True):
            src = fusion.kernel_source(g, [torch.float32] * g.nin, (fusion.FULL,) * g.nin, (torch.float32,) * len(g.outputs), 4,
                                       backward, [True] * g.nin)
            fusion.compile_cubin(src)


@pytest.mark.gpu
@pytest.mark.parametrize('dtype', [torch.float32, torch.float16])
def test_generated_kernels_match_the_unfused_graph(dtype):
    from mxnet_b200 import env
    s = _graph()
    rng = np.random.RandomState(1)
    results = []
    for fuse in ('1', '0'):
        with env.scope('MXNET_USE_FUSION', fuse):
            feed = {k: v.requires_grad_(True) for k, v in _feed(rng if fuse == '1' else np.random.RandomState(1), dtype, 'cuda').items()}
            before = fusion.stats['kernel_calls']
            outs = mx.sym.Group(list(s))._run(feed)
            (outs[0].float().sum() + (outs[1].float() ** 2).sum()).backward()
            if fuse == '1':
                assert fusion.stats['kernel_calls'] >= before + 4       # two groups, forward and backward
            results.append([o.detach().float().cpu() for o in outs] + [feed[k].grad.float().cpu() for k in sorted(feed)])
    tol = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    for a, b in zip(*results):
        torch.testing.assert_close(a, b, **tol)


@pytest.mark.gpu
def test_every_template_on_the_gpu_against_the_operators():
    """One fused node per operator pair (the operator followed by a scale): values and gradients against the same
    operators run one by one."""
    from mxnet_b200 import env
    from mxnet_b200.ops import registry
    x, y = mx.sym.var('x'), mx.sym.var('y')
    torch.manual_seed(0)
    xv = (torch.rand(5, 24, device='cuda') * 0.8 + 0.1)           # inside every domain used here (0.1 .. 0.9)
    yv = (torch.rand(5, 24, device='cuda') * 0.8 + 0.1)
    cases = []
    for name in sorted(fusion.templates()):
        op = registry.get(name)
        if name == 'Activation':
            cases += [(name + act, mx.sym.Activation(x, act_type=act)) for act in ('relu', 'sigmoid', 'tanh', 'softrelu', 'softsign',
                                                                                   'log_sigmoid', 'mish')]
        elif name == 'LeakyReLU':
            cases += [(name + act, mx.sym.LeakyReLU(x - 0.5, act_type=act, slope=0.1)) for act in ('leaky', 'elu', 'selu', 'gelu')]
        elif name == 'clip':
            cases.append((name, mx.sym.clip(x, a_min=0.3, a_max=0.7)))
        elif name in ('Cast', 'amp_cast'):
            cases.append((name, getattr(mx.sym, name)(x, dtype='float32')))
        elif name == 'arccosh':
            cases.append((name, mx.sym.arccosh(x + 1.5)))
        elif len(op.inputs) == 2:
            cases.append((name, getattr(mx.sym.op, name)(x, y)))
        elif 'scalar' in name:
            cases.append((name, getattr(mx.sym.op, name)(x, scalar=1.5)))
        else:
            cases.append((name, getattr(mx.sym.op, name)(x)))
    for name, s in cases:
        s = s * 3.0
        res = []
        for fuse in ('1', '0'):
            with env.scope('MXNET_USE_FUSION', fuse):
                feed = {'x': xv.clone().requires_grad_(True)}
                if 'y' in s.list_arguments():
                    feed['y'] = yv.clone().requires_grad_(True)
                calls = fusion.stats['kernel_calls']
                out = mx.sym.Group([s])._run(feed)[0]
                if out.requires_grad:             # BlockGrad and friends: nothing to differentiate when run one by one
                    out.sum().backward()
                if fuse == '1':
                    assert fusion.stats['kernel_calls'] == calls + 2, name
                res.append([out.detach()] + [v.grad if v.grad is not None else torch.zeros_like(v) for v in feed.values()])
        for a, b in zip(*res):
            torch.testing.assert_close(a, b, rtol=2e-4, atol=2e-5, msg=lambda m, n=name: '%s: %s' % (n, m))


def test_hybridize_with_the_fusion_backend_runs_the_partitioned_graph():
    from mxnet_b200.gluon import nn

    class Net(mx.gluon.HybridBlock):
        def __init__(self):
            super().__init__()
            self.fc1, self.fc2 = nn.Dense(16, in_units=8), nn.Dense(4, in_units=16)
            self.bn = nn.BatchNorm(in_channels=16)

        def forward(self, x):
            h = self.bn(self.fc1(x))
            h = mx.npx.activation(h, 'tanh') * 0.5 + mx.np.exp(-mx.np.square(h))
            return self.fc2(h), h

    mx.npx.set_np()
    try:
        net = Net()
        net.initialize()
        x = mx.np.array(np.random.RandomState(0).randn(5, 8).astype('float32'))
        ref_eval = [o.asnumpy() for o in net(x)]
        with autograd.record():
            ref = net(x)
            loss = ref[0].sum() + ref[1].sum()
        loss.backward()
        ref_train = [o.asnumpy() for o in ref]
        ref_grad = net.fc1.weight.grad().asnumpy().copy()
        ref_mean = net.bn.running_mean.data().asnumpy().copy()

        def reset_stats():
            net.bn.running_mean.set_data(mx.np.zeros(16))
            net.bn.running_var.set_data(mx.np.ones(16))

        reset_stats()
        net.hybridize(backend='pointwise_fusion')
        for _ in range(2):                       # first call builds, second runs the partitioned graph
            out = net(x)
        assert any(n.op is not None and n.op.name == '_FusedOp' for n in _topo(net._partitioned._outputs))
        for a, b in zip(out, ref_eval):
            np.testing.assert_allclose(a.asnumpy(), b, rtol=1e-5, atol=1e-6)
        reset_stats()
        with autograd.record():
            out = net(x)
            loss = out[0].sum() + out[1].sum()
        loss.backward()
        for a, b in zip(out, ref_train):
            np.testing.assert_allclose(a.asnumpy(), b, rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(net.fc1.weight.grad().asnumpy(), ref_grad, rtol=1e-4, atol=1e-6)
        np.testing.assert_allclose(net.bn.running_mean.data().asnumpy(), ref_mean, rtol=1e-5, atol=1e-7)
    finally:
        mx.npx.reset_np()


@pytest.mark.gpu
def test_hybridized_block_with_fusion_backend_on_the_gpu():
    from mxnet_b200.gluon import nn

    class Net(mx.gluon.HybridBlock):
        def __init__(self):
            super().__init__()
            self.fc1, self.fc2 = nn.Dense(64, in_units=32), nn.Dense(8, in_units=64)

        def forward(self, x):
            h = self.fc1(x)
            h = mx.npx.activation(h, 'tanh') * 0.5 + mx.np.exp(-mx.np.square(h))
            return self.fc2(h)

    mx.npx.set_np()
    try:
        ctx = mx.gpu(0)
        net = Net()
        net.initialize(ctx=ctx)
        x = mx.np.array(np.random.RandomState(0).randn(16, 32).astype('float32'), ctx=ctx)
        with autograd.record():
            ref = net(x)
            ref.sum().backward()
        ref_out, ref_grad = ref.asnumpy(), net.fc1.weight.grad().asnumpy().copy()
        net.hybridize(backend='pointwise_fusion')
        net(x)
        before = fusion.stats['kernel_calls']
        with autograd.record():
            out = net(x)
            out.sum().backward()
        assert fusion.stats['kernel_calls'] >= before + 2            # the fused group ran forward and backward
        np.testing.assert_allclose(out.asnumpy(), ref_out, rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(net.fc1.weight.grad().asnumpy(), ref_grad, rtol=1e-3, atol=1e-4)
    finally:
        mx.npx.reset_np()


def _two_output_graph():
    x, b, s = mx.sym.var('x'), mx.sym.var('b'), mx.sym.var('s')
    h = mx.sym.broadcast_add(x, b)                       # bias over the last axis
    u = mx.sym.broadcast_mul(mx.sym.tanh(h), s)          # one-element scale
    v = mx.sym.exp(-mx.sym.square(h)) + u                # reads u inside the group
    return mx.sym.Group([mx.sym.sum(u, axis=1), mx.sym.FullyConnected(v, num_hidden=3, no_bias=True, name='fc')])


def test_group_with_two_outputs_and_broadcast_inputs():
    g = _two_output_graph()
    f = fusion.fuse_pointwise(g)
    groups = [n.attrs['group'] for n in _topo(f._outputs) if n.op is not None and n.op.name == '_FusedOp']
    assert len(groups) == 1 and len(groups[0].outputs) == 2 and groups[0].nin == 3
    rng = np.random.RandomState(0)
    feed = {'x': torch.tensor(rng.randn(4, 6), dtype=torch.float32), 'b': torch.tensor(rng.randn(6), dtype=torch.float32),
            's': torch.tensor([1.5]), 'fc_weight': torch.tensor(rng.randn(3, 6), dtype=torch.float32)}
    for a, b in zip(g._run(feed), f._run(feed)):
        torch.testing.assert_close(a, b)


@pytest.mark.gpu
@pytest.mark.parametrize('rows,cols', [(64, 96), (7, 13)])       # vector and scalar code paths
def test_two_output_kernels_with_bias_and_scalar_inputs_on_the_gpu(rows, cols):
    from mxnet_b200 import env
    g = _two_output_graph()
    rng = np.random.RandomState(1)
    base = {'x': rng.randn(rows, cols), 'b': rng.randn(cols), 's': np.array([1.5]), 'fc_weight': rng.randn(3, cols) * 0.3}
    res = []
    for fuse in ('1', '0'):
        with env.scope('MXNET_USE_FUSION', fuse):
            feed = {k: torch.tensor(v, dtype=torch.float32, device='cuda').requires_grad_(True) for k, v in base.items()}
            calls = fusion.stats['kernel_calls']
            outs = mx.sym.Group(list(g))._run(feed)
            (outs[0].sum() + (outs[1] ** 2).sum()).backward()
            if fuse == '1':
                assert fusion.stats['kernel_calls'] == calls + 2
            res.append([o.detach().cpu() for o in outs] + [feed[k].grad.cpu() for k in sorted(feed)])
    for a, b in zip(*res):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-4)

"""Symbol graphs: composition, attributes, JSON round trip, shape/type inference, executors (reference:
tests/python/unittest/test_symbol.py, test_executor.py, test_infer_shape.py)."""
import json

import numpy as np
import pytest

import mxnet_b200 as mx
from mxnet_b200 import nd, sym
from mxnet_b200.test_utils import assert_almost_equal, same


def _mlp():
    data = sym.Variable('data')
    fc1 = sym.FullyConnected(data=data, name='fc1', num_hidden=16)
    act = sym.Activation(data=fc1, name='relu1', act_type='relu')
    fc2 = sym.FullyConnected(data=act, name='fc2', num_hidden=4)
    return sym.SoftmaxOutput(data=fc2, name='softmax')


def test_compose_and_list():
    net = _mlp()
    assert net.list_arguments() == ['data', 'fc1_weight', 'fc1_bias', 'fc2_weight', 'fc2_bias', 'softmax_label']
    assert net.list_outputs() == ['softmax_output']
    assert net.name == 'softmax'
    internals = net.get_internals()
    assert 'fc1_output' in internals.list_outputs()
    fc1 = internals['fc1_output']
    assert fc1.list_arguments() == ['data', 'fc1_weight', 'fc1_bias']
    children = net.get_children()
    assert children.list_outputs() == ['fc2_output', 'softmax_label']


def test_json_round_trip_and_format():
    net = _mlp()
    js = net.tojson()
    graph = json.loads(js)
    assert set(graph) >= {'nodes', 'arg_nodes', 'node_row_ptr', 'heads', 'attrs'}
    assert graph['attrs']['mxnet_version'][0] == 'int'
    node = [n for n in graph['nodes'] if n['name'] == 'fc1'][0]
    assert node['op'] == 'FullyConnected' and node['attrs'] == {'num_hidden': '16'}
    assert node['inputs'] == [[0, 0, 0], [1, 0, 0], [2, 0, 0]]
    assert [graph['nodes'][i]['op'] for i in graph['arg_nodes']] == ['null'] * len(graph['arg_nodes'])
    back = sym.load_json(js)
    assert back.list_arguments() == net.list_arguments()
    assert json.loads(back.tojson())['nodes'] == graph['nodes']


def test_attribute_stringification():
    data = sym.Variable('data')
    conv = sym.Convolution(data=data, kernel=(3, 3), num_filter=8, pad=(1, 1), no_bias=True, name='conv')
    pool = sym.Pooling(data=conv, kernel=(2, 2), stride=(2, 2), pool_type='max', name='pool')
    graph = json.loads(pool.tojson())
    attrs = {n['name']: n.get('attrs', {}) for n in graph['nodes']}
    assert attrs['conv'] == {'kernel': '(3, 3)', 'no_bias': 'True', 'num_filter': '8', 'pad': '(1, 1)'}
    assert attrs['pool']['pool_type'] == 'max' and attrs['pool']['stride'] == '(2, 2)'
    back = sym.load_json(pool.tojson())
    arg_shapes, out_shapes, _ = back.infer_shape(data=(2, 3, 8, 8))
    assert out_shapes == [(2, 8, 4, 4)]


def test_load_reference_style_json():
    """A graph written the way the reference serialises it (string attrs, legacy `param`/`attr` keys accepted)."""
    js = json.dumps({
        'nodes': [
            {'op': 'null', 'name': 'data', 'inputs': []},
            {'op': 'null', 'name': 'w', 'attrs': {'__shape__': '(5, 7)', '__lr_mult__': '2.0'}, 'inputs': []},
            {'op': 'FullyConnected', 'name': 'fc', 'attrs': {'num_hidden': '5', 'no_bias': 'True', 'flatten': 'True'},
             'inputs': [[0, 0, 0], [1, 0, 0]]},
            {'op': 'Activation', 'name': 'act', 'attrs': {'act_type': 'tanh'}, 'inputs': [[2, 0, 0]]}],
        'arg_nodes': [0, 1], 'node_row_ptr': [0, 1, 2, 3, 4], 'heads': [[3, 0, 0]],
        'attrs': {'mxnet_version': ['int', 10600]}})
    s = sym.load_json(js)
    assert s.list_arguments() == ['data', 'w']
    assert s.attr_dict()['w']['__lr_mult__'] == '2.0'
    x, w = np.random.randn(3, 7).astype('float32'), np.random.randn(5, 7).astype('float32')
    out = s.eval(data=nd.array(x), w=nd.array(w))[0]
    assert_almost_equal(out.asnumpy(), np.tanh(x @ w.T), rtol=1e-5, atol=1e-6)


def test_infer_shape_and_type():
    net = _mlp()
    arg_shapes, out_shapes, aux_shapes = net.infer_shape(data=(8, 10))
    assert dict(zip(net.list_arguments(), arg_shapes)) == {
        'data': (8, 10), 'fc1_weight': (16, 10), 'fc1_bias': (16,), 'fc2_weight': (4, 16), 'fc2_bias': (4,),
        'softmax_label': (8,)}
    assert out_shapes == [(8, 4)] and aux_shapes == []
    arg_types, out_types, _ = net.infer_type(data='float32')
    assert all(t == np.float32 for t in arg_types) and out_types == [np.float32]
    data = sym.Variable('data')
    bn = sym.BatchNorm(data=data, name='bn')
    assert bn.list_auxiliary_states() == ['bn_moving_mean', 'bn_moving_var']
    a, o, x = bn.infer_shape(data=(2, 5, 3, 3))
    assert x == [(5,), (5,)] and o == [(2, 5, 3, 3)]
    partial = net.infer_shape_partial()
    assert partial[0][0] in ((), None) or partial[0][0] == ()


def test_symbol_arithmetic_and_grouping():
    a, b = sym.Variable('a'), sym.Variable('b')
    c = (a + b) * 2 - a / b + a ** 2
    av, bv = np.array([1., 2.], 'float32'), np.array([4., 5.], 'float32')
    out = c.eval(a=nd.array(av), b=nd.array(bv))[0].asnumpy()
    assert_almost_equal(out, (av + bv) * 2 - av / bv + av ** 2, rtol=1e-6)
    g = sym.Group([a + b, a * b])
    assert len(g.list_outputs()) == 2
    o1, o2 = g.eval(a=nd.array(av), b=nd.array(bv))
    assert same(o1.asnumpy(), av + bv) and same(o2.asnumpy(), av * bv)
    assert g[1].list_outputs() == g.list_outputs()[1:]


def test_simple_bind_forward_backward():
    net = _mlp()
    ex = net.simple_bind(mx.cpu(), data=(6, 10), grad_req='write')
    for name, arr in ex.arg_dict.items():
        if name.endswith('weight'):
            arr[:] = nd.array(np.random.randn(*arr.shape) * 0.1)
    x = np.random.randn(6, 10).astype('float32')
    y = np.random.randint(0, 4, (6,)).astype('float32')
    ex.arg_dict['data'][:] = nd.array(x)
    ex.arg_dict['softmax_label'][:] = nd.array(y)
    out = ex.forward(is_train=True)[0].asnumpy()
    assert out.shape == (6, 4) and np.allclose(out.sum(1), 1, atol=1e-5)
    ex.backward()
    # SoftmaxOutput gradient w.r.t. its input is (p - onehot); chain to fc2_bias = column sums
    p = out.copy()
    p[np.arange(6), y.astype(int)] -= 1
    assert_almost_equal(ex.grad_dict['fc2_bias'].asnumpy(), p.sum(0), rtol=1e-4, atol=1e-5)
    assert float(abs(ex.grad_dict['fc1_weight']).sum().asscalar()) > 0


def test_bind_with_explicit_arrays_and_grad_req_add():
    a, b = sym.Variable('a'), sym.Variable('b')
    c = a * b
    av, bv = nd.array([1., 2., 3.]), nd.array([4., 5., 6.])
    ga, gb = nd.zeros((3,)), nd.zeros((3,))
    ex = c.bind(mx.cpu(), args={'a': av, 'b': bv}, args_grad={'a': ga, 'b': gb}, grad_req='add')
    for _ in range(2):
        ex.forward(is_train=True)
        ex.backward(out_grads=nd.ones((3,)))
    assert same(ga.asnumpy(), 2 * bv.asnumpy()) and same(gb.asnumpy(), 2 * av.asnumpy())


def test_variable_attributes_and_scopes():
    with mx.AttrScope(ctx_group='dev1', lr_mult='0.5'):
        v = sym.Variable('v')
        fc = sym.FullyConnected(v, num_hidden=3, name='fc')
    assert v.attr('ctx_group') == 'dev1' and fc.attr('lr_mult') == '0.5'
    w = sym.Variable('w', shape=(3, 4), lr_mult=2.0, wd_mult=0.0, dtype='float16', init=mx.init.One())
    ad = w.attr_dict()['w']
    assert ad['__shape__'] == '(3, 4)' and ad['__lr_mult__'] == '2.0' and ad['__wd_mult__'] == '0.0'
    assert ad['__dtype__'] in ('2', 'float16')
    with mx.name.Prefix('stage1_'):
        s = sym.Activation(sym.Variable('x'), act_type='relu')
    assert s.name.startswith('stage1_activation')


def test_save_load_file(tmp_path):
    net = _mlp()
    f = str(tmp_path / 'net-symbol.json')
    net.save(f)
    back = sym.load(f)
    assert back.tojson() == net.tojson()


def test_symbol_numpy_namespace_and_optimize_for():
    x = sym.Variable('x')
    y = sym.relu(x) + sym.sigmoid(x)
    out = y.eval(x=nd.array([-1., 1.]))[0].asnumpy()
    assert_almost_equal(out, np.maximum([-1., 1.], 0) + 1 / (1 + np.exp(-np.array([-1., 1.]))), rtol=1e-6)
    z = y.optimize_for('default')
    assert z.list_arguments() == ['x']


def test_symbolic_control_flow_foreach_while_cond(tmp_path):
    """mx.sym.contrib.foreach / while_loop / cond: evaluation, shape inference, gradients and the JSON round trip."""
    import numpy as onp
    rng = onp.random.RandomState(0)
    data, init, w = mx.sym.var('data'), mx.sym.var('init'), mx.sym.var('w')

    def step(x, state):
        new = mx.sym.tanh(mx.sym.dot(x, w) + state)
        return new * 2.0, new
    outs, final = mx.sym.contrib.foreach(step, data, init)
    g = mx.sym.Group([outs, final])
    assert g.list_arguments() == ['data', 'init', 'w']
    xv, hv, wv = rng.randn(5, 3, 4).astype('float32'), rng.randn(3, 4).astype('float32'), rng.randn(4, 4).astype('float32') * 0.5
    ref, h = [], hv
    for t in range(5):
        h = onp.tanh(xv[t] @ wv + h)
        ref.append(2 * h)
    _, out_shapes, _ = g.infer_shape(data=(5, 3, 4), init=(3, 4), w=(4, 4))
    assert out_shapes == [(5, 3, 4), (3, 4)]
    for sym in (g, mx.sym.load_json(g.tojson())):                       # as built, and after a trip through JSON
        args = {'data': nd.array(xv), 'init': nd.array(hv), 'w': nd.array(wv)}
        grads = {k: nd.zeros(v.shape) for k, v in args.items()}
        ex = sym._bind(mx.cpu(), args, args_grad=grads)
        res = ex.forward(is_train=True)
        onp.testing.assert_allclose(res[0].asnumpy(), onp.stack(ref), rtol=1e-5, atol=1e-6)
        onp.testing.assert_allclose(res[1].asnumpy(), h, rtol=1e-5, atol=1e-6)
        ex.backward([nd.ones((5, 3, 4)), nd.zeros((3, 4))])
        assert float(grads['w'].abs().sum().asscalar()) > 0 and float(grads['data'].abs().sum().asscalar()) > 0
    saved = str(tmp_path / 'loop-symbol.json')
    g.save(saved)
    import json
    node = [n for n in json.load(open(saved))['nodes'] if n['op'] == '_foreach'][0]
    assert len(node['subgraphs']) == 1 and any(m['op'] == 'tanh' for m in node['subgraphs'][0]['nodes'])

    # while_loop: s += i for i < 4, outputs padded to max_iterations
    i0, s0 = mx.sym.var('i'), mx.sym.var('s')
    outs, (i_f, s_f) = mx.sym.contrib.while_loop(lambda i, s: i < 4, lambda i, s: (s + i, [i + 1, s + i]), [i0, s0], max_iterations=6)
    wl = mx.sym.load_json(mx.sym.Group([outs, i_f, s_f]).tojson())
    r = wl._bind(mx.cpu(), {'i': nd.array([0.0]), 's': nd.array([10.0])}).forward()
    onp.testing.assert_allclose(r[0].asnumpy().ravel(), [10, 11, 13, 16, 0, 0])
    assert float(r[1].asscalar()) == 4 and float(r[2].asscalar()) == 16

    # cond with outer variables captured by the branches
    p, a, b = mx.sym.var('p'), mx.sym.var('a'), mx.sym.var('b')
    c = mx.sym.contrib.cond(p, lambda: a * 2.0, lambda: b - 1.0)
    c = mx.sym.load_json(c.tojson())
    for pv, expect in ((1.0, [2.0, 4.0]), (0.0, [4.0, 5.0])):
        got = c._bind(mx.cpu(), {'p': nd.array([pv]), 'a': nd.array([1.0, 2.0]), 'b': nd.array([5.0, 6.0])}).forward()[0]
        onp.testing.assert_allclose(got.asnumpy(), expect)


def test_group2ctx_places_operators_and_arguments():
    """Model parallelism through ``ctx_group`` attributes and ``group2ctx`` (python/mxnet/symbol/symbol.py bind;
    tests/python/unittest/test_model_parallel.py in the reference): operators and their arguments live on the context of
    their group, ungrouped nodes follow their inputs, one value crosses between the stages, and the results and gradients
    equal those of the unplaced graph."""
    import numpy as np
    import mxnet_b200 as mx
    from mxnet_b200 import nd
    with mx.AttrScope(ctx_group='stage1'):
        x = mx.sym.var('data')
        w1 = mx.sym.var('w1')
        h = mx.sym.FullyConnected(x, w1, num_hidden=8, no_bias=True, name='fc1')
    h = mx.sym.relu(h, name='act')                                   # no group: follows its input
    with mx.AttrScope(ctx_group='stage2'):
        w2 = mx.sym.var('w2')
        out = mx.sym.FullyConnected(h, w2, num_hidden=3, no_bias=True, name='fc2')
    shapes = dict(data=(4, 5), w1=(8, 5), w2=(3, 8))
    placed = out.simple_bind(mx.cpu(0), group2ctx={'stage1': mx.cpu(1), 'stage2': mx.cpu(2)}, **shapes)
    plain = out.simple_bind(mx.cpu(0), **shapes)
    where = {n.name: placed._placement[id(n)] for n in mx.symbol.symbol._topo(out._outputs)}
    assert where == {'data': mx.cpu(1), 'w1': mx.cpu(1), 'fc1': mx.cpu(1), 'act': mx.cpu(1), 'w2': mx.cpu(2), 'fc2': mx.cpu(2)}
    assert placed.arg_dict['w1'].context == mx.cpu(1) and placed.arg_dict['w2'].context == mx.cpu(2)
    assert placed.grad_dict['w2'].context == mx.cpu(2)
    rng = np.random.RandomState(0)
    for k, s in shapes.items():
        v = rng.randn(*s).astype('float32')
        placed.arg_dict[k][:] = v
        plain.arg_dict[k][:] = v
    a = placed.forward(is_train=True)[0]
    b = plain.forward(is_train=True)[0]
    assert placed.cross_device_copies == 1
    np.testing.assert_allclose(a.asnumpy(), b.asnumpy(), rtol=1e-6)
    placed.backward(nd.ones(a.shape, ctx=a.context))
    plain.backward(nd.ones(b.shape, ctx=b.context))
    for k in shapes:
        np.testing.assert_allclose(placed.grad_dict[k].asnumpy(), plain.grad_dict[k].asnumpy(), rtol=1e-5, atol=1e-6)


def _mirror_net():
    data = mx.sym.Variable('data')
    x = mx.sym.Convolution(data, num_filter=4, kernel=(3, 3), pad=(1, 1), name='c1')
    x = mx.sym.Activation(x, act_type='relu')
    x = x * 2.0 + 1.0
    x = mx.sym.tanh(x)
    x = mx.sym.Pooling(x, kernel=(2, 2), stride=(2, 2), pool_type='max')
    x = mx.sym.Convolution(x, num_filter=3, kernel=(1, 1), name='c2')
    x = mx.sym.sigmoid(x)
    x = mx.sym.Flatten(x)
    x = mx.sym.FullyConnected(x, num_hidden=5, name='fc')
    return mx.sym.sum(mx.sym.square(x))


def _mirror_grads(flag, monkeypatch):
    for name in ('MXNET_BACKWARD_DO_MIRROR', 'MXNET_MEMORY_OPT'):
        monkeypatch.delenv(name, raising=False)
    if flag:
        monkeypatch.setenv(flag, '1')
    net = _mirror_net()
    ex = net.simple_bind(mx.cpu(), data=(2, 3, 8, 8))
    rng = np.random.RandomState(0)
    for name, arr in ex.arg_dict.items():
        arr[:] = rng.uniform(-0.5, 0.5, arr.shape).astype('float32')
    out = ex.forward(is_train=True)[0].asnumpy()
    ex.backward()
    return out, {k: v.asnumpy() for k, v in ex.grad_dict.items() if v is not None}, ex.mirrored_nodes


@pytest.mark.parametrize('flag', ['MXNET_BACKWARD_DO_MIRROR', 'MXNET_MEMORY_OPT'])
def test_backward_mirroring_recomputes_cheap_runs_and_keeps_gradients(flag, monkeypatch):
    """Backward mirroring (reference: src/nnvm/gradient.cc with a mirror function; docs env_var MXNET_BACKWARD_DO_MIRROR):
    runs of cheap operators between the convolutions are recomputed in backward; outputs and gradients are unchanged."""
    out0, g0, m0 = _mirror_grads(None, monkeypatch)
    out1, g1, m1 = _mirror_grads(flag, monkeypatch)
    assert m0 == 0
    assert m1 == 9          # three runs: relu, *2, +1, tanh, pooling | sigmoid, flatten | square, sum
    np.testing.assert_array_equal(out0, out1)
    assert set(g0) == set(g1)
    for k in g0:
        np.testing.assert_allclose(g0[k], g1[k], rtol=1e-6, atol=1e-7)


def test_force_mirroring_attribute_marks_single_operators(monkeypatch):
    for name in ('MXNET_BACKWARD_DO_MIRROR', 'MXNET_MEMORY_OPT'):
        monkeypatch.delenv(name, raising=False)
    data = mx.sym.Variable('data')
    with mx.AttrScope(force_mirroring='True'):
        x = mx.sym.tanh(data * 3.0)
        x = mx.sym.sigmoid(x)
    y = mx.sym.sum(mx.sym.FullyConnected(x, num_hidden=2, name='fc'))
    ex = y.simple_bind(mx.cpu(), data=(4, 6))
    for name, arr in ex.arg_dict.items():
        arr[:] = np.random.RandomState(1).uniform(-1, 1, arr.shape).astype('float32')
    ex.forward(is_train=True)
    ex.backward()
    assert ex.mirrored_nodes == 3
    d = ex.arg_dict['data'].asnumpy()
    w = ex.arg_dict['fc_weight'].asnumpy()
    t = np.tanh(3 * d)
    s = 1 / (1 + np.exp(-t))
    expect = (w.sum(0)[None, :] * s * (1 - s)) * (1 - t * t) * 3
    np.testing.assert_allclose(ex.grad_dict['data'].asnumpy(), expect, rtol=1e-5, atol=1e-6)


def _nchw_trunk():
    data = mx.sym.Variable('data')
    x = mx.sym.Convolution(data, num_filter=8, kernel=(3, 3), pad=(1, 1), no_bias=True, name='c1')
    x = mx.sym.BatchNorm(x, fix_gamma=False, name='bn1')
    x = mx.sym.Activation(x, act_type='relu')
    skip = x
    y = mx.sym.Convolution(x, num_filter=8, kernel=(3, 3), pad=(1, 1), name='c2')
    y = mx.sym.BatchNorm(y, fix_gamma=False, name='bn2')
    x = mx.sym.relu(y + skip) * 0.5
    x = mx.sym.Pooling(x, kernel=(2, 2), stride=(2, 2), pool_type='max')
    a = mx.sym.Convolution(x, num_filter=4, kernel=(1, 1), name='c3a')
    b = mx.sym.Convolution(x, num_filter=6, kernel=(3, 3), pad=(1, 1), stride=(1, 1), name='c3b')
    x = mx.sym.Concat(a, b, dim=1)
    x = mx.sym.Pooling(x, global_pool=True, pool_type='avg', kernel=(1, 1))
    x = mx.sym.Flatten(x)
    return mx.sym.FullyConnected(x, num_hidden=3, name='fc')


def test_layout_pass_moves_the_convolutional_trunk_to_nhwc():
    """Automatic layout management (reference: src/common/alm.cc): same outputs, gradients and running statistics, with
    transposes only at the borders of the trunk."""
    from mxnet_b200.symbol.layout import optimize_layout
    net = _nchw_trunk()
    opt = optimize_layout(net)
    nodes = json.loads(opt.tojson())['nodes']
    ops = [n['op'] for n in nodes]
    # one transpose for the image, one per convolution weight (4), one back to NCHW before Flatten
    assert ops.count('_layout_transpose') == 6
    for n in nodes:
        if n['op'] == 'Convolution':
            assert n['attrs']['layout'] == 'NHWC'
        if n['op'] == 'BatchNorm':
            assert n['attrs']['axis'] == '3'
        if n['op'] == 'Concat':
            assert n['attrs']['dim'] == '3'
        if n['op'] == 'Pooling':
            assert n['attrs']['layout'] == 'NHWC'
    assert opt.list_arguments() == net.list_arguments() and opt.list_auxiliary_states() == net.list_auxiliary_states()
    results = []
    for graph in (net, opt):
        ex = graph.simple_bind(mx.cpu(), data=(2, 3, 8, 8))
        rng = np.random.RandomState(4)
        for name, arr in ex.arg_dict.items():
            arr[:] = rng.uniform(-0.5, 0.5, arr.shape).astype('float32')
        out = ex.forward(is_train=True)[0].asnumpy()
        ex.backward(mx.nd.ones((2, 3), ctx=mx.cpu()))
        results.append((out, {k: v.asnumpy() for k, v in ex.grad_dict.items() if v is not None},
                        {k: v.asnumpy() for k, v in ex.aux_dict.items()}))
    (o0, g0, a0), (o1, g1, a1) = results
    np.testing.assert_allclose(o0, o1, rtol=1e-4, atol=1e-5)
    for k in g0:
        np.testing.assert_allclose(g0[k], g1[k], rtol=2e-4, atol=1e-5, err_msg=k)
    for k in a0:
        np.testing.assert_allclose(a0[k], a1[k], rtol=1e-5, atol=1e-6, err_msg=k)


def test_layout_pass_leaves_graphs_without_convolutions_alone():
    from mxnet_b200.symbol.layout import optimize_layout
    x = mx.sym.Variable('x')
    y = mx.sym.FullyConnected(mx.sym.relu(x), num_hidden=4, name='fc')
    assert optimize_layout(y) is y


def test_hybridized_block_runs_through_the_layout_pass_when_enabled():
    from mxnet_b200.symbol import layout
    from mxnet_b200.gluon import nn
    net = nn.HybridSequential()
    net.add(nn.Conv2D(6, 3, padding=1), nn.BatchNorm(), nn.Activation('relu'), nn.MaxPool2D(2), nn.Conv2D(4, 1),
            nn.GlobalAvgPool2D(), nn.Flatten(), nn.Dense(3))
    net.initialize()
    x = mx.nd.array(np.random.RandomState(5).uniform(-1, 1, (2, 3, 8, 8)).astype('float32'))
    expect = net(x).asnumpy()
    net.hybridize()
    net(x)
    assert not layout.get_optimize_layout()
    layout.set_optimize_layout(True)
    try:
        got = net(x)
        assert net._partitioned_by == 'optimize_layout'
        assert '_layout_transpose' in net._partitioned.tojson()
        np.testing.assert_allclose(got.asnumpy(), expect, rtol=5e-3, atol=5e-3)   # a GPU run may use tf32 convolutions
        with mx.autograd.record():
            loss = net(x).sum()
        loss.backward()
        assert float(np.abs(net[0].weight.grad().asnumpy()).sum()) > 0
    finally:
        layout.set_optimize_layout(False)


def test_symbol_surface_found_by_the_reference_tests():
    """``python/mxnet/symbol/symbol.py``: abs(), children of grouped heads, deep copies that can be renamed,
    a missing data input becomes ``<name>_data`` for later composition, same-shape operands infer from one another;
    ``python/mxnet/executor.py``: an executor bound with gradient buffers differentiates after a plain forward();
    ``mx.nd.CachedOp`` runs a symbol on arrays."""
    import copy
    import numpy as np
    import pytest
    import mxnet_b200 as mx
    from mxnet_b200.base import NotImplementedForSymbol
    x = mx.sym.Variable('x')
    assert issubclass(NotImplementedForSymbol, mx.base.MXNetError) and mx.sym.symbol.NotImplementedForSymbol is NotImplementedForSymbol
    assert abs(x).list_arguments() == ['x']
    b = copy.copy(x)
    b._set_attr(name='b')
    assert x.name == 'x' and b.name == 'b'

    data = mx.sym.Variable('data')
    sliced = mx.sym.SliceChannel(data, num_outputs=3, name='slice')
    assert sliced.get_children().list_outputs() == ['data']
    assert mx.sym.Concat(*list(sliced)).get_children().list_outputs() == ['slice_output0', 'slice_output1', 'slice_output2']

    net1 = mx.sym.FullyConnected(data=data, name='fc1', num_hidden=10)
    net2 = mx.sym.FullyConnected(name='fc3', num_hidden=10)
    assert 'fc3_data' in net2.list_arguments()
    composed = net2(fc3_data=net1, name='composed')
    assert 'fc3_data' not in composed.list_arguments() and 'data' in composed.list_arguments()

    a = mx.sym.Variable('a', shape=(2, 3))
    c = mx.sym.elemwise_add(a, mx.sym.Variable('b'))
    arg_shapes, out_shapes, _ = c.infer_shape()
    assert arg_shapes == [(2, 3), (2, 3)] and out_shapes == [(2, 3)]

    lhs, rhs = mx.nd.array([[1., 2.]]), mx.nd.array([[3., 4.]])
    gl, gr = mx.nd.empty((1, 2)), mx.nd.empty((1, 2))
    prod = mx.sym.Variable('lhs') * mx.sym.Variable('rhs')
    exe = prod._bind(mx.cpu(), args=[lhs, rhs], args_grad=[gl, gr])
    exe.forward()
    exe.backward([mx.nd.ones((1, 2))])
    np.testing.assert_allclose(gl.asnumpy(), rhs.asnumpy())
    np.testing.assert_allclose(gr.asnumpy(), lhs.asnumpy())

    op = mx.nd.CachedOp(prod, [('static_alloc', True)])
    np.testing.assert_allclose(op(lhs, rhs).asnumpy(), [[3., 8.]])
    z = mx.nd.CachedOp(mx.sym.zeros((3, 3)))(None, default_device=mx.cpu())
    assert z.shape == (3, 3) and float(z.sum()) == 0.0

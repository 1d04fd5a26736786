"""``import mxnet`` resolves to this framework, module by module."""
import numpy as np


def test_import_mxnet_alias_runs_reference_style_code():
    import mxnet as mx
    from mxnet import autograd, gluon, nd
    from mxnet.gluon import nn
    import mxnet.gluon.data.vision as vision
    import mxnet_b200
    assert mx is mxnet_b200 and gluon is mxnet_b200.gluon and nn is mxnet_b200.gluon.nn
    assert vision is mxnet_b200.gluon.data.vision
    net = nn.Sequential()
    net.add(nn.Dense(8, activation='relu'), nn.Dense(2))
    net.initialize(mx.init.Xavier())
    trainer = gluon.Trainer(net.collect_params(), 'adam', {'learning_rate': 0.01})
    x, y = nd.array(np.random.randn(16, 4)), nd.array(np.random.randint(0, 2, (16,)))
    loss_fn = gluon.loss.SoftmaxCrossEntropyLoss()
    first = None
    for _ in range(20):
        with autograd.record():
            loss = loss_fn(net(x), y)
        loss.backward()
        trainer.step(16)
        first = first if first is not None else float(loss.mean().asscalar())
    assert float(loss.mean().asscalar()) < first
    assert mx.np.ones((2, 2)).sum().item() == 4
    assert mx.cpu(0) == mx.context.cpu(0)

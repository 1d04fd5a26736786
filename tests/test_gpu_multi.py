"""Multi-GPU checks (one process per GPU, launched as child processes)."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _launch(script, nproc, port, extra_env=None, timeout=600):
    env = dict(os.environ)
    env.update({'NCCL_NVLS_ENABLE': '0'})
    env.update(extra_env or {})
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node', str(nproc),
           '--master-addr', '127.0.0.1', '--master-port', str(port), os.path.join(HERE, 'dist', script)]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)


@pytest.mark.parametrize('nproc', [2, 4, 8])
def test_fused_step_matches_nccl_path_across_ranks(nproc):
    if torch.cuda.device_count() < nproc:
        pytest.skip('needs %d GPUs' % nproc)
    r = _launch('fused_step_worker.py', nproc, 29611 + nproc)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith('REPORT ')][-1]
    rep = json.loads(line[len('REPORT '):])
    assert rep['world'] == nproc
    assert rep['float32']['ranks_identical'] and rep['float16']['ranks_identical']
    assert rep['float32']['max_abs_diff_vs_nccl_path'] < 1e-5
    assert rep['float16']['max_abs_diff_vs_nccl_path'] < 5e-3
    for name in ('lamb', 'adam'):
        assert rep[name]['ranks_identical'] and rep[name]['max_abs_diff_vs_nccl_path'] < 1e-4


@pytest.mark.parametrize('nproc', [2, 8])
def test_fused_step_through_the_nvlink_switch(nproc):
    """``MXNET_KVSTORE_NVLS=1``: the arenas are symmetric memory with a multicast mapping, gradients are summed by
    ``multimem.ld_reduce`` and weights broadcast by ``multimem.st``.  Same checks as the peer-memory step (agreement with the
    NCCL path, identical ranks, every optimizer).  Where the machine offers no multicast object the step falls back to
    peer loads and stores and the test only records that."""
    if torch.cuda.device_count() < nproc:
        pytest.skip('needs %d GPUs' % nproc)
    r = _launch('fused_step_worker.py', nproc, 29731 + nproc, {'MXNET_KVSTORE_NVLS': '1'})
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith('REPORT ')][-1]
    rep = json.loads(line[len('REPORT '):])
    assert rep['world'] == nproc and rep['nvls_requested']
    assert rep['float32']['ranks_identical'] and rep['float16']['ranks_identical']
    assert rep['float32']['max_abs_diff_vs_nccl_path'] < 1e-5
    assert rep['float16']['max_abs_diff_vs_nccl_path'] < 5e-3
    for name in ('lamb', 'adam'):
        assert rep[name]['ranks_identical'] and rep[name]['max_abs_diff_vs_nccl_path'] < 1e-4
    print('multicast steps:', rep['multicast_steps'])


@pytest.mark.parametrize('nproc', [1, 2, 8])
def test_data_parallel_training_converges(nproc):
    """A small residual conv net (NHWC, BatchNorm, fp16 AMP, CUDA graphs, fused peer-memory SGD step) on a fixed learnable
    data set: the loss must fall and the training accuracy must rise well above chance at every world size, with all ranks
    holding identical weights (``tests/dist/convergence_worker.py``)."""
    if torch.cuda.device_count() < nproc:
        pytest.skip('needs %d GPUs' % nproc)
    r = _launch('convergence_worker.py', nproc, 29711 + nproc)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith('REPORT ')][-1]
    rep = json.loads(line[len('REPORT '):])
    assert rep['world'] == nproc and rep['fused'] and rep['finite'] and rep['ranks_identical'], rep
    assert rep['last'] < 0.5 * rep['first'], rep
    assert rep['accuracy'] > 0.6, rep


@pytest.mark.parametrize('nproc', [2, 4])
def test_sync_batchnorm_over_peer_memory(nproc):
    """SyncBatchNorm statistics through the peer-memory all-reduce kernel: same sums as the library collective, same
    normalisation and gradients as BatchNorm over the whole batch."""
    if torch.cuda.device_count() < nproc:
        pytest.skip('needs %d GPUs' % nproc)
    r = _launch('sync_bn_worker.py', nproc, 29651 + nproc)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith('REPORT ')][-1]
    rep = json.loads(line[len('REPORT '):])
    assert rep['world'] == nproc and rep['status'] == 0 and rep['status_after'] == 0
    assert rep['allreduce_max_abs_diff'] == 0.0
    assert rep['y_diff'] < 1e-4 and rep['dx_diff'] < 1e-4 and rep['mean_diff'] < 1e-5


@pytest.mark.parametrize('ngpu', [2, 4])
def test_single_process_multi_gpu_trainer_runs_on_the_fused_kernels(ngpu):
    """``Trainer`` over ``ctx=[gpu(0), ..., gpu(n-1)]`` in ONE process (the reference's main multi-GPU mode): the fused
    peer-memory step over the process's GPUs gives every replica the same weights, equal to one-GPU training on the
    whole batch up to summation order."""
    if torch.cuda.device_count() < ngpu:
        pytest.skip('needs %d GPUs' % ngpu)
    r = subprocess.run([sys.executable, os.path.join(HERE, 'dist', 'single_process_worker.py'), str(ngpu)],
                       capture_output=True, text=True, timeout=600, env=dict(os.environ, NCCL_NVLS_ENABLE='0'))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    rep = json.loads([l for l in r.stdout.splitlines() if l.startswith('REPORT ')][-1][len('REPORT '):])
    assert rep['gpus'] == ngpu and rep['states_round_trip']
    for key, tol in (('float32_sgd', 1e-5), ('float16_sgd', 5e-3), ('float32_adam', 2e-3), ('float32_lamb', 1e-4)):
        assert rep[key]['replicas_identical'], key
        assert rep[key]['max_abs_diff_vs_one_gpu'] < tol, (key, rep[key])


def test_device_kvstore_reduces_on_prioritised_communication_streams():
    """The generic ``device`` store over two GPUs of one process (fused step off): reductions run on the high / low
    priority communication streams picked by the key's priority, the compute streams wait for them by events, and
    2-bit compressed gradients cross between the GPUs as packed words."""
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    import numpy as np
    import mxnet_b200 as mx
    from mxnet_b200 import engine, kv, nd
    ctxs = [mx.gpu(0), mx.gpu(1)]
    store = kv.create('device')
    n = 1 << 20
    for k in range(12):
        store.init(k, nd.zeros((n,), ctx=ctxs[0]))
    vals = [[nd.full((n,), float(k + 1 + d), ctx=c) for d, c in enumerate(ctxs)] for k in range(12)]
    outs = [[nd.zeros((n,), ctx=c) for c in ctxs] for k in range(12)]
    for k in range(12):
        store.pushpull(k, vals[k], out=outs[k], priority=-k)
    assert store._pending, 'reductions of multi-GPU keys are queued on the communication streams'
    st = engine.streams(0)
    assert st.comm_high.cuda_stream != st.comm_low.cuda_stream
    store.wait_pending()
    for k in range(12):
        for o in outs[k]:
            assert float(o.asnumpy()[0]) == 2 * k + 3 and float(o.asnumpy()[-1]) == 2 * k + 3
    comp = kv.create('device')
    comp.set_gradient_compression({'type': '2bit', 'threshold': 0.5})
    comp.init('g', nd.zeros((n,), ctx=ctxs[0]))
    g = [nd.full((n,), 0.75, ctx=c) for c in ctxs]
    out = nd.zeros((n,), ctx=ctxs[0])
    comp.pushpull('g', g, out=out)
    comp.wait_pending()
    assert float(out.asnumpy()[7]) == 1.0                       # 0.5 from each GPU
    assert comp.wire_bytes == n // 16 * 4                       # only GPU 1's packed words crossed


def test_model_parallel_executor_across_two_gpus():
    """``group2ctx`` with real devices: the first stage runs on GPU 0, the second on GPU 1, the activation crosses once, the
    arguments and gradients live with their stage, and everything equals the single-device executor."""
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    import numpy as np
    import mxnet_b200 as mx
    from mxnet_b200 import nd
    with mx.AttrScope(ctx_group='stage1'):
        x = mx.sym.var('data')
        w1 = mx.sym.var('w1')
        h = mx.sym.relu(mx.sym.FullyConnected(x, w1, num_hidden=64, no_bias=True, name='fc1'))
    with mx.AttrScope(ctx_group='stage2'):
        w2 = mx.sym.var('w2')
        out = mx.sym.FullyConnected(h, w2, num_hidden=16, no_bias=True, name='fc2')
    shapes = dict(data=(32, 48), w1=(64, 48), w2=(16, 64))
    placed = out.simple_bind(mx.gpu(0), group2ctx={'stage1': mx.gpu(0), 'stage2': mx.gpu(1)}, **shapes)
    plain = out.simple_bind(mx.gpu(0), **shapes)
    assert placed.arg_dict['w2'].context == mx.gpu(1) and placed.arg_dict['w1'].context == mx.gpu(0)
    rng = np.random.RandomState(0)
    for k, s in shapes.items():
        v = rng.randn(*s).astype('float32')
        placed.arg_dict[k][:] = v
        plain.arg_dict[k][:] = v
    a = placed.forward(is_train=True)[0]
    b = plain.forward(is_train=True)[0]
    assert a.context == mx.gpu(1) and placed.cross_device_copies == 1
    np.testing.assert_allclose(a.asnumpy(), b.asnumpy(), rtol=1e-4, atol=1e-4)
    placed.backward(nd.ones(a.shape, ctx=mx.gpu(1)))
    plain.backward(nd.ones(b.shape, ctx=mx.gpu(0)))
    for k in shapes:
        assert placed.grad_dict[k].context == placed.arg_dict[k].context
        np.testing.assert_allclose(placed.grad_dict[k].asnumpy(), plain.grad_dict[k].asnumpy(), rtol=1e-3, atol=1e-3)

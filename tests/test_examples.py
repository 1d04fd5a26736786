"""The scripts under example/ run with tiny settings (synthetic data, CPU)."""
import importlib.util
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(rel):
    path = os.path.join(ROOT, 'example', rel)
    spec = importlib.util.spec_from_file_location('example_' + os.path.basename(rel)[:-3], path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_mnist_example_learns_the_synthetic_classes():
    acc = _load('gluon/mnist/mnist.py').main(['--epochs', '1', '--samples', '1200', '--hybridize'])
    assert acc > 0.9


def test_image_classification_example_steps():
    import math
    loss = _load('gluon/image_classification.py').main(['--iters', '2', '--batch-size', '2', '--image-size', '32',
                                                        '--model', 'resnet18_v1'])
    assert math.isfinite(loss)


def test_language_model_example_beats_the_uniform_guess():
    ppl = _load('gluon/word_language_model/train.py').main(['--tokens', '12000', '--vocab', '50', '--epochs', '1', '--lr', '2.0'])
    assert ppl < 45


def test_profiler_example_writes_a_trace(tmp_path):
    out = str(tmp_path / 'trace.json')
    table = _load('profiler/profiler_matmul.py').main(['--iters', '3', '--size', '32', '--file', out])
    assert 'dot' in table and os.path.getsize(out) > 100


def test_quantization_example_stays_close_to_fp32():
    err = _load('quantization/quantize_model.py').main(['--image-size', '32', '--batch-size', '2', '--calib-batches', '1'])
    assert err < 0.2


def test_distributed_example_with_two_gloo_workers():
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node', '2', '--master-addr', '127.0.0.1',
           '--master-port', '29641', os.path.join(ROOT, 'example', 'distributed_training', 'cifar10_dist.py'), '--cpu',
           '--samples', '128', '--batch-size', '16']
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert 'worker 0/2 epoch 0' in res.stdout and 'worker 1/2 epoch 0' in res.stdout

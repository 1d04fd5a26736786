#!/usr/bin/env python
"""Per-operator forward/backward timing (the counterpart of the reference's ``benchmark/opperf``).

    python benchmark/opperf/opperf.py                               # default operator set, JSON lines
    python benchmark/opperf/opperf.py --op BatchNorm --dtype float16 --runs 20
    python benchmark/opperf/opperf.py --list

Each case runs through the public ``mx.nd`` operators (so it times what a user gets), after ``--warmup``
untimed runs, with CUDA events around ``--runs`` repetitions on the launching stream and a write of a
buffer larger than the L2 cache between repetitions.  Output: one JSON object per case with mean forward
and backward milliseconds, the algorithmic bytes / FLOPs of the case and the achieved GB/s or TFLOP/s.
On a machine without a GPU the cases run on the CPU with wall-clock timing (functional check only).
"""
import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import numpy as np                                          # noqa: E402
import torch                                                # noqa: E402

import mxnet_b200 as mx                                     # noqa: E402
from mxnet_b200 import autograd, nd                         # noqa: E402


def _rand(shape, ctx, dtype, scale=1.0):
    t = torch.randn(*shape, device=ctx.torch_device) * scale
    return nd.NDArray._from_tensor(t.to(mx.base.to_torch_dtype(dtype)), ctx)


def _esize(dtype):
    return np.dtype(dtype).itemsize


# Each case: name -> function(ctx, dtype, small) returning dict(inputs=[...], fn=callable(*inputs) -> output,
# fwd_bytes, bwd_bytes, fwd_flops, bwd_flops).  Shapes follow the ResNet-50 / BERT-base hot spots.
def case_batchnorm(ctx, dtype, small, relu=False, residual=False):
    n, h, c = (32, 56, 256) if small else (256, 56, 256)
    x = _rand((n, h, h, c), ctx, dtype)
    res = _rand((n, h, h, c), ctx, dtype) if residual else None
    gamma, beta = _rand((c,), ctx, dtype), _rand((c,), ctx, dtype)
    mean, var = nd.zeros((c,), ctx=ctx), nd.ones((c,), ctx=ctx)
    kw = dict(eps=1e-5, momentum=0.9, fix_gamma=False, axis=3)
    if relu:
        kw['act_type'] = 'relu'
    ins = [x, gamma, beta] + ([res] if residual else [])

    def fn(x, gamma, beta, res=None):
        return nd.BatchNorm(x, gamma, beta, mean, var, res, **kw) if res is not None else \
            nd.BatchNorm(x, gamma, beta, mean, var, **kw)
    nb = x.size * _esize(dtype)
    return dict(inputs=ins, fn=fn, fwd_bytes=nb * (3 + residual), bwd_bytes=nb * (5 + 3 * residual + (0 if not relu else 0)))


def case_conv(ctx, dtype, small, cin=64, cout=64, k=3, hw=56, stride=1):
    n = 32 if small else 256
    x = _rand((n, hw, hw, cin), ctx, dtype)
    w = _rand((cout, k, k, cin), ctx, dtype, 0.05)

    def fn(x, w):
        return nd.Convolution(x, w, kernel=(k, k), stride=(stride, stride), pad=(k // 2, k // 2), num_filter=cout,
                              no_bias=True, layout='NHWC')
    ho = hw // stride
    fl = 2.0 * n * ho * ho * cout * cin * k * k
    return dict(inputs=[x, w], fn=fn, fwd_flops=fl, bwd_flops=2 * fl)


def case_fc(ctx, dtype, small, m=8192, k=768, n=3072):
    if small:
        m //= 8
    x, w, b = _rand((m, k), ctx, dtype), _rand((n, k), ctx, dtype, 0.05), _rand((n,), ctx, dtype)

    def fn(x, w, b):
        return nd.FullyConnected(x, w, b, num_hidden=n, flatten=False)
    fl = 2.0 * m * n * k
    return dict(inputs=[x, w, b], fn=fn, fwd_flops=fl, bwd_flops=2 * fl)


def case_softmax(ctx, dtype, small, log=False):
    rows, c = (4096, 1000) if small else (65536, 1000)
    x = _rand((rows, c), ctx, dtype)
    fn = (lambda x: nd.log_softmax(x, axis=-1)) if log else (lambda x: nd.softmax(x, axis=-1))
    nb = x.size * _esize(dtype)
    return dict(inputs=[x], fn=fn, fwd_bytes=2 * nb, bwd_bytes=3 * nb)


def case_layernorm(ctx, dtype, small):
    rows, c = (4096, 768) if small else (65536, 768)
    x, g, b = _rand((rows, c), ctx, dtype), _rand((c,), ctx, 'float32'), _rand((c,), ctx, 'float32')
    nb = x.size * _esize(dtype)
    return dict(inputs=[x, g, b], fn=lambda x, g, b: nd.LayerNorm(x, g, b, axis=-1, eps=1e-5), fwd_bytes=2 * nb,
                bwd_bytes=3 * nb)


def case_maxpool(ctx, dtype, small):
    n = 32 if small else 256
    x = _rand((n, 112, 112, 64), ctx, dtype)
    nb = x.size * _esize(dtype)

    def fn(x):
        return nd.Pooling(x, kernel=(3, 3), stride=(2, 2), pad=(1, 1), pool_type='max', layout='NHWC')
    return dict(inputs=[x], fn=fn, fwd_bytes=nb * 1.25 + nb / 8, bwd_bytes=nb * 1.25 + nb / 8)


def case_attention(ctx, dtype, small, dropout=0.0, t=128, heads=12):
    n = max(1, (16 if small else 64) * 128 // t)            # the same number of tokens at every sequence length
    c = heads * 64
    qkv = _rand((n, t, 3 * c), ctx, dtype, 0.5)
    fl = 4.0 * n * heads * t * t * 64            # QKt and PV

    def fn(qkv):
        return nd.contrib.fused_self_attention(qkv, heads=heads, dropout=dropout, layout='NTC')
    nb = qkv.size * _esize(dtype)
    return dict(inputs=[qkv], fn=fn, fwd_flops=fl, bwd_flops=2.5 * fl, fwd_bytes=nb * 4 / 3, bwd_bytes=nb * (2 + 2 / 3))


def case_gelu(ctx, dtype, small):
    rows, c = (8192, 3072) if small else (65536, 3072)
    x = _rand((rows, c), ctx, dtype)
    nb = x.size * _esize(dtype)
    return dict(inputs=[x], fn=lambda x: nd.LeakyReLU(x, act_type='gelu'), fwd_bytes=2 * nb, bwd_bytes=3 * nb)


def case_dropout_add(ctx, dtype, small):
    rows, c = (8192, 768) if small else (262144, 768)
    x, r = _rand((rows, c), ctx, dtype), _rand((rows, c), ctx, dtype)
    nb = x.size * _esize(dtype)

    def fn(x, r):
        with mx.autograd.train_mode():
            return nd.contrib.dropout_add(x, r, p=0.1)
    return dict(inputs=[x, r], fn=fn, fwd_bytes=3 * nb, bwd_bytes=2 * nb)


def case_embedding(ctx, dtype, small):
    n, rows, d = (8192, 30522, 768) if small else (65536, 30522, 768)
    idx = nd.array(np.random.RandomState(0).randint(0, rows, (n,)), ctx=ctx, dtype='int32')
    w = _rand((rows, d), ctx, dtype)
    nb = n * d * _esize(dtype)
    # forward: gather n rows, write n rows; backward: read n rows of dy, zero and write the table gradient
    return dict(inputs=[w], fn=lambda w: nd.Embedding(idx, w, input_dim=rows, output_dim=d), fwd_bytes=2 * nb,
                bwd_bytes=nb + 2 * rows * d * _esize(dtype))


def case_avgpool(ctx, dtype, small):
    n = 256
    x = _rand((n, 7, 7, 2048), ctx, dtype)
    nb = x.size * _esize(dtype)

    def fn(x):
        return nd.Pooling(x, global_pool=True, pool_type='avg', kernel=(1, 1), layout='NHWC')
    return dict(inputs=[x], fn=fn, fwd_bytes=nb * (1 + 1 / 49), bwd_bytes=nb * (1 + 1 / 49))


def case_add(ctx, dtype, small):
    n = 2 ** 24 if small else 2 ** 28
    a, b = _rand((n,), ctx, dtype), _rand((n,), ctx, dtype)
    return dict(inputs=[a, b], fn=lambda a, b: a + b, fwd_bytes=3 * n * _esize(dtype), bwd_bytes=0, no_backward=True)


def case_csr_dot(ctx, dtype, small, transpose_a=False, library=False):
    """dot(csr, dense) from the compressed components: 200k x 1M features, 40 non-zeros per row, 64 dense columns (the
    sparse linear / factorisation-machine shape).  ``library``: the tensor library's CSR product on the same data."""
    import scipy.sparse as sp
    from mxnet_b200.ndarray import sparse
    m, k, per_row, n = (20000, 100000, 40, 64) if small else (200000, 1000000, 40, 64)
    rng = np.random.RandomState(0)
    cols = rng.randint(0, k, (m, per_row))
    cols.sort(axis=1)
    mat = sp.csr_matrix((rng.uniform(-1, 1, m * per_row).astype('float32'), cols.reshape(-1), np.arange(0, m * per_row + 1, per_row)),
                        shape=(m, k))
    a = sparse.csr_matrix(mat, ctx=ctx, dtype=dtype)
    rhs = _rand((m if transpose_a else k, n), ctx, dtype)
    es = _esize(dtype)
    # every non-zero gathers (or scatters) one dense row of n values; plus the components and the result
    nbytes = m * per_row * (n * es + es + 8) + (k if transpose_a else m) * n * (4 if transpose_a else es)
    if library:
        data, indices, indptr = a._comp
        t = torch.sparse_csr_tensor(indptr, indices, data, size=(m, k))
        if transpose_a:
            t = t.to_sparse_coo().t().coalesce().to_sparse_csr()

        def fn(rhs):
            return nd.NDArray._from_tensor(t @ rhs._data, ctx)
    else:
        def fn(rhs):
            return sparse.dot(a, rhs, transpose_a=transpose_a)
    return dict(inputs=[rhs], fn=fn, fwd_bytes=nbytes, bwd_bytes=0, no_backward=True)


def case_rnn(ctx, dtype, small, mode='lstm', bidirectional=False):
    """The RNN operator on the shape of the LSTM language model: 2 layers of 650 units, 35 steps, batch 80."""
    from mxnet_b200.ops.nn import rnn_param_size
    T, B, I, H, layers = (35, 80, 650, 650, 2) if not small else (12, 32, 128, 128, 2)
    d = 2 if bidirectional else 1
    rng = np.random.RandomState(0)
    x = _rand((T, B, I), ctx, dtype)
    params = nd.array(rng.uniform(-0.05, 0.05, (rnn_param_size(mode, layers, I, H, bidirectional),)), ctx=ctx, dtype=dtype)
    h0 = nd.zeros((layers * d, B, H), ctx=ctx, dtype=dtype)
    states = [h0] + ([nd.zeros((layers * d, B, H), ctx=ctx, dtype=dtype)] if mode == 'lstm' else [])
    gates = {'lstm': 4, 'gru': 3}.get(mode, 1)
    fl = 2.0 * T * B * gates * H * (I + H) * layers * d          # layer 0 input size equals H here
    if bidirectional:
        fl += 2.0 * T * B * gates * H * H * d                    # second layer reads 2H features

    def fn(x, params):
        with mx.autograd.train_mode():
            return nd.RNN(x, params, *states, state_size=H, num_layers=layers, mode=mode, bidirectional=bidirectional)
    return dict(inputs=[x, params], fn=fn, fwd_flops=fl, bwd_flops=2 * fl)


CASES = {
    'csr_dot_dense': case_csr_dot,
    'csr_dot_dense_library': lambda c, d, s: case_csr_dot(c, d, s, library=True),
    'csr_t_dot_dense': lambda c, d, s: case_csr_dot(c, d, s, transpose_a=True),
    'csr_t_dot_dense_library': lambda c, d, s: case_csr_dot(c, d, s, transpose_a=True, library=True),
    'RNN_lstm': case_rnn,
    'RNN_gru': lambda c, d, s: case_rnn(c, d, s, mode='gru'),
    'RNN_tanh': lambda c, d, s: case_rnn(c, d, s, mode='rnn_tanh'),
    'RNN_lstm_bidirectional': lambda c, d, s: case_rnn(c, d, s, bidirectional=True),
    'BatchNorm': case_batchnorm,
    'BatchNormReLU': lambda c, d, s: case_batchnorm(c, d, s, relu=True),
    'BatchNormAddReLU': lambda c, d, s: case_batchnorm(c, d, s, relu=True, residual=True),
    'Convolution3x3': case_conv,
    'Convolution1x1': lambda c, d, s: case_conv(c, d, s, cin=256, cout=64, k=1),
    'Convolution1x1_wide': lambda c, d, s: case_conv(c, d, s, cin=512, cout=2048, k=1, hw=7),
    'FullyConnected': case_fc,
    'FullyConnected_resnet_head': lambda c, d, s: case_fc(c, d, False, m=256, k=2048, n=1000),
    'softmax': case_softmax,
    'log_softmax': lambda c, d, s: case_softmax(c, d, s, log=True),
    'LayerNorm': case_layernorm,
    'MaxPool3x3s2': case_maxpool,
    'fused_self_attention': case_attention,
    'fused_self_attention_t256': lambda c, d, s: case_attention(c, d, s, t=256),
    'fused_self_attention_t512': lambda c, d, s: case_attention(c, d, s, t=512, heads=16),
    'elemwise_add': case_add,
    'GELU': case_gelu,
    'dropout_add': case_dropout_add,
    'Embedding': case_embedding,
    'GlobalAvgPool': case_avgpool,
}


def run_case(name, ctx, dtype, runs, warmup, small):
    spec = CASES[name](ctx, dtype, small)
    ins, fn = spec['inputs'], spec['fn']
    cuda = ctx.device_type == 'gpu'
    flush = torch.empty(160 * 2 ** 20, dtype=torch.uint8, device=ctx.torch_device) if cuda else None
    backward = not spec.get('no_backward')
    for a in ins:
        if backward:
            a.attach_grad()
    out = None

    def fwd():
        nonlocal out
        if backward:
            with autograd.record():
                out = fn(*ins)
        else:
            out = fn(*ins)
        return out
    head = None
    fwd_ms, bwd_ms = [], []
    for it in range(warmup + runs):
        if cuda:
            flush.zero_()
            e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            e[0].record()
            o = fwd()
            e[1].record()
            if backward:
                if head is None:
                    head = nd.ones(o.shape, ctx=ctx, dtype=o.dtype)
                o.backward(head)
            e[2].record()
            torch.cuda.synchronize()
            t_f, t_b = e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2])
        else:
            t0 = time.perf_counter()
            o = fwd()
            t1 = time.perf_counter()
            if backward:
                if head is None:
                    head = nd.ones(o.shape, ctx=ctx, dtype=o.dtype)
                o.backward(head)
            t2 = time.perf_counter()
            t_f, t_b = (t1 - t0) * 1e3, (t2 - t1) * 1e3
        if it >= warmup:
            fwd_ms.append(t_f)
            bwd_ms.append(t_b)
    res = {'op': name, 'dtype': dtype, 'device': str(ctx), 'runs': runs,
           'inputs': [list(a.shape) for a in ins], 'fwd_ms': float(np.mean(fwd_ms)),
           'bwd_ms': float(np.mean(bwd_ms)) if backward else None}
    for tag, ms in (('fwd', res['fwd_ms']), ('bwd', res['bwd_ms'])):
        if ms is None or ms <= 0:
            continue
        if spec.get(tag + '_bytes'):
            res[tag + '_GBps'] = spec[tag + '_bytes'] / ms / 1e6
        if spec.get(tag + '_flops'):
            res[tag + '_TFLOPs'] = spec[tag + '_flops'] / ms / 1e9
    return res


def gemm_burst(ctx, dtype, reps=50, shapes=None):
    """Kernel-only GEMM throughput: `reps` back-to-back launches between two events, so that host launch
    overhead does not count; the in-tree tcgen05 kernel and the library GEMM on identical operands."""
    from mxnet_b200.ops.cuda import gemm_ops
    td = mx.base.to_torch_dtype(dtype)
    out = []
    for m, n, k in shapes or [(8192, 3072, 768), (8192, 768, 3072), (4096, 4096, 4096), (16384, 1024, 1024), (8192, 8192, 8192),
                              (802816, 64, 256), (200704, 512, 128)]:
        a = torch.randn(m, k, device=ctx.torch_device).to(td)
        b = torch.randn(n, k, device=ctx.torch_device).to(td)
        d = torch.empty(m, n, device=ctx.torch_device, dtype=td)
        res = {'op': 'gemm_burst', 'M': m, 'N': n, 'K': k, 'dtype': dtype, 'reps': reps}
        for name, fn in (('tcgen05', lambda: gemm_ops.gemm_tn(a, b, out=d)), ('single_cta', lambda: gemm_ops.gemm_tn(a, b, out=d)),
                         ('library', lambda: torch.matmul(a, b.t(), out=d))):
            gemm_ops.set_variant(1 if name == 'single_cta' else 0)
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / reps
            res[name + '_us'] = ms * 1e3
            res[name + '_TFLOPs'] = 2.0 * m * n * k / ms / 1e9
        gemm_ops.check_errors()
        res['ratio'] = res['tcgen05_TFLOPs'] / res['library_TFLOPs']
        out.append(res)
    return out


def gemm_batched(ctx, dtype, reps=30):
    """Batched products: the in-tree batched tcgen05 launch against the library's strided-batched GEMM on identical
    operands (the per-head attention products of BERT-base at 64 x 128 tokens, and 32 square products of 1024)."""
    from mxnet_b200.ops.cuda import gemm_ops
    td = mx.base.to_torch_dtype(dtype)
    out = []
    for b, m, n, k, tb in [(768, 128, 128, 64, True), (768, 128, 64, 128, False), (32, 1024, 1024, 1024, False),
                           (32, 1024, 1024, 1024, True)]:
        x = torch.randn(b, m, k, device=ctx.torch_device).to(td)
        y = (torch.randn(b, n, k, device=ctx.torch_device) if tb else torch.randn(b, k, n, device=ctx.torch_device)).to(td)
        res = {'op': 'gemm_batched', 'batch': b, 'M': m, 'N': n, 'K': k, 'transpose_b': tb, 'dtype': dtype, 'reps': reps}
        for name, fn in (('tcgen05', lambda: gemm_ops.bgemm(x, False, y, not tb)),
                         ('library', lambda: torch.bmm(x, y.transpose(1, 2) if tb else y))):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / reps
            res[name + '_us'] = round(ms * 1e3, 1)
            res[name + '_TFLOPs'] = round(2.0 * b * m * n * k / ms / 1e9, 1)
        gemm_ops.check_errors()
        res['ratio'] = round(res['tcgen05_TFLOPs'] / res['library_TFLOPs'], 3)
        out.append(res)
    return out


def gemm_int8(ctx, reps=30):
    """int8 x int8 -> int32 products: the in-tree ``tcgen05.mma.kind::i8`` kernel against the library's int8 GEMM
    (``torch._int_mm``, cuBLASLt) on identical operands; TOP/s counts 2 M N K integer operations."""
    from mxnet_b200.ops.cuda import gemm_ops
    out = []
    for m, n, k in [(8192, 8192, 8192), (8192, 3072, 768), (8192, 768, 3072), (4096, 4096, 4096), (256, 1000, 2048)]:
        a = torch.randint(-128, 128, (m, k), device=ctx.torch_device, dtype=torch.int32).to(torch.int8)
        b = torch.randint(-128, 128, (n, k), device=ctx.torch_device, dtype=torch.int32).to(torch.int8)
        d = torch.empty(m, n, dtype=torch.int32, device=ctx.torch_device)
        res = {'op': 'gemm_int8', 'M': m, 'N': n, 'K': k, 'reps': reps}
        cases = [('tcgen05', lambda: gemm_ops.gemm_i8(a, b, out=d))]
        if n % 8 == 0:
            cases.append(('library', lambda: torch._int_mm(a, b.t())))
        for name, fn in cases:
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / reps
            res[name + '_us'] = round(ms * 1e3, 1)
            res[name + '_TOPs'] = round(2.0 * m * n * k / ms / 1e9, 1)
        gemm_ops.check_errors()
        if 'library_TOPs' in res:
            res['ratio'] = round(res['tcgen05_TOPs'] / res['library_TOPs'], 3)
        out.append(res)
    return out


def gemm_layouts(ctx, dtype, reps=30):
    """The three products of a FullyConnected layer on BERT-base shapes (8192 tokens): forward y = x w^T (both K-major),
    data gradient dx = dy w (w MN-major), weight gradient dw = dy^T x (both MN-major); in-tree kernel against the
    library on identical operands, `reps` back-to-back launches between two events."""
    from mxnet_b200.ops.cuda import gemm_ops
    td = mx.base.to_torch_dtype(dtype)
    out = []
    tokens = 8192
    for cin, cout in [(768, 2304), (768, 768), (768, 3072), (3072, 768)]:
        x = torch.randn(tokens, cin, device=ctx.torch_device).to(td)
        w = torch.randn(cout, cin, device=ctx.torch_device).to(td)
        dy = torch.randn(tokens, cout, device=ctx.torch_device).to(td)
        cases = {
            'fwd': (lambda: gemm_ops.gemm_tn(x, w), lambda: torch.matmul(x, w.t())),
            'dgrad': (lambda: gemm_ops.gemm(dy, w, False, True), lambda: torch.matmul(dy, w)),
            'wgrad': (lambda: gemm_ops.gemm(dy, x, True, True), lambda: torch.matmul(dy.t(), x)),
        }
        for kind, (own, libf) in cases.items():
            res = {'op': 'gemm_layouts', 'layer': '%d->%d' % (cin, cout), 'product': kind, 'dtype': dtype, 'reps': reps}
            for name, fn in (('tcgen05', own), ('single_cta', own), ('library', libf)):
                gemm_ops.set_variant(1 if name == 'single_cta' else 0)
                for _ in range(3):
                    fn()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(reps):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                ms = e0.elapsed_time(e1) / reps
                res[name + '_us'] = round(ms * 1e3, 1)
                res[name + '_TFLOPs'] = round(2.0 * tokens * cin * cout / ms / 1e9, 1)
            gemm_ops.check_errors()
            res['ratio'] = round(res['tcgen05_TFLOPs'] / res['library_TFLOPs'], 3)
            out.append(res)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--op', action='append', help='case name (repeatable); default: all')
    ap.add_argument('--dtype', default='float16')
    ap.add_argument('--runs', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--small', action='store_true', help='shapes sized for a profiler capture (a few hundred MB)')
    ap.add_argument('--list', action='store_true')
    ap.add_argument('--shape', type=int, nargs=3, metavar=('M', 'N', 'K'), help='gemm_burst: this one product only')
    ap.add_argument('--reps', type=int, default=50, help='gemm_burst: launches between the two events')
    args = ap.parse_args()
    if args.list:
        print('\n'.join(CASES))
        return 0
    cuda = torch.cuda.is_available()
    ctx = mx.gpu(0) if cuda else mx.cpu(0)
    dtype = args.dtype if cuda else 'float32'
    small = args.small or not cuda
    for name in (args.op or list(CASES)):
        if name == 'gemm_layouts':
            if ctx.device_type == 'gpu':
                for r in gemm_layouts(ctx, dtype):
                    print(json.dumps(r), flush=True)
            continue
        if name == 'gemm_batched':
            if cuda:
                for r in gemm_batched(ctx, dtype):
                    print(json.dumps(r), flush=True)
            continue
        if name == 'gemm_int8':
            if cuda:
                for r in gemm_int8(ctx):
                    print(json.dumps(r), flush=True)
            continue
        if name == 'gemm_burst':
            if cuda:
                for r in gemm_burst(ctx, dtype, reps=args.reps, shapes=[tuple(args.shape)] if args.shape else None):
                    print(json.dumps(r), flush=True)
            continue
        print(json.dumps(run_case(name, ctx, dtype, args.runs, args.warmup, small)), flush=True)
    return 0


if __name__ == '__main__':
    sys.exit(main())

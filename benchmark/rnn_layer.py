"""One recurrent layer, forward and forward + backward: tensor-core recurrence, fp32-pipe recurrence, library recurrence.

    python -m benchmark.rnn_layer --mode gru --shapes 35x80x650x650,50x64x1024x1024 --dtypes float32,float16

Times, with CUDA events after warm-up, the three implementations of one LSTM or GRU layer on the same tensors:
``rnn_ops._LSTMLayerTC`` / ``_GRULayerTC`` (tcgen05 recurrence), ``rnn_ops._LSTMLayer`` / ``_RecurrentLayer`` (cooperative
fp32-pipe kernels) and the cuDNN recurrence behind ``torch._VF.lstm`` / ``torch._VF.gru``.  Prints one JSON line per case.
"""
import argparse
import json

import torch


def _time_us(fn, reps, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps * 1e3


def run_case(mode, dtype, T, B, I, H, reps):
    from mxnet_b200.ops.cuda import rnn_ops
    G = 4 if mode == 'lstm' else 3
    dev = 'cuda'
    x = torch.randn(T, B, I, device=dev).to(dtype).requires_grad_(True)
    ws = [(torch.randn(G * H, I, device=dev) * 0.1).to(dtype).requires_grad_(True),
          (torch.randn(G * H, H, device=dev) * 0.1).to(dtype).requires_grad_(True),
          (torch.randn(G * H, device=dev) * 0.1).to(dtype).requires_grad_(True),
          (torch.randn(G * H, device=dev) * 0.1).to(dtype).requires_grad_(True)]
    states = [torch.zeros(B, H, device=dev, dtype=dtype).requires_grad_(True) for _ in range(2 if mode == 'lstm' else 1)]
    leaves = [x] + ws + states
    if mode == 'lstm':
        impls = {'tcgen05': lambda tr: rnn_ops._LSTMLayerTC.apply(x, *ws, *states, tr),
                 'fp32_pipe': lambda tr: rnn_ops._LSTMLayer.apply(x, *ws, *states, tr),
                 'library': lambda tr: torch._VF.lstm(x, tuple(s[None] for s in states), ws, True, 1, 0.0, tr, False, False)}
        if not rnn_ops.tc_supported(dtype, B, H):
            impls.pop('tcgen05')
    else:
        impls = {'tcgen05': lambda tr: rnn_ops._GRULayerTC.apply(x, *ws, *states, tr),
                 'fp32_pipe': lambda tr: rnn_ops._RecurrentLayer.apply(x, *ws, *states, rnn_ops._MODES['gru'], tr),
                 'library': lambda tr: torch._VF.gru(x, states[0][None], ws, True, 1, 0.0, tr, False, False)}
        if not rnn_ops.gru_tc_supported(dtype, B, H):
            impls.pop('tcgen05')
    rec = {'mode': mode, 'dtype': str(dtype).replace('torch.', ''), 'T': T, 'N': B, 'input': I, 'hidden': H, 'unit': 'us'}
    for name, fn in impls.items():
        def fwd(fn=fn):
            with torch.no_grad():
                fn(False)

        def fwd_bwd(fn=fn):
            out = fn(True)
            torch.autograd.grad([out[0].float().sum() + out[1].float().sum()], leaves, allow_unused=True)
        rec[name] = {'forward': round(_time_us(fwd, reps), 1), 'forward_backward': round(_time_us(fwd_bwd, reps), 1)}
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--mode', default='gru', choices=['lstm', 'gru'])
    ap.add_argument('--shapes', default='35x80x650x650,50x64x1024x1024', help='TxNxIxH, comma separated')
    ap.add_argument('--dtypes', default='float32,float16')
    ap.add_argument('--reps', type=int, default=20)
    args = ap.parse_args()
    import warnings
    warnings.filterwarnings('ignore', message='RNN module weights are not part')
    for dname in args.dtypes.split(','):
        for shape in args.shapes.split(','):
            T, B, I, H = (int(v) for v in shape.split('x'))
            print(json.dumps(run_case(args.mode, getattr(torch, dname), T, B, I, H, args.reps)), flush=True)


if __name__ == '__main__':
    main()

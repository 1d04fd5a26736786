"""FullyConnected / matmul on the tcgen05 GEMM kernel (``gemm_tcgen05.cu``).

Forward, data gradient and weight gradient all run on the hand-written kernel: it takes each operand
either with the contraction axis contiguous ("K-major") or with the output axis contiguous
("MN-major"), so no transposed copies are made."""
import torch

from . import lib, ptr, stream_ptr, count_launch, check
from ._util import dt, require, job_wide

_ACT = {None: 0, 'relu': 1, 'gelu': 2}
_err = {}
_tuned = {}          # (product, dtype, M, N, K, bias, act) -> True when the in-tree kernel won
_flush = {}
_tuned_us = {}       # key -> (in-tree, library) microseconds measured by the autotuner on this rank
_ws = {}
_MARGIN = 1.02      # ties (within 2 %) go to the in-tree kernel


def _autotune():
    from ... import env
    return env.get('MXNET_B200_GEMM_AUTOTUNE')


def _time_us(fn, reps=5):
    """Median device time with the L2 cache flushed before every run."""
    dev = torch.cuda.current_device()
    flush = _flush.get(dev)
    if flush is None:
        flush = _flush[dev] = torch.empty(192 << 20, dtype=torch.uint8, device='cuda')
    fn()
    times = []
    for _ in range(reps):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e3)
    times.sort()
    return times[len(times) // 2]


def use_own(key, own_fn, lib_fn):
    """Per-shape choice between the in-tree kernel and the library GEMM (``MXNET_B200_GEMM_AUTOTUNE``, the counterpart
    of the convolution autotune): timed once, outside of graph capture, on the first call with this key."""
    if not _autotune():
        return True
    hit = _tuned.get(key)
    if hit is None:
        if torch.cuda.is_current_stream_capturing():
            return True
        with torch.no_grad():
            t_own, t_lib = _time_us(own_fn), _time_us(lib_fn)
            _tuned_us[key] = (round(t_own, 1), round(t_lib, 1))
            hit = _tuned[key] = job_wide(t_own <= _MARGIN * t_lib)
    return hit


def tuned_choices():
    return dict(_tuned)


def tuned_times():
    """{(product, dtype, M, N, K, bias, act): (in-tree, library) microseconds with a cold L2, as timed on this rank}."""
    return dict(_tuned_us)


def _error_flag(device):
    f = _err.get(device)
    if f is None:
        f = _err[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return f


def _workspace(device):
    """Stream-K workspace of the GEMM kernel (fp32 slots for partial tiles): one buffer per device, created on first
    use.  Launches that share it must not overlap: the framework issues its GEMMs on
    the device's compute stream (graph replays included).  Never created while a graph is being captured (the memory would
    belong to that graph); such a call runs without stream-K."""
    ws = _ws.get(device)
    if ws is None:
        if torch.cuda.is_current_stream_capturing():
            return None
        ws = _ws[device] = torch.empty(int(lib().mxb_gemm_workspace_bytes()), dtype=torch.uint8, device=device)
    return ws


def check_errors():
    """Raise if any GEMM CTA gave up waiting on a barrier (the result would be incomplete)."""
    for dev, f in _err.items():
        if int(f.item()) != 0:
            f.zero_()
            raise RuntimeError('tcgen05 GEMM reported a barrier time-out on %s' % dev)


def set_variant(v):
    """Kernel selection of later ``gemm`` calls: 0 = per shape (CTA-pair kernel where it applies), 1 = single-CTA kernel
    only.  For benchmarks and tests that compare the two."""
    lib().mxb_gemm_set_variant(int(v))


def supported(M, N, K):
    return M >= 1 and N >= 8 and K >= 8 and K % 8 == 0 and N % 8 == 0


def gemm_tn(a, b, bias=None, act=None, out=None):
    """``act(a @ b.T + bias)`` with a: [M, K], b: [N, K] (row-major, K contiguous)."""
    if not a.is_contiguous():
        a = a.contiguous()
    if not b.is_contiguous():
        b = b.contiguous()
    M, K = a.shape
    N = b.shape[0]
    require(a, 'a')
    require(b, 'b', dtype=a.dtype, device=a.device, shape=(N, K))
    if out is not None:
        require(out, 'out', dtype=a.dtype, device=a.device, shape=(M, N))
    if bias is not None:
        require(bias, 'bias', numel=N, device=a.device)
    return gemm(a, b, False, False, bias, act, out)


def gemm(a, b, a_mn=False, b_mn=False, bias=None, act=None, out=None):
    """``act(op(a) @ op(b) + bias)``.  ``a`` is [M, K] (``a_mn=False``) or [K, M] (``a_mn=True``); ``b`` is
    [N, K] (``b_mn=False``) or [K, N] (``b_mn=True``); all row-major contiguous."""
    if not a.is_contiguous():
        a = a.contiguous()
    if not b.is_contiguous():
        b = b.contiguous()
    K, M = (a.shape if a_mn else a.shape[::-1])
    Kb, N = (b.shape if b_mn else b.shape[::-1])
    require(a, 'a')
    require(b, 'b', dtype=a.dtype, device=a.device)
    if K != Kb:
        raise ValueError('contraction sizes differ: %d vs %d' % (K, Kb))
    d = out if out is not None else torch.empty(M, N, dtype=a.dtype, device=a.device)
    require(d, 'out', dtype=a.dtype, device=a.device, shape=(M, N))
    if bias is not None:
        if bias.dtype != a.dtype:
            bias = bias.to(a.dtype)
        require(bias, 'bias', numel=N, device=a.device)
    L = lib()
    rc = L.mxb_gemm_ws(dt(a), ptr(a), ptr(b), ptr(d), ptr(bias), M, N, K, a.shape[1], b.shape[1], N,
                       1 if a_mn else 0, 1 if b_mn else 0, _ACT[act], ptr(_workspace(a.device)), ptr(_error_flag(a.device)),
                       stream_ptr(a.device))
    check(rc, 'gemm')
    count_launch(1)
    return d


def gemm_i8_supported(a, b):
    """int8 CUDA operands [M, K] and [N, K] whose rows a TMA descriptor can address (K a multiple of 16)."""
    return (a.is_cuda and b.is_cuda and a.dtype == torch.int8 and b.dtype == torch.int8 and a.dim() == 2 and b.dim() == 2
            and a.shape[1] == b.shape[1] and a.shape[1] % 16 == 0 and a.shape[0] >= 1 and b.shape[0] >= 1)


def gemm_i8(a, b, bias=None, out=None):
    """``a @ b.T + bias`` with int8 ``a`` [M, K], ``b`` [N, K], int32 ``bias`` [N] and int32 result, on the
    ``tcgen05.mma.kind::i8`` kernel (``gemm_i8.cu``): exact integer arithmetic with 32-bit accumulation."""
    if not a.is_contiguous():
        a = a.contiguous()
    if not b.is_contiguous():
        b = b.contiguous()
    require(a, 'a', dtype=torch.int8)
    require(b, 'b', dtype=torch.int8, device=a.device)
    (M, K), (N, Kb) = a.shape, b.shape
    if K != Kb:
        raise ValueError('contraction sizes differ: %d vs %d' % (K, Kb))
    if K % 16:
        raise ValueError('the int8 kernel needs K to be a multiple of 16, got %d' % K)
    d = out if out is not None else torch.empty(M, N, dtype=torch.int32, device=a.device)
    require(d, 'out', dtype=torch.int32, device=a.device, shape=(M, N))
    if bias is not None:
        require(bias, 'bias', numel=N, dtype=torch.int32, device=a.device)
    rc = lib().mxb_gemm_i8(ptr(a), ptr(b), ptr(d), ptr(bias), M, N, K, K, K, N, ptr(_error_flag(a.device)), stream_ptr(a.device))
    check(rc, 'gemm_i8')
    count_launch(1)
    return d


def operand_ok(t):
    """Row pitch a multiple of 8 elements and a 16-byte aligned base: what a TMA descriptor needs."""
    return t.dim() == 2 and t.shape[1] % 8 == 0 and t.shape[0] >= 1 and t.data_ptr() % 16 == 0


def _bias_grad(dy):
    """fp32 column sums of dy: the two-stage kernel, or the library reduction with fp32 accumulation."""
    from . import elementwise_ops as ew
    from ... import env
    if env.get('MXNET_B200_ELEMENTWISE') and ew.colsum_supported(dy):
        return ew.colsum(dy)
    return dy.sum(0, dtype=torch.float32)


def _lib_linear(x, w, bias, act):
    y = torch.nn.functional.linear(x, w, bias.to(x.dtype) if bias is not None and bias.dtype != x.dtype else bias)
    if act == 'relu':
        y = torch.relu(y)
    elif act == 'gelu':
        y = torch.nn.functional.gelu(y)
    return y


class LinearFn(torch.autograd.Function):
    """y = act(x @ w.T + b)."""

    @staticmethod
    def forward(ctx, x, w, bias, act):
        key = ('fwd', x.dtype, x.shape[0], w.shape[0], x.shape[1], bias is not None, act)
        if use_own(key, lambda: gemm_tn(x, w, bias, act), lambda: _lib_linear(x, w, bias, act)):
            y = gemm_tn(x, w, bias, act)
        else:
            y = _lib_linear(x, w, bias, act)
        ctx.save_for_backward(x, w, y if act is not None else None)
        ctx.act, ctx.has_bias = act, bias is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, y = ctx.saved_tensors
        dy = dy.contiguous()
        if ctx.act == 'relu':
            dy = dy * (y > 0).to(dy.dtype)
        elif ctx.act == 'gelu':
            raise RuntimeError('gelu epilogue has no fused backward; use act=None for training')
        dx = dw = db = None
        ok = operand_ok(dy) and operand_ok(w) and operand_ok(x)
        shape = (x.dtype, x.shape[0], w.shape[0], x.shape[1])
        if ctx.needs_input_grad[0]:
            # dx[M, K] = dy[M, N] . w[N, K]: w is read as an MN-major operand ([contraction, output])
            if ok and use_own(('dgrad',) + shape, lambda: gemm(dy, w, False, True), lambda: dy @ w):
                dx = gemm(dy, w, False, True)
            else:
                dx = dy @ w
        if ctx.needs_input_grad[1]:
            # dw[N, K] = dy[M, N]^T . x[M, K]: both operands MN-major, contraction over the batch axis
            if ok and use_own(('wgrad',) + shape, lambda: gemm(dy, x, True, True), lambda: torch.matmul(dy.t(), x)):
                dw = gemm(dy, x, True, True)
            else:
                dw = torch.matmul(dy.t(), x)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = _bias_grad(dy).to(ctx.bias_dtype)
        return dx, dw, db, None


class MatmulFn(torch.autograd.Function):
    """c = a @ b for 2-D row-major operands."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return gemm(a, b, False, True)

    @staticmethod
    def backward(ctx, dc):
        a, b = ctx.saved_tensors
        dc = dc.contiguous()
        da = db = None
        ok = operand_ok(dc) and operand_ok(a) and operand_ok(b)
        if ctx.needs_input_grad[0]:
            da = gemm(dc, b, False, False) if ok else dc @ b.t()          # dc[M, N] . b[K, N]^T
        if ctx.needs_input_grad[1]:
            db = gemm(a, dc, True, True) if ok else torch.matmul(a.t(), dc)  # a[M, K]^T . dc[M, N]
        return da, db


def bgemm(a, a_mn, b, b_mn, out=None):
    """Batched product on the tcgen05 kernel: ``out[i] = op(a[i]) @ op(b[i])`` for 3-D contiguous half-precision operands.
    ``a`` is ``[batch, rows, k]`` (``a_mn=False``) or ``[batch, k, rows]``; ``b`` is ``[batch, cols, k]`` (``b_mn=False``) or
    ``[batch, k, cols]``; the result is ``[batch, rows, cols]``.  All matrices of the batch form one persistent grid."""
    if not a.is_contiguous():
        a = a.contiguous()
    if not b.is_contiguous():
        b = b.contiguous()
    nb = a.shape[0]
    K, M = (a.shape[1], a.shape[2]) if a_mn else (a.shape[2], a.shape[1])
    Kb, N = (b.shape[1], b.shape[2]) if b_mn else (b.shape[2], b.shape[1])
    require(a, 'a')
    require(b, 'b', dtype=a.dtype, device=a.device)
    if K != Kb or b.shape[0] != nb:
        raise ValueError('batched product: operands disagree (%s, %s)' % (tuple(a.shape), tuple(b.shape)))
    d = out if out is not None else torch.empty(nb, M, N, dtype=a.dtype, device=a.device)
    require(d, 'out', dtype=a.dtype, device=a.device, shape=(nb, M, N))
    rc = lib().mxb_gemm_batched(dt(a), ptr(a), ptr(b), ptr(d), None, nb, M, N, K, a.shape[2], b.shape[2], N,
                                a.shape[1] * a.shape[2], b.shape[1] * b.shape[2], M * N, 1 if a_mn else 0, 1 if b_mn else 0, 0,
                                ptr(_workspace(a.device)), ptr(_error_flag(a.device)), stream_ptr(a.device))
    check(rc, 'batched gemm')
    count_launch(1)
    return d


def bgemm_supported(a, b):
    """3-D half-precision CUDA operands whose innermost extents are multiples of 8 (16-byte rows for the copy engine)."""
    return (a.dim() == 3 and b.dim() == 3 and a.is_cuda and a.dtype == b.dtype and a.dtype in (torch.float16, torch.bfloat16)
            and a.shape[0] == b.shape[0] and a.shape[0] >= 1 and a.shape[2] % 8 == 0 and b.shape[2] % 8 == 0
            and a.shape[1] % 8 == 0 and b.shape[1] % 8 == 0 and a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0)


def _lib_bmm(a, ta, b, tb):
    return torch.bmm(a.transpose(1, 2) if ta else a, b.transpose(1, 2) if tb else b)


class BatchMatmulFn(torch.autograd.Function):
    """``c[i] = op(a[i]) @ op(b[i])`` (``batch_dot`` with its ``transpose_a`` / ``transpose_b`` flags): forward and both
    gradients are batched products on the same kernel, each read in the layout it is stored in (no transposed copies);
    per shape and product the faster of this kernel and the library's strided-batched GEMM is kept
    (``MXNET_B200_GEMM_AUTOTUNE``)."""

    @staticmethod
    def forward(ctx, a, b, ta, tb):
        ctx.save_for_backward(a, b)
        ctx.flags = (ta, tb)
        key = ('bfwd', a.dtype, tuple(a.shape), tuple(b.shape), ta, tb)
        if use_own(key, lambda: bgemm(a, ta, b, not tb), lambda: _lib_bmm(a, ta, b, tb)):
            return bgemm(a, ta, b, not tb)
        return _lib_bmm(a, ta, b, tb)

    @staticmethod
    def backward(ctx, dc):
        a, b = ctx.saved_tensors
        ta, tb = ctx.flags
        dc = dc.contiguous()
        da = db = None
        ok = bgemm_supported(dc, dc)
        if ctx.needs_input_grad[0]:
            own = (lambda: bgemm(dc, False, b, tb)) if not ta else (lambda: bgemm(b, tb, dc, False))
            ref = (lambda: _lib_bmm(dc, False, b, not tb)) if not ta else (lambda: _lib_bmm(b, tb, dc, True))
            da = own() if ok and use_own(('bdgrad_a', a.dtype, tuple(a.shape), tuple(b.shape), ta, tb), own, ref) else ref()
        if ctx.needs_input_grad[1]:
            own = (lambda: bgemm(a, not ta, dc, True)) if not tb else (lambda: bgemm(dc, True, a, not ta))
            ref = (lambda: _lib_bmm(a, not ta, dc, False)) if not tb else (lambda: _lib_bmm(dc, True, a, ta))
            db = own() if ok and use_own(('bdgrad_b', a.dtype, tuple(a.shape), tuple(b.shape), ta, tb), own, ref) else ref()
        return da, db, None, None

"""Fused LSTM on the persistent recurrence kernels (``lstm.cu``).

One layer = an input-projection GEMM over all time steps (tcgen05 kernel for half precision), the
cooperative recurrence kernel, and in backward the reverse recurrence plus three GEMMs over the saved
gate gradients (weight gradients contract over time*batch: MN-major operands)."""
import torch

from . import lib, ptr, stream_ptr, count_launch, check
from ._util import dt, require, job_wide


def supported(data, state_size, num_layers, mode='lstm'):
    if not data.is_cuda or data.dim() != 3 or data.numel() == 0:
        return False
    if mode == 'lstm' and tc_supported(data.dtype, int(data.shape[1]), int(state_size)):
        return True
    if mode == 'gru' and gru_tc_supported(data.dtype, int(data.shape[1]), int(state_size)):
        return True
    return bool(lib().mxb_lstm_supported(int(data.shape[1]), int(state_size)))


_tuned = {}
_gru_ok = {}          # (dtype, batch, hidden size, device) -> the tensor-core GRU kernels fit the device
_tuned_us = {}        # configuration -> (in-tree, library) microseconds measured by the autotuner on this rank


def use_own(key, own_fn, lib_fn, inputs, training):
    """Whether the RNN configuration `key` runs on the in-tree recurrence kernels (``MXNET_B200_RNN``).  In auto mode
    both implementations run the forward pass (plus the backward pass when training) on the caller's tensors once,
    timed on the device, and the faster one is remembered for the configuration."""
    from ... import env
    mode = str(env.get('MXNET_B200_RNN')).lower()
    if mode in ('1', 'true', 'on', 'force'):
        return True
    if mode in ('0', 'false', 'off'):
        return False
    hit = _tuned.get(key)
    if hit is None:
        if torch.cuda.is_current_stream_capturing():
            return True                    # cannot time inside a capture; the eager warm-up run normally comes first
        from .conv_ops import _time_us

        def run(fn):
            def step():
                if not training:
                    with torch.no_grad():
                        fn(*inputs)
                    return
                leaves = [t.detach().requires_grad_(True) if t.is_floating_point() else t for t in inputs]
                with torch.enable_grad():
                    out = fn(*leaves)
                    outs = [o for o in (out if isinstance(out, (tuple, list)) else (out,)) if o.requires_grad]
                    torch.autograd.grad([o.float().sum() for o in outs], [l for l in leaves if l.requires_grad],
                                        allow_unused=True)
            return step
        rng = torch.cuda.get_rng_state()
        try:
            t_own, t_lib = _time_us(run(own_fn), reps=3), _time_us(run(lib_fn), reps=3)
            _tuned_us[key] = (round(t_own, 1), round(t_lib, 1))
            hit = _tuned[key] = job_wide(t_own <= 1.02 * t_lib)
        finally:
            torch.cuda.set_rng_state(rng)
    return hit


def tuned_choices():
    """{(mode, dtype, T, N, input size, state size, layers, bidirectional, training): in-tree kernels chosen}."""
    return dict(_tuned)


def tuned_times():
    """{configuration: (in-tree, library) microseconds of forward (+ backward) as timed by the autotuner}."""
    return dict(_tuned_us)


class _tf32_products(object):
    """fp32 library GEMMs inside the block run with tf32 operands and fp32 accumulation: the precision of the
    tensor-core recurrence they surround (and of the library recurrence, whose internal products are tf32 as well)."""

    def __enter__(self):
        self._old = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True

    def __exit__(self, *exc):
        torch.backends.cuda.matmul.allow_tf32 = self._old


def _mm(a, b, a_mn, b_mn, tf32=False):
    """op(a) @ op(b) with the tcgen05 kernel when the operands qualify, else the library."""
    from . import gemm_ops
    if a.dtype in (torch.float16, torch.bfloat16) and gemm_ops.operand_ok(a) and gemm_ops.operand_ok(b):
        return gemm_ops.gemm(a, b, a_mn, b_mn)
    aa = a.t() if a_mn else a
    bb = b if b_mn else b.t()
    if tf32 and a.dtype == torch.float32:
        with _tf32_products():
            return aa @ bb
    return aa @ bb


def _barrier_words(device):
    return torch.zeros(2, dtype=torch.int32, device=device)


class _LSTMLayer(torch.autograd.Function):
    """y, hT, cT = lstm(x[T,B,I], w_ih[4H,I], w_hh[4H,H], b_ih[4H], b_hh[4H], h0[B,H], c0[B,H])."""

    @staticmethod
    def forward(ctx, x, w_ih, w_hh, b_ih, b_hh, h0, c0, training):
        L = lib()
        T, B, I = x.shape
        H = w_hh.shape[1]
        x = x.contiguous()
        w_ih, w_hh, h0, c0 = w_ih.contiguous(), w_hh.contiguous(), h0.contiguous(), c0.contiguous()
        for t, name, shape in ((w_ih, 'w_ih', (4 * H, I)), (w_hh, 'w_hh', (4 * H, H)), (h0, 'h0', (B, H)), (c0, 'c0', (B, H))):
            require(t, name, dtype=x.dtype, device=x.device, shape=shape)
        bias = (b_ih.float() + b_hh.float()).to(x.dtype)
        require(bias, 'bias', numel=4 * H, device=x.device)
        from . import gemm_ops
        x2 = x.reshape(T * B, I)
        if x.dtype in (torch.float16, torch.bfloat16) and gemm_ops.operand_ok(x2) and gemm_ops.operand_ok(w_ih):
            xproj = gemm_ops.gemm(x2, w_ih, False, False, bias)
        else:
            xproj = torch.addmm(bias, x2, w_ih.t())
        y = torch.empty(T, B, H, dtype=x.dtype, device=x.device)
        hT, cT = torch.empty_like(h0), torch.empty_like(c0)
        Bp = L.mxb_lstm_bp(B)        # the kernels keep their own tensors k-major: [T, rows, Bp]
        gates = torch.empty(T, 4 * H, Bp, dtype=x.dtype, device=x.device) if training else None
        cs = torch.empty(T, H, Bp, dtype=torch.float32, device=x.device) if training else None
        hbuf = torch.empty(L.mxb_lstm_exchange_bytes(B, H), dtype=torch.uint8, device=x.device)
        bar = _barrier_words(x.device)
        check(L.mxb_lstm_forward(dt(x), ptr(xproj), ptr(w_hh), ptr(h0), ptr(c0), ptr(y), ptr(hT), ptr(cT), ptr(gates), ptr(cs),
                                 ptr(hbuf), ptr(bar), T, B, H, stream_ptr(x.device)), 'lstm_forward')
        count_launch(1)
        ctx.save_for_backward(x, w_ih, w_hh, h0, c0, y, gates, cs)
        ctx.bias_dtypes = (b_ih.dtype, b_hh.dtype)
        ctx.fwd_bar = bar
        ctx.set_materialize_grads(False)
        return y, hT, cT

    @staticmethod
    def backward(ctx, dy, dhT, dcT):
        x, w_ih, w_hh, h0, c0, y, gates, cs = ctx.saved_tensors
        if gates is None:
            raise RuntimeError('LSTM backward needs a forward pass in training mode')
        L = lib()
        T, B, I = x.shape
        H = w_hh.shape[1]
        dy = torch.zeros_like(y) if dy is None else dy.contiguous()
        require(dy, 'out_grad', dtype=x.dtype, device=x.device, shape=y.shape)
        dhT = dhT.contiguous() if dhT is not None else None
        dcT = dcT.contiguous() if dcT is not None else None
        dgates_t = torch.empty_like(gates)                      # [T, 4H, Bp], k-major
        dh0, dc0 = torch.empty_like(h0), torch.empty_like(c0)
        bar = _barrier_words(x.device)
        check(L.mxb_lstm_backward(dt(x), ptr(dy), ptr(dhT), ptr(dcT), ptr(gates), ptr(cs), ptr(c0), ptr(w_hh), ptr(dgates_t),
                                  ptr(dh0), ptr(dc0), ptr(bar), T, B, H, stream_ptr(x.device)), 'lstm_backward')
        count_launch(1)
        dg2 = dgates_t[:, :, :B].permute(0, 2, 1).reshape(T * B, 4 * H)      # row-major copy for the GEMMs
        hprev = torch.cat([h0.unsqueeze(0), y[:-1]], 0).reshape(T * B, H)
        dx = _mm(dg2, w_ih, False, True).reshape(T, B, I) if ctx.needs_input_grad[0] else None   # dg[TB,4H] . w_ih[4H,I]
        dw_ih = _mm(dg2, x.reshape(T * B, I), True, True)                                         # dg^T . x
        dw_hh = _mm(dg2, hprev, True, True)                                                        # dg^T . h_{t-1}
        db = dg2.sum(0, dtype=torch.float32)
        return dx, dw_ih, dw_hh, db.to(ctx.bias_dtypes[0]), db.to(ctx.bias_dtypes[1]), dh0, dc0, None


def tc_supported(dtype, B, H):
    """Whether the tensor-core LSTM recurrence (``lstm_tc.cu``) takes this (dtype, batch, hidden size)."""
    from ... import env
    if not env.get('MXNET_B200_RNN_TC') or dtype not in (torch.float32, torch.float16, torch.bfloat16):
        return False
    if int(H) < 32:
        return False        # narrow layers gain nothing from the tensor cores and keep exact fp32 products (fp32-pipe kernels)
    code = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[dtype]
    return bool(lib().mxb_lstm_tc_supported(code, int(B), int(H)))


def _tc_dims(x, B, H):
    import ctypes
    out = (ctypes.c_int32 * 8)()
    check(lib().mxb_lstm_tc_dims(dt(x), int(B), int(H), out), 'lstm_tc_dims')
    return tuple(int(v) for v in out[:6])


def _tc_perm_rows(w, dims):
    """Rows of a [4H, X] gate-major matrix (or a [4H] vector) regrouped per CTA: row c*4U + g*U + u = row g*H + c*U + u,
    zero rows for the padded units of the last CTA.  Result [KK, X]."""
    U, _Bp, _Hp, C, Hc, KK = dims
    H = w.shape[0] // 4
    tail = w.shape[1:]
    out = w.new_zeros((4, Hc) + tuple(tail))
    out[:, :H] = w.reshape((4, H) + tuple(tail))
    lead = list(range(4, 4 + len(tail)))
    return out.reshape((4, C, U) + tuple(tail)).permute(1, 0, 2, *[i - 1 for i in lead]).reshape((KK,) + tuple(tail)).contiguous()


def _tc_unperm_rows(w, dims, H):
    """Inverse of :func:`_tc_perm_rows`: [KK, X] in the per-CTA order back to [4H, X] gate-major."""
    U, _Bp, _Hp, C, Hc, _KK = dims
    tail = w.shape[1:]
    lead = list(range(3, 3 + len(tail)))
    g = w.reshape((C, 4, U) + tuple(tail)).permute(1, 0, 2, *lead).reshape((4, Hc) + tuple(tail))
    return g[:, :H].reshape((4 * H,) + tuple(tail))


def _tc_pack_forward(w_hh, dims):
    """[KK, Hp]: the gate rows of W_hh regrouped per CTA, the contraction axis zero padded to whole 128-byte chunks."""
    Hp = dims[2]
    H = w_hh.shape[1]
    w = _tc_perm_rows(w_hh, dims)
    return w if Hp == H else torch.nn.functional.pad(w, (0, Hp - H))


def _tc_pack_backward(w_hh, dims):
    """[Hc, KK]: row n holds column n of W_hh with the gate rows in the per-CTA order of the saved gates."""
    Hc = dims[4]
    H = w_hh.shape[1]
    w = _tc_perm_rows(w_hh, dims)                 # [KK, H]
    if Hc != H:
        w = torch.nn.functional.pad(w, (0, Hc - H))
    return w.t().contiguous()


class _LSTMLayerTC(torch.autograd.Function):
    """The LSTM layer of :class:`_LSTMLayer` with the recurrence on the tensor cores (``lstm_tc.cu``): h is exchanged
    row-major, the packed recurrent weights stay in shared memory, one tcgen05 product per time step and CTA.  The gate
    axis of the input projection, of the saved gates and of the gate gradients is kept in the kernel's per-CTA order
    (so each thread moves whole 16-byte vectors); only weight-sized tensors are regrouped, before and after."""

    @staticmethod
    def forward(ctx, x, w_ih, w_hh, b_ih, b_hh, h0, c0, training):
        L = lib()
        T, B, I = x.shape
        H = w_hh.shape[1]
        x = x.contiguous()
        w_ih, w_hh, h0, c0 = w_ih.contiguous(), w_hh.contiguous(), h0.contiguous(), c0.contiguous()
        for t, name, shape in ((w_ih, 'w_ih', (4 * H, I)), (w_hh, 'w_hh', (4 * H, H)), (h0, 'h0', (B, H)), (c0, 'c0', (B, H))):
            require(t, name, dtype=x.dtype, device=x.device, shape=shape)
        dims = _tc_dims(x, B, H)
        _U, Bp, Hp, _C, Hc, KK = dims
        bias = _tc_perm_rows((b_ih.float() + b_hh.float()).to(x.dtype), dims)
        require(bias, 'bias', numel=KK, device=x.device)
        wi = _tc_perm_rows(w_ih, dims)                                     # [KK, I]
        x2 = x.reshape(T * B, I)
        from . import gemm_ops
        if x.dtype in (torch.float16, torch.bfloat16) and gemm_ops.operand_ok(x2) and gemm_ops.operand_ok(wi):
            xproj = gemm_ops.gemm(x2, wi, False, False, bias)
        else:
            with _tf32_products():
                xproj = torch.addmm(bias, x2, wi.t())
        wp = _tc_pack_forward(w_hh, dims)
        y = torch.empty(T, B, H, dtype=x.dtype, device=x.device)
        hT, cT = torch.empty_like(h0), torch.empty_like(c0)
        gates = torch.empty(T, B, KK, dtype=x.dtype, device=x.device) if training else None
        cs = torch.empty(T, B, Hc, dtype=torch.float32, device=x.device) if training else None
        hbuf = torch.zeros(2, Bp, Hp, dtype=x.dtype, device=x.device)
        bar = _barrier_words(x.device)
        check(L.mxb_lstm_tc_forward(dt(x), ptr(xproj), ptr(wp), ptr(h0), ptr(c0), ptr(y), ptr(hT), ptr(cT), ptr(gates), ptr(cs),
                                    ptr(hbuf), ptr(bar), T, B, H, stream_ptr(x.device)), 'lstm_tc_forward')
        count_launch(1)
        ctx.save_for_backward(x, wi, w_hh, h0, c0, y, gates, cs)
        ctx.bias_dtypes = (b_ih.dtype, b_hh.dtype)
        ctx.dims = dims
        ctx.fwd_bar = bar
        ctx.set_materialize_grads(False)
        return y, hT, cT

    @staticmethod
    def backward(ctx, dy, dhT, dcT):
        x, wi, w_hh, h0, c0, y, gates, cs = ctx.saved_tensors
        if gates is None:
            raise RuntimeError('LSTM backward needs a forward pass in training mode')
        L = lib()
        T, B, I = x.shape
        H = w_hh.shape[1]
        dims = ctx.dims
        KK = dims[5]
        dy = torch.zeros_like(y) if dy is None else dy.contiguous()
        require(dy, 'out_grad', dtype=x.dtype, device=x.device, shape=y.shape)
        dhT = dhT.contiguous() if dhT is not None else None
        dcT = dcT.contiguous() if dcT is not None else None
        wb = _tc_pack_backward(w_hh, dims)
        dgates = torch.empty(T, B, KK, dtype=x.dtype, device=x.device)          # per-CTA column order, row-major
        dh0, dc0 = torch.empty_like(h0), torch.empty_like(c0)
        bar = _barrier_words(x.device)
        check(L.mxb_lstm_tc_backward(dt(x), ptr(dy), ptr(dhT), ptr(dcT), ptr(gates), ptr(cs), ptr(c0), ptr(wb), ptr(dgates),
                                     ptr(dh0), ptr(dc0), ptr(bar), T, B, H, stream_ptr(x.device)), 'lstm_tc_backward')
        count_launch(1)
        ctx.bwd_bar = bar
        dg2 = dgates.view(T * B, KK)
        hprev = torch.cat([h0.unsqueeze(0), y[:-1]], 0).reshape(T * B, H)
        dx = _mm(dg2, wi, False, True, True).reshape(T, B, I) if ctx.needs_input_grad[0] else None      # dg[TB,KK] . wi[KK,I]
        dw_ih = _tc_unperm_rows(_mm(dg2, x.reshape(T * B, I), True, True, True), dims, H)                # (dg^T . x) regrouped
        dw_hh = _tc_unperm_rows(_mm(dg2, hprev, True, True, True), dims, H)
        db = _tc_unperm_rows(dg2.sum(0, dtype=torch.float32), dims, H)
        return dx, dw_ih, dw_hh, db.to(ctx.bias_dtypes[0]), db.to(ctx.bias_dtypes[1]), dh0, dc0, None


# ---- GRU on the tensor cores (gru_tc.inl) ---------------------------------------------------------------------------------
def gru_tc_supported(dtype, B, H):
    """Whether the tensor-core GRU recurrence takes this (dtype, batch, hidden size); layers under 32 units stay on the exact
    fp32-pipe kernels, like the LSTM."""
    from ... import env
    if not env.get('MXNET_B200_RNN_TC') or dtype not in (torch.float32, torch.float16, torch.bfloat16) or int(H) < 32:
        return False
    code = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[dtype]
    key = (code, int(B), int(H), torch.cuda.current_device())
    hit = _gru_ok.get(key)
    if hit is None:
        hit = _gru_ok[key] = bool(lib().mxb_gru_tc_supported(code, int(B), int(H)))
    return hit


def _gru_dims(x, B, H):
    import ctypes
    out = (ctypes.c_int32 * 8)()
    check(lib().mxb_gru_tc_dims(dt(x), int(B), int(H), out), 'gru_tc_dims')
    return tuple(int(v) for v in out[:7])             # U, Bp, Hp, C, Hc, KK, NGP


def _gru_perm_rows(w, dims):
    """Rows of a [3H, X] gate-major matrix (or a [3H] vector) regrouped per CTA and padded: row c*NGP + g*U + u = row
    g*H + c*U + u; rows of padded units and the NGP - 3U filler rows of every CTA are zero.  Result [KK, X]."""
    U, _Bp, _Hp, C, Hc, KK, NGP = dims
    H = w.shape[0] // 3
    tail = tuple(w.shape[1:])
    g = w.new_zeros((3, Hc) + tail)
    g[:, :H] = w.reshape((3, H) + tail)
    lead = [i + 3 for i in range(len(tail))]
    per_cta = g.reshape((3, C, U) + tail).permute(1, 0, 2, *lead).reshape((C, 3 * U) + tail)
    out = w.new_zeros((C, NGP) + tail)
    out[:, :3 * U] = per_cta
    return out.reshape((KK,) + tail)


def _gru_unperm_rows(w, dims, H):
    U, _Bp, _Hp, C, Hc, _KK, NGP = dims
    tail = tuple(w.shape[1:])
    lead = [i + 3 for i in range(len(tail))]
    g = w.reshape((C, NGP) + tail)[:, :3 * U].reshape((C, 3, U) + tail).permute(1, 0, 2, *lead).reshape((3, Hc) + tail)
    return g[:, :H].reshape((3 * H,) + tail)


class _GRULayerTC(torch.autograd.Function):
    """y, hT = gru(x[T,B,I], w_ih[3H,I], w_hh[3H,H], b_ih[3H], b_hh[3H], h0[B,H]) with the recurrence on the tensor cores."""

    @staticmethod
    def forward(ctx, x, w_ih, w_hh, b_ih, b_hh, h0, training):
        L = lib()
        T, B, I = x.shape
        H = w_hh.shape[1]
        x = x.contiguous()
        w_ih, w_hh, h0 = w_ih.contiguous(), w_hh.contiguous(), h0.contiguous()
        for t, name, shape in ((w_ih, 'w_ih', (3 * H, I)), (w_hh, 'w_hh', (3 * H, H)), (h0, 'h0', (B, H))):
            require(t, name, dtype=x.dtype, device=x.device, shape=shape)
        dims = _gru_dims(x, B, H)
        _U, Bp, Hp, _C, Hc, KK, _NGP = dims
        bias = b_ih.float() + b_hh.float()
        bias[2 * H:] = b_ih.float()[2 * H:]                  # the candidate gate's hidden-side bias stays inside r * (...)
        bias = _gru_perm_rows(bias.to(x.dtype), dims)
        bhn = torch.zeros(Hc, dtype=torch.float32, device=x.device)
        bhn[:H] = b_hh.float()[2 * H:]
        wi = _gru_perm_rows(w_ih, dims)                      # [KK, I]
        x2 = x.reshape(T * B, I)
        from . import gemm_ops
        if x.dtype in (torch.float16, torch.bfloat16) and gemm_ops.operand_ok(x2) and gemm_ops.operand_ok(wi):
            xproj = gemm_ops.gemm(x2, wi, False, False, bias)
        else:
            with _tf32_products():
                xproj = torch.addmm(bias, x2, wi.t())
        wp = _gru_perm_rows(w_hh, dims)
        if Hp != H:
            wp = torch.nn.functional.pad(wp, (0, Hp - H))
        y = torch.empty(T, B, H, dtype=x.dtype, device=x.device)
        hT = torch.empty_like(h0)
        gates = torch.empty(T, B, KK, dtype=x.dtype, device=x.device) if training else None
        hnb = torch.empty(T, B, Hc, dtype=torch.float32, device=x.device) if training else None
        hbuf = torch.zeros(2, Bp, Hp, dtype=x.dtype, device=x.device)
        bar = _barrier_words(x.device)
        check(L.mxb_gru_tc_forward(dt(x), ptr(xproj), ptr(wp), ptr(bhn), ptr(h0), ptr(y), ptr(hT), ptr(gates), ptr(hnb), ptr(hbuf),
                                   ptr(bar), T, B, H, stream_ptr(x.device)), 'gru_tc_forward')
        count_launch(1)
        ctx.save_for_backward(x, wi, w_hh, h0, y, gates, hnb)
        ctx.bias_dtypes = (b_ih.dtype, b_hh.dtype)
        ctx.dims = dims
        ctx.fwd_bar = bar
        ctx.set_materialize_grads(False)
        return y, hT

    @staticmethod
    def backward(ctx, dy, dhT):
        x, wi, w_hh, h0, y, gates, hnb = ctx.saved_tensors
        if gates is None:
            raise RuntimeError('GRU backward needs a forward pass in training mode')
        L = lib()
        T, B, I = x.shape
        H = w_hh.shape[1]
        dims = ctx.dims
        Hc, KK = dims[4], dims[5]
        dy = torch.zeros_like(y) if dy is None else dy.contiguous()
        require(dy, 'out_grad', dtype=x.dtype, device=x.device, shape=y.shape)
        dhT = dhT.contiguous() if dhT is not None else None
        wb = _gru_perm_rows(w_hh, dims)                      # [KK, H]
        if Hc != H:
            wb = torch.nn.functional.pad(wb, (0, Hc - H))
        wb = wb.t().contiguous()                             # [Hc, KK]
        dgh = torch.empty(T, B, KK, dtype=x.dtype, device=x.device)
        dgx = torch.empty(T, B, KK, dtype=x.dtype, device=x.device)
        dh0 = torch.empty_like(h0)
        bar = _barrier_words(x.device)
        check(L.mxb_gru_tc_backward(dt(x), ptr(dy), ptr(dhT), ptr(gates), ptr(hnb), ptr(y), ptr(h0), ptr(wb), ptr(dgh), ptr(dgx),
                                    ptr(dh0), ptr(bar), T, B, H, stream_ptr(x.device)), 'gru_tc_backward')
        count_launch(1)
        ctx.bwd_bar = bar
        gh2, gx2 = dgh.view(T * B, KK), dgx.view(T * B, KK)
        hprev = torch.cat([h0.unsqueeze(0), y[:-1]], 0).reshape(T * B, H)
        dx = _mm(gx2, wi, False, True, True).reshape(T, B, I) if ctx.needs_input_grad[0] else None
        dw_ih = _gru_unperm_rows(_mm(gx2, x.reshape(T * B, I), True, True, True), dims, H)
        dw_hh = _gru_unperm_rows(_mm(gh2, hprev, True, True, True), dims, H)
        db_ih = _gru_unperm_rows(gx2.sum(0, dtype=torch.float32), dims, H)
        db_hh = _gru_unperm_rows(gh2.sum(0, dtype=torch.float32), dims, H)
        return dx, dw_ih, dw_hh, db_ih.to(ctx.bias_dtypes[0]), db_hh.to(ctx.bias_dtypes[1]), dh0, None


def check_errors(bar):
    """Raise when a grid barrier of the recurrence timed out (outputs incomplete)."""
    if int(bar[1].item()) != 0:
        raise RuntimeError('LSTM recurrence kernel: grid barrier timed out')


_MODES = {'gru': 0, 'rnn_tanh': 1, 'rnn_relu': 2}


class _RecurrentLayer(torch.autograd.Function):
    """y, hT = layer(x[T,B,I], w_ih[G*H,I], w_hh[G*H,H], b_ih[G*H], b_hh[G*H], h0[B,H]) for a GRU (G = 3, gates r, z, n)
    or a vanilla RNN (G = 1).  The input projection of all steps is one GEMM; the recurrence is one cooperative kernel."""

    @staticmethod
    def forward(ctx, x, w_ih, w_hh, b_ih, b_hh, h0, mode, training):
        L = lib()
        T, B, I = x.shape
        H = w_hh.shape[1]
        G = 3 if mode == 0 else 1
        x = x.contiguous()
        w_ih, w_hh, h0 = w_ih.contiguous(), w_hh.contiguous(), h0.contiguous()
        for t, name, shape in ((w_ih, 'w_ih', (G * H, I)), (w_hh, 'w_hh', (G * H, H)), (h0, 'h0', (B, H))):
            require(t, name, dtype=x.dtype, device=x.device, shape=shape)
        bias = b_ih.float() + b_hh.float()
        bhn = None
        if mode == 0:                    # the candidate gate's hidden-side bias stays inside r * (...)
            bias[2 * H:] = b_ih.float()[2 * H:]
            bhn = b_hh[2 * H:].to(x.dtype).contiguous()
        bias = bias.to(x.dtype)
        from . import gemm_ops
        x2 = x.reshape(T * B, I)
        if x.dtype in (torch.float16, torch.bfloat16) and gemm_ops.operand_ok(x2) and gemm_ops.operand_ok(w_ih):
            xproj = gemm_ops.gemm(x2, w_ih, False, False, bias)
        else:
            xproj = torch.addmm(bias, x2, w_ih.t())
        y = torch.empty(T, B, H, dtype=x.dtype, device=x.device)
        hT = torch.empty_like(h0)
        Bp = L.mxb_lstm_bp(B)
        save = training and mode == 0
        gates = torch.empty(T, 3 * H, Bp, dtype=x.dtype, device=x.device) if save else None
        hnb = torch.empty(T, H, Bp, dtype=x.dtype, device=x.device) if save else None
        hbuf = torch.empty(L.mxb_lstm_exchange_bytes(B, H), dtype=torch.uint8, device=x.device)
        bar = _barrier_words(x.device)
        check(L.mxb_rnn_forward(dt(x), mode, ptr(xproj), ptr(w_hh), ptr(bhn), ptr(h0), ptr(y), ptr(hT), ptr(gates), ptr(hnb),
                                ptr(hbuf), ptr(bar), T, B, H, stream_ptr(x.device)), 'rnn_forward')
        count_launch(1)
        ctx.save_for_backward(x, w_ih, w_hh, h0, y, gates, hnb)
        ctx.mode, ctx.trained = mode, bool(training)
        ctx.bias_dtypes = (b_ih.dtype, b_hh.dtype)
        ctx.fwd_bar = bar
        ctx.set_materialize_grads(False)
        return y, hT

    @staticmethod
    def backward(ctx, dy, dhT):
        x, w_ih, w_hh, h0, y, gates, hnb = ctx.saved_tensors
        mode = ctx.mode
        if not ctx.trained:
            raise RuntimeError('RNN backward needs a forward pass in training mode')
        L = lib()
        T, B, I = x.shape
        H = w_hh.shape[1]
        G = 3 if mode == 0 else 1
        Bp = L.mxb_lstm_bp(B)
        dy = torch.zeros_like(y) if dy is None else dy.contiguous()
        require(dy, 'out_grad', dtype=x.dtype, device=x.device, shape=y.shape)
        dhT = dhT.contiguous() if dhT is not None else None
        dgh = torch.empty(T, G * H, Bp, dtype=x.dtype, device=x.device)          # hidden-side gate gradients, k-major
        dan = torch.empty(T, H, Bp, dtype=x.dtype, device=x.device) if mode == 0 else None
        dh0 = torch.empty_like(h0)
        bar = _barrier_words(x.device)
        check(L.mxb_rnn_backward(dt(x), mode, ptr(dy), ptr(dhT), ptr(gates), ptr(hnb), ptr(y), ptr(h0), ptr(w_hh), ptr(dgh),
                                 ptr(dan), ptr(dh0), ptr(bar), T, B, H, stream_ptr(x.device)), 'rnn_backward')
        count_launch(1)
        dgh2 = dgh[:, :, :B].permute(0, 2, 1).reshape(T * B, G * H)
        if mode == 0:                    # the input side sees the candidate gradient without the factor r
            dgx2 = torch.cat([dgh2[:, :2 * H], dan[:, :, :B].permute(0, 2, 1).reshape(T * B, H)], 1)
        else:
            dgx2 = dgh2
        hprev = torch.cat([h0.unsqueeze(0), y[:-1]], 0).reshape(T * B, H)
        dx = _mm(dgx2, w_ih, False, True).reshape(T, B, I) if ctx.needs_input_grad[0] else None
        dw_ih = _mm(dgx2, x.reshape(T * B, I), True, True)
        dw_hh = _mm(dgh2, hprev, True, True)
        db_ih = dgx2.sum(0, dtype=torch.float32)
        db_hh = dgh2.sum(0, dtype=torch.float32) if mode == 0 else db_ih
        return dx, dw_ih, dw_hh, db_ih.to(ctx.bias_dtypes[0]), db_hh.to(ctx.bias_dtypes[1]), dh0, None, None


def recurrent(mode, data, parameters, state, state_size, num_layers, p, training, bidirectional=False):
    """Multi-layer GRU / vanilla RNN over (T, N, C) data with the flat parameter vector of the RNN operator; layout and
    direction handling as in :func:`lstm`."""
    from ..nn import rnn_unpack
    T, N, I = data.shape
    d = 2 if bidirectional else 1
    layers = rnn_unpack(parameters, mode, num_layers, I, state_size, bool(bidirectional), None)
    x = data
    hs = []
    for l in range(num_layers):
        outs = []
        for di in range(d):
            w_ih, w_hh, _w_hr, b_ih, b_hh = layers[l * d + di]
            xin = x if di == 0 else x.flip(0)
            if mode == 'gru' and gru_tc_supported(xin.dtype, N, state_size):
                y, h = _GRULayerTC.apply(xin.contiguous(), w_ih, w_hh, b_ih, b_hh, state[l * d + di], bool(training))
            else:
                y, h = _RecurrentLayer.apply(xin.contiguous(), w_ih, w_hh, b_ih, b_hh, state[l * d + di], _MODES[mode],
                                             bool(training))
            outs.append(y if di == 0 else y.flip(0))
            hs.append(h)
        x = outs[0] if d == 1 else torch.cat(outs, -1)
        if p > 0 and training and l < num_layers - 1:
            x = torch.nn.functional.dropout(x, p, True)
    return x, torch.stack(hs, 0)


def lstm(data, parameters, state, state_cell, state_size, num_layers, p, training, bidirectional=False):
    """Multi-layer LSTM over (T, N, C) data with the flat parameter vector of the RNN operator.  A bidirectional layer
    runs the recurrence kernel twice, the second time on the time-reversed sequence with the reverse direction's
    weights, and concatenates the two outputs along the feature axis (states are ordered layer * 2 + direction)."""
    from ..nn import rnn_unpack
    T, N, I = data.shape
    d = 2 if bidirectional else 1
    layers = rnn_unpack(parameters, 'lstm', num_layers, I, state_size, bool(bidirectional), None)
    x = data
    hs, cs = [], []
    for l in range(num_layers):
        outs = []
        for di in range(d):
            w_ih, w_hh, _w_hr, b_ih, b_hh = layers[l * d + di]
            xin = x if di == 0 else x.flip(0)
            layer = _LSTMLayerTC if tc_supported(xin.dtype, N, state_size) else _LSTMLayer
            y, h, c = layer.apply(xin.contiguous(), w_ih, w_hh, b_ih, b_hh, state[l * d + di], state_cell[l * d + di],
                                  bool(training))
            outs.append(y if di == 0 else y.flip(0))
            hs.append(h)
            cs.append(c)
        x = outs[0] if d == 1 else torch.cat(outs, -1)
        if p > 0 and training and l < num_layers - 1:
            x = torch.nn.functional.dropout(x, p, True)
    return x, torch.stack(hs, 0), torch.stack(cs, 0)

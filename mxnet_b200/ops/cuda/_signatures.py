"""ctypes prototypes of the kernel library's ``extern "C"`` entry points."""
import ctypes as C

vp, i32, i64, f32, u32, u64 = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_uint32, C.c_uint64
pvp = C.POINTER(C.c_void_p)


def declare(L):
    def sig(name, res, *args):
        if not hasattr(L, name):
            return
        f = getattr(L, name)
        f.restype, f.argtypes = res, list(args)
    sig('mxb_bn_grid', i32, i64, i32)
    sig('mxb_ln_grid', i32, i64)
    sig('mxb_bn_forward', i32, i32, vp, vp, vp, vp, i32, vp, vp, vp, vp, vp, vp, vp, i64, i32, f32, f32, i32, i32, vp)
    sig('mxb_bn_backward', i32, i32, vp, vp, vp, vp, i32, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, i32, vp)
    sig('mxb_maxpool_forward', i32, i32, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp)
    sig('mxb_maxpool_backward', i32, i32, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp)
    sig('mxb_lstm_supported', i32, i32, i32)
    sig('mxb_lstm_forward', i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp)
    sig('mxb_lstm_backward', i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp)
    sig('mxb_lstm_exchange_bytes', i64, i32, i32)
    sig('mxb_ln_forward', i32, i32, vp, vp, vp, vp, vp, vp, i64, i32, f32, vp)
    sig('mxb_ln_backward', i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, vp)
    sig('mxb_softmax_forward', i32, i32, vp, vp, i64, i32, i32, vp)
    sig('mxb_softmax_backward', i32, i32, vp, vp, vp, i64, i32, i32, vp)
    sig('mxb_softmax_ce_forward', i32, i32, vp, vp, vp, vp, i64, i32, i64, i32, vp)
    sig('mxb_softmax_ce_backward', i32, i32, vp, vp, vp, vp, vp, i64, i32, i64, i32, vp)
    sig('mxb_max_tensors', i32)
    sig('mxb_chunk_elems', i32)
    sig('mxb_multi_sgd', i32, i32, i32, pvp, pvp, pvp, pvp, C.POINTER(f32), C.POINTER(f32), C.POINTER(i64), f32, f32, f32, vp)
    sig('mxb_multi_all_finite', i32, i32, pvp, C.POINTER(i64), C.POINTER(i32), vp, i32, vp)
    sig('mxb_sum_sq_chunks', i32, i32, C.POINTER(i64))
    sig('mxb_multi_sum_sq', i32, i32, pvp, C.POINTER(i64), C.POINTER(i32), vp, vp, i32, vp)
    sig('mxb_step_ctrl_bytes', i32)
    sig('mxb_step_params_bytes', i32)
    sig('mxb_step_max_ranks', i32)
    sig('mxb_step_ctrl_offset', i32, i32)
    sig('mxb_fused_reduce', i32, i32, vp, vp)
    sig('mxb_fused_update', i32, i32, vp, vp)
    sig('mxb_fused_lamb', i32, i32, vp, vp)
    sig('mxb_wait_probe', i32, vp, i32, u32, C.c_ulonglong, vp)
    sig('mxb_dev_alloc', i32, pvp, u64)
    sig('mxb_dev_free', i32, vp)
    sig('mxb_ipc_handle_bytes', i32)
    sig('mxb_ipc_get_handle', i32, vp, vp)
    sig('mxb_ipc_open', i32, vp, pvp)
    sig('mxb_ipc_close', i32, vp)
    sig('mxb_memcpy_d2h', i32, vp, vp, u64, vp)
    sig('mxb_memcpy_h2d', i32, vp, vp, u64, vp)
    sig('mxb_error_string', C.c_char_p, i32)
    sig('mxb_gemm_tn', i32, i32, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp, vp)
    sig('mxb_gemm', i32, i32, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp)

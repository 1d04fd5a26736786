"""The allocation-free sum-of-squares entry point (``mxb_multi_sum_sq_static``) called through its C
symbol, against the regular entry point that takes a caller-provided workspace."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

ERR_BAD_COUNT, ERR_TOO_LARGE = -2, -4
CHUNK, MAX_CHUNKS = 8192, 65536


def _symbol():
    from mxnet_b200.ops import cuda
    fn = cuda.lib().mxb_multi_sum_sq_static
    fn.restype = C.c_int
    fn.argtypes = [C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_int64), C.POINTER(C.c_int), C.c_void_p, C.c_int, C.c_void_p]
    return fn


def _call(fn, tensors, out, offset=0):
    n = len(tensors)
    codes = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
    ptrs = (C.c_void_p * n)(*[t.data_ptr() for t in tensors])
    sizes = (C.c_int64 * n)(*[t.numel() for t in tensors])
    dts = (C.c_int * n)(*[codes[t.dtype] for t in tensors])
    return fn(n, ptrs, sizes, dts, C.c_void_p(out.data_ptr()), offset, C.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_static_scratch_matches_workspace_entry_point_twice_in_a_row():
    from mxnet_b200.ops.cuda import optim_ops
    fn = _symbol()
    dev = torch.device('cuda', 0)
    torch.manual_seed(11)
    sets = [[torch.randn(n, device=dev).to(dt) for n, dt in
             [(1, torch.float32), (8191, torch.float16), (8193, torch.bfloat16), (300000, torch.float16), (77, torch.float32)]],
            [torch.randn(n, device=dev).to(dt) * 3 for n, dt in
             [(1000000, torch.float16), (5, torch.float32), (65536, torch.bfloat16)]]]
    for tensors in sets:                      # two calls in a row share the scratch array
        out = torch.full((len(tensors) + 2,), -1.0, device=dev)
        assert _call(fn, tensors, out, offset=1) == 0
        ref = optim_ops.multi_sum_sq(tensors)
        torch.cuda.synchronize()
        assert torch.equal(out[1:-1], ref)    # same chunking and order of additions: bitwise equal
        assert float(out[0]) == -1.0 and float(out[-1]) == -1.0
        fp32 = torch.stack([(t.double() ** 2).sum() for t in tensors]).float()
        torch.testing.assert_close(out[1:-1], fp32, rtol=1e-4, atol=1e-4)
    # and again on the first set: nothing left over from the previous call matters
    out = torch.zeros(len(sets[0]), device=dev)
    assert _call(fn, sets[0], out) == 0
    assert torch.equal(out, optim_ops.multi_sum_sq(sets[0]))


def test_static_scratch_rejects_requests_beyond_its_size():
    fn = _symbol()
    dev = torch.device('cuda', 0)
    out = torch.zeros(4, device=dev)
    small = torch.ones(8, device=dev)
    # the sizes alone decide: the call is refused before any pointer is used or any kernel is launched
    n = 2
    ptrs = (C.c_void_p * n)(small.data_ptr(), small.data_ptr())
    sizes = (C.c_int64 * n)(CHUNK * MAX_CHUNKS, 1)
    dts = (C.c_int * n)(0, 0)
    rc = fn(n, ptrs, sizes, dts, C.c_void_p(out.data_ptr()), 0, C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == ERR_TOO_LARGE
    # element counts near the top of int64: the chunk count must not wrap around into an acceptable number
    for huge in (2 ** 63 - 1, 2 ** 63 - 8191, 2 ** 62):
        sizes_huge = (C.c_int64 * n)(huge, 1)
        assert fn(n, ptrs, sizes_huge, dts, C.c_void_p(out.data_ptr()), 0, None) == ERR_TOO_LARGE
    assert fn(0, ptrs, sizes, dts, C.c_void_p(out.data_ptr()), 0, None) == ERR_BAD_COUNT
    assert fn(49, ptrs, sizes, dts, C.c_void_p(out.data_ptr()), 0, None) == ERR_BAD_COUNT
    torch.cuda.synchronize()
    assert float(out.sum()) == 0.0

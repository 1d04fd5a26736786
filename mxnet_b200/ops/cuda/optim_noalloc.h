// Sum of squares of up to 48 tensors without any allocation.
//
// This entry point has no counterpart in the reference (its multi_sum_sq takes a workspace from the
// framework's resource manager on every call).  It exists for callers that have no allocator they may
// use at the moment they need a gradient norm:
//   * a C or C++ host program that links this library without the Python tensor library, so there is no
//     caching allocator to ask for a workspace;
//   * a monitoring or logging thread that must not take the allocator's lock, nor move the memory pool's
//     high-water mark, while the training thread is in the middle of a step;
//   * an out-of-memory handler that reports the state of the gradients exactly when no request for
//     device memory can succeed.
//
// The partial sums of stage 1 live in one fixed array in device global memory that is part of the
// library image (MXB_SUM_SQ_STATIC_MAX_CHUNKS floats = 256 KiB per device).  Consequences:
//   * the tensors of one call may hold at most MXB_SUM_SQ_STATIC_MAX_CHUNKS chunks of
//     MXB_SUM_SQ_CHUNK_ELEMS elements (each tensor occupies ceil(n / chunk) chunks); a larger request is
//     refused with MXB_SUM_SQ_ERR_TOO_LARGE before anything is launched;
//   * nothing in the array has to start at zero: every slot that stage 2 reads was written by stage 1 of
//     the same call;
//   * every call on a device uses the same array.  Calls issued to one stream run in order and are safe;
//     two calls that can overlap (different streams, or different host threads without ordering between
//     their streams) race on the array and give wrong sums;
//   * the first call on each device looks up the array's device address and caches it.  The look-up launches
//     nothing, but it can be the moment the CUDA runtime loads this library's device code onto that device
//     (lazy module loading), and loading does allocate: the code image and this 256 KiB array.  So make the
//     first call on every device at start-up, with the device current, before any stream capture begins there
//     and well before the situations listed above (an out-of-memory handler must not be the first caller).
//     Later calls on that device allocate nothing.
// The call does not use cudaMalloc, cudaFree, nor any library routine that allocates.
#pragma once
#include <stdint.h>

#define MXB_SUM_SQ_CHUNK_ELEMS 8192
#define MXB_SUM_SQ_STATIC_MAX_CHUNKS 65536
#define MXB_SUM_SQ_ERR_BAD_COUNT (-2)    /* count < 1 or count > 48 */
#define MXB_SUM_SQ_ERR_TOO_LARGE (-4)    /* the tensors need more chunks than the fixed array holds */
#define MXB_SUM_SQ_ERR_DEVICE (-5)       /* the current device index is outside the supported range (0..63) */

#ifdef __cplusplus
extern "C" {
#endif

// out[out_offset + i] = sum of squares of tensor i, accumulated in fp32.
//   count    number of tensors (1..48)
//   p        host array of `count` device pointers
//   sizes    host array of element counts
//   dtypes   host array of dtype codes (0 fp32, 1 fp16, 2 bf16)
//   out      device array of at least out_offset + count floats
//   stream   cudaStream_t (0 = the default stream)
// Returns 0, one of the MXB_SUM_SQ_ERR_* codes, or a positive cudaError_t.
int mxb_multi_sum_sq_static(int count, void** p, const int64_t* sizes, const int* dtypes, float* out, int out_offset,
                            void* stream);

#ifdef __cplusplus
}
#endif

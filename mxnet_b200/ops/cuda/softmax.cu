// Row softmax / log-softmax and fused softmax cross-entropy (forward + gradient) for sm_100a.
//
// Reference behaviour: src/operator/nn/softmax.cu (row cached in shared memory, rows-per-block
// heuristic) and the SoftmaxOutput gradient kernels of mshadow (tensor_gpu-inl.cuh: SoftmaxGradKernel).
// One CTA per row with an online (max, sum) reduction: the logits are read once for the statistics
// and once more (L2-resident) for the output; cross-entropy never writes the probabilities in the
// forward pass, only the per-row loss and log-sum-exp, and the backward pass rebuilds
// p = exp(x - lse) on the fly.  Large vocabularies (30522 / 33278 columns) stay one row per CTA
// (256 threads striding over the row).
#include "common.cuh"

namespace mxb {

constexpr int kSmThreads = 256;

struct MaxSum { float m, s; };

__device__ __forceinline__ MaxSum ms_combine(MaxSum a, MaxSum b) {
  float m = fmaxf(a.m, b.m);
  if (m == -INFINITY) return {m, 0.f};
  return {m, a.s * __expf(a.m - m) + b.s * __expf(b.m - m)};
}

__device__ __forceinline__ MaxSum block_maxsum(MaxSum v, MaxSum* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum other{__shfl_xor_sync(0xffffffffu, v.m, o), __shfl_xor_sync(0xffffffffu, v.s, o)};
    v = ms_combine(v, other);
  }
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    MaxSum r = lane < nw ? red[lane] : MaxSum{-INFINITY, 0.f};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      MaxSum other{__shfl_xor_sync(0xffffffffu, r.m, o), __shfl_xor_sync(0xffffffffu, r.s, o)};
      r = ms_combine(r, other);
    }
    if (lane == 0) red[0] = r;
  }
  __syncthreads();
  return red[0];
}

template <typename T>
__device__ __forceinline__ MaxSum row_stats(const T* __restrict__ xr, int C) {
  MaxSum acc{-INFINITY, 0.f};
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float f = Cvt<T>::to_f(xr[c]);
    if (f > acc.m) { acc.s = acc.s * __expf(acc.m - f) + 1.f; acc.m = f; }
    else if (f != -INFINITY) acc.s += __expf(f - acc.m);
  }
  return acc;
}

template <typename T, bool kLog>
__global__ void __launch_bounds__(kSmThreads)
softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int C) {
  __shared__ MaxSum red[32];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * C;
    MaxSum st = block_maxsum(row_stats(xr, C), red);
    const float lse = st.m + __logf(st.s);
    T* yr = y + row * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      float f = Cvt<T>::to_f(xr[c]) - lse;
      yr[c] = Cvt<T>::from_f(kLog ? f : __expf(f));
    }
  }
}

// dx = y * (dy - sum(dy * y))  (softmax)   |   dx = dy - exp(y) * sum(dy)  (log-softmax)
template <typename T, bool kLog>
__global__ void __launch_bounds__(kSmThreads)
softmax_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx, int64_t rows, int C) {
  __shared__ float red[32];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* yr = y + row * C;
    const T* gr = dy + row * C;
    float s = 0.f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      float g = Cvt<T>::to_f(gr[c]);
      s += kLog ? g : g * Cvt<T>::to_f(yr[c]);
    }
    s = block_sum(s, red);
    T* dr = dx + row * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      float g = Cvt<T>::to_f(gr[c]), o = Cvt<T>::to_f(yr[c]);
      dr[c] = Cvt<T>::from_f(kLog ? g - __expf(o) * s : o * (g - s));
    }
  }
}

// loss[row] = lse(x[row]) - x[row, label[row]];  rows whose label equals ignore_label give 0.
template <typename T>
__global__ void __launch_bounds__(kSmThreads)
softmax_ce_fwd_kernel(const T* __restrict__ x, const int64_t* __restrict__ label, float* __restrict__ loss,
                      float* __restrict__ lse_out, int64_t rows, int C, int64_t ignore_label, int use_ignore) {
  __shared__ MaxSum red[32];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * C;
    MaxSum st = block_maxsum(row_stats(xr, C), red);
    if (threadIdx.x == 0) {
      const float lse = st.m + __logf(st.s);
      int64_t l = label[row];
      lse_out[row] = lse;
      if (use_ignore && l == ignore_label) loss[row] = 0.f;
      else {
        l = l < 0 ? 0 : (l >= C ? C - 1 : l);
        loss[row] = lse - Cvt<T>::to_f(xr[l]);
      }
    }
  }
}

// dx[row, c] = gout[row] * (exp(x - lse) - [c == label])
template <typename T>
__global__ void __launch_bounds__(kSmThreads)
softmax_ce_bwd_kernel(const T* __restrict__ x, const int64_t* __restrict__ label, const float* __restrict__ lse,
                      const float* __restrict__ gout, T* __restrict__ dx, int64_t rows, int C, int64_t ignore_label,
                      int use_ignore) {
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * C;
    T* dr = dx + row * C;
    int64_t l = label[row];
    float g = gout[row];
    if (use_ignore && l == ignore_label) g = 0.f;
    l = l < 0 ? 0 : (l >= C ? C - 1 : l);
    const float ls = lse[row];
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      float p = __expf(Cvt<T>::to_f(xr[c]) - ls);
      dr[c] = Cvt<T>::from_f(g * (p - (c == l ? 1.f : 0.f)));
    }
  }
}

inline int row_grid(int64_t rows) {
  int64_t cap = (int64_t)sm_count() * 8;
  return (int)(rows < cap ? (rows < 1 ? 1 : rows) : cap);
}

}  // namespace mxb

using namespace mxb;

#define DISPATCH_T(dtype, CALL)                                  \
  switch (dtype) {                                               \
    case kF32: { typedef float T; CALL; break; }                 \
    case kF16: { typedef __half T; CALL; break; }                \
    case kBF16: { typedef __nv_bfloat16 T; CALL; break; }        \
    default: return -1;                                          \
  }

MXB_EXPORT int mxb_softmax_forward(int dtype, const void* x, void* y, int64_t rows, int C, int log, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  int g = row_grid(rows);
  if (log) { DISPATCH_T(dtype, (softmax_fwd_kernel<T, true><<<g, kSmThreads, 0, st>>>((const T*)x, (T*)y, rows, C))) }
  else { DISPATCH_T(dtype, (softmax_fwd_kernel<T, false><<<g, kSmThreads, 0, st>>>((const T*)x, (T*)y, rows, C))) }
  return (int)cudaGetLastError();
}

MXB_EXPORT int mxb_softmax_backward(int dtype, const void* y, const void* dy, void* dx, int64_t rows, int C, int log,
                                    void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  int g = row_grid(rows);
  if (log) { DISPATCH_T(dtype, (softmax_bwd_kernel<T, true><<<g, kSmThreads, 0, st>>>((const T*)y, (const T*)dy, (T*)dx, rows, C))) }
  else { DISPATCH_T(dtype, (softmax_bwd_kernel<T, false><<<g, kSmThreads, 0, st>>>((const T*)y, (const T*)dy, (T*)dx, rows, C))) }
  return (int)cudaGetLastError();
}

MXB_EXPORT int mxb_softmax_ce_forward(int dtype, const void* x, const int64_t* label, float* loss, float* lse, int64_t rows,
                                      int C, int64_t ignore_label, int use_ignore, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  int g = row_grid(rows);
  DISPATCH_T(dtype, (softmax_ce_fwd_kernel<T><<<g, kSmThreads, 0, st>>>((const T*)x, label, loss, lse, rows, C, ignore_label, use_ignore)))
  return (int)cudaGetLastError();
}

MXB_EXPORT int mxb_softmax_ce_backward(int dtype, const void* x, const int64_t* label, const float* lse, const float* gout,
                                       void* dx, int64_t rows, int C, int64_t ignore_label, int use_ignore, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  int g = row_grid(rows);
  DISPATCH_T(dtype, (softmax_ce_bwd_kernel<T><<<g, kSmThreads, 0, st>>>((const T*)x, label, lse, gout, (T*)dx, rows, C, ignore_label, use_ignore)))
  return (int)cudaGetLastError();
}

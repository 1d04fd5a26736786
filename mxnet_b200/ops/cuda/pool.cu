// Max pooling for NHWC half-precision activations (sm_100a).
//
// Reference behaviour: src/operator/nn/pool.cuh (pool_max_2d_gpu_kernel / unpool_max_2d_gpu_kernel, one thread
// per output element, backward by atomics) and the cuDNN pooling path.  Here one thread owns 8 channels of one
// output pixel (a 16-byte vector), so every load and store is a full vector; the forward pass records the
// position of the maximum inside the window (one byte per element), and the backward pass is a gather over the
// at most ceil(k/s)^2 windows that cover an input pixel: no atomics, deterministic, each dx vector written once.
// Padded positions never win (they count as -inf), like the reference.
#include "common.cuh"

namespace mxb {

struct PoolShape {
  int N, H, W, C, Ho, Wo, kh, kw, sh, sw, ph, pw;
};

template <typename T>
__global__ void __launch_bounds__(256)
maxpool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int8_t* __restrict__ idx, const PoolShape p) {
  const int L = p.C >> 3;
  const int64_t nvec = (int64_t)p.N * p.Ho * p.Wo * L;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    const int cv = (int)(i % L);
    int64_t t = i / L;
    const int ow = (int)(t % p.Wo); t /= p.Wo;
    const int oh = (int)(t % p.Ho);
    const int n = (int)(t / p.Ho);
    float best[8];
    int bi[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { best[j] = -INFINITY; bi[j] = -1; }
    for (int r = 0; r < p.kh; ++r) {
      const int ih = oh * p.sh - p.ph + r;
      if (ih < 0 || ih >= p.H) continue;
      for (int s = 0; s < p.kw; ++s) {
        const int iw = ow * p.sw - p.pw + s;
        if (iw < 0 || iw >= p.W) continue;
        const Vec16<T> v = ld16(x + (((int64_t)n * p.H + ih) * p.W + iw) * p.C + cv * 8);
        const int code = r * p.kw + s;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float f = Cvt<T>::to_f(v.v[j]);
          if (bi[j] < 0 || f > best[j]) { best[j] = f; bi[j] = code; }
        }
      }
    }
    Vec16<T> o;
    int8_t codes[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { o.v[j] = Cvt<T>::from_f(best[j]); codes[j] = (int8_t)bi[j]; }
    st16(y + i * 8, o);
    *reinterpret_cast<uint2*>(idx + i * 8) = *reinterpret_cast<const uint2*>(codes);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
maxpool_bwd_kernel(const T* __restrict__ dy, const int8_t* __restrict__ idx, T* __restrict__ dx, const PoolShape p) {
  const int L = p.C >> 3;
  const int64_t nvec = (int64_t)p.N * p.H * p.W * L;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    const int cv = (int)(i % L);
    int64_t t = i / L;
    const int iw = (int)(t % p.W); t /= p.W;
    const int ih = (int)(t % p.H);
    const int n = (int)(t / p.H);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    // windows (oh, ow) with oh*sh - ph <= ih <= oh*sh - ph + kh - 1
    int oh0 = ih + p.ph - p.kh + 1;
    oh0 = oh0 <= 0 ? 0 : (oh0 + p.sh - 1) / p.sh;
    int oh1 = (ih + p.ph) / p.sh;
    if (oh1 > p.Ho - 1) oh1 = p.Ho - 1;
    int ow0 = iw + p.pw - p.kw + 1;
    ow0 = ow0 <= 0 ? 0 : (ow0 + p.sw - 1) / p.sw;
    int ow1 = (iw + p.pw) / p.sw;
    if (ow1 > p.Wo - 1) ow1 = p.Wo - 1;
    for (int oh = oh0; oh <= oh1; ++oh) {
      const int r = ih - (oh * p.sh - p.ph);
      for (int ow = ow0; ow <= ow1; ++ow) {
        const int s = iw - (ow * p.sw - p.pw);
        const int code = r * p.kw + s;
        const int64_t o = ((((int64_t)n * p.Ho + oh) * p.Wo + ow) * L + cv) * 8;
        const Vec16<T> g = ld16(dy + o);
        const uint2 raw = *reinterpret_cast<const uint2*>(idx + o);
        const int8_t* codes = reinterpret_cast<const int8_t*>(&raw);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if ((int)codes[j] == code) acc[j] += Cvt<T>::to_f(g.v[j]);
      }
    }
    Vec16<T> out;
#pragma unroll
    for (int j = 0; j < 8; ++j) out.v[j] = Cvt<T>::from_f(acc[j]);
    st16(dx + i * 8, out);
  }
}

inline int pool_grid(int64_t nvec) {
  int64_t blocks = (nvec + 255) / 256;
  int64_t cap = (int64_t)sm_count() * 8;
  if (blocks < 1) blocks = 1;
  return (int)(blocks < cap ? blocks : cap);
}

static bool pool_shape_ok(const PoolShape& p) {
  return p.N > 0 && p.H > 0 && p.W > 0 && p.C > 0 && (p.C % 8) == 0 && p.Ho > 0 && p.Wo > 0 && p.kh > 0 && p.kw > 0 &&
         p.kh * p.kw <= 127 && p.sh > 0 && p.sw > 0 && p.ph >= 0 && p.pw >= 0 && p.ph < p.kh && p.pw < p.kw &&
         (int64_t)(p.Ho - 1) * p.sh - p.ph < p.H && (int64_t)(p.Wo - 1) * p.sw - p.pw < p.W;
}

}  // namespace mxb

using namespace mxb;

// x: [N, H, W, C], y: [N, Ho, Wo, C] of `dtype` (fp16 / bf16), idx: [N, Ho, Wo, C] int8 (window position of the maximum).
MXB_EXPORT int mxb_maxpool_forward(int dtype, const void* x, void* y, void* idx, int N, int H, int W, int C, int Ho, int Wo,
                                   int kh, int kw, int sh, int sw, int ph, int pw, void* stream) {
  PoolShape p{N, H, W, C, Ho, Wo, kh, kw, sh, sw, ph, pw};
  if (!pool_shape_ok(p)) return -2;
  const int grid = pool_grid((int64_t)N * Ho * Wo * (C >> 3));
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == kF16) maxpool_fwd_kernel<__half><<<grid, 256, 0, st>>>((const __half*)x, (__half*)y, (int8_t*)idx, p);
  else if (dtype == kBF16) maxpool_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, (int8_t*)idx, p);
  else return -1;
  return (int)cudaGetLastError();
}

MXB_EXPORT int mxb_maxpool_backward(int dtype, const void* dy, const void* idx, void* dx, int N, int H, int W, int C, int Ho,
                                    int Wo, int kh, int kw, int sh, int sw, int ph, int pw, void* stream) {
  PoolShape p{N, H, W, C, Ho, Wo, kh, kw, sh, sw, ph, pw};
  if (!pool_shape_ok(p)) return -2;
  const int grid = pool_grid((int64_t)N * H * W * (C >> 3));
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == kF16) maxpool_bwd_kernel<__half><<<grid, 256, 0, st>>>((const __half*)dy, (const int8_t*)idx, (__half*)dx, p);
  else if (dtype == kBF16) maxpool_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)dy, (const int8_t*)idx, (__nv_bfloat16*)dx, p);
  else return -1;
  return (int)cudaGetLastError();
}

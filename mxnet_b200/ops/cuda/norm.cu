// BatchNorm (NHWC, fused ReLU / residual add) and LayerNorm kernels for sm_100a.
//
// Reference behaviour: src/operator/nn/batch_norm.cu (block-per-channel kernels, any axis) and the
// cuDNN spatial-persistent path; src/operator/nn/layer_norm.cu (fused row kernels).  These are
// HBM-bound: every pass moves 16-byte vectors, statistics are accumulated in fp32, and the
// activation (and the residual add of a ResNet block) are applied in the same pass that normalises,
// so a BN+add+ReLU group reads x (twice), the residual (once) and writes y (once).
//
// BatchNorm layout: x is [M, C] with C contiguous (M = N*H*W), C = 8*L with L a power of two <= 256.
// Statistics are reduced in two deterministic stages: per-CTA partial sums into a scratch buffer
// [grid][2][C], then a per-channel finalize kernel (no atomics, bitwise reproducible).
#include "common.cuh"

namespace mxb {

constexpr int kBnThreads = 256;

template <typename T, bool kBackward, bool kRelu>
__global__ void __launch_bounds__(kBnThreads)
bn_reduce_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ y,
                 const float* __restrict__ mean, const float* __restrict__ invstd, int64_t M, int C,
                 float* __restrict__ partial) {
  // forward: partial = {sum x, sum x^2};  backward: partial = {sum dy', sum dy' * xhat}
  __shared__ float sh[2][kBnThreads * 8];
  const int L = C >> 3;
  const int v = threadIdx.x % L, r = threadIdx.x / L, R = kBnThreads / L;
  float s[8], q[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { s[j] = 0.f; q[j] = 0.f; }
  float mu[8], is[8];
  if (kBackward) {
#pragma unroll
    for (int j = 0; j < 8; ++j) { mu[j] = mean[v * 8 + j]; is[j] = invstd[v * 8 + j]; }
  }
  for (int64_t row = (int64_t)blockIdx.x * R + r; row < M; row += (int64_t)gridDim.x * R) {
    const int64_t off = row * C + v * 8;
    Vec16<T> a = ld16(x + off);
    if (!kBackward) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { float f = Cvt<T>::to_f(a.v[j]); s[j] += f; q[j] += f * f; }
    } else {
      Vec16<T> g = ld16(dy + off);
      Vec16<T> o;
      if (kRelu) o = ld16(y + off);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float d = Cvt<T>::to_f(g.v[j]);
        if (kRelu && !(Cvt<T>::to_f(o.v[j]) > 0.f)) d = 0.f;
        float xh = (Cvt<T>::to_f(a.v[j]) - mu[j]) * is[j];
        s[j] += d;
        q[j] += d * xh;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    sh[0][r * C + v * 8 + j] = s[j];
    sh[1][r * C + v * 8 + j] = q[j];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += kBnThreads) {
    float a = 0.f, b = 0.f;
    for (int rr = 0; rr < R; ++rr) { a += sh[0][rr * C + c]; b += sh[1][rr * C + c]; }
    partial[((int64_t)blockIdx.x * 2 + 0) * C + c] = a;
    partial[((int64_t)blockIdx.x * 2 + 1) * C + c] = b;
  }
}

// Forward finalize: statistics, running averages, fused scale/shift.
__global__ void bn_fwd_finalize_kernel(const float* __restrict__ partial, int nblocks, int C, int64_t M, float eps,
                                       float momentum, const float* __restrict__ gamma, const float* __restrict__ beta,
                                       float* __restrict__ running_mean, float* __restrict__ running_var,
                                       float* __restrict__ save_mean, float* __restrict__ save_invstd,
                                       float* __restrict__ scale, float* __restrict__ shift, int training) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float mean, var;
  if (training) {
    float s = 0.f, q = 0.f;
    for (int b = 0; b < nblocks; ++b) { s += partial[((int64_t)b * 2) * C + c]; q += partial[((int64_t)b * 2 + 1) * C + c]; }
    mean = s / (float)M;
    var = fmaxf(q / (float)M - mean * mean, 0.f);
    running_mean[c] = running_mean[c] * momentum + mean * (1.f - momentum);
    running_var[c] = running_var[c] * momentum + var * (1.f - momentum);
  } else {
    mean = running_mean[c];
    var = running_var[c];
  }
  float is = rsqrtf(var + eps);
  save_mean[c] = mean;
  save_invstd[c] = is;
  float sc = gamma[c] * is;
  scale[c] = sc;
  shift[c] = beta[c] - mean * sc;
}

template <typename T, bool kRelu, bool kRes>
__global__ void __launch_bounds__(256)
bn_fwd_apply_kernel(const T* __restrict__ x, const T* __restrict__ res, const float* __restrict__ scale,
                    const float* __restrict__ shift, T* __restrict__ y, int64_t nvec, int L) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    const int c0 = (int)(i % L) * 8;
    Vec16<T> a = ld16(x + i * 8), o, rr;
    if (kRes) rr = ld16(res + i * 8);
    const float4 s0 = *reinterpret_cast<const float4*>(scale + c0), s1 = *reinterpret_cast<const float4*>(scale + c0 + 4);
    const float4 h0 = *reinterpret_cast<const float4*>(shift + c0), h1 = *reinterpret_cast<const float4*>(shift + c0 + 4);
    const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    const float sf[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float f = Cvt<T>::to_f(a.v[j]) * sc[j] + sf[j];
      if (kRes) f += Cvt<T>::to_f(rr.v[j]);
      if (kRelu) f = fmaxf(f, 0.f);
      o.v[j] = Cvt<T>::from_f(f);
    }
    st16(y + i * 8, o);
  }
}

// Backward finalize: dgamma, dbeta and the three per-channel coefficients of dx.
__global__ void bn_bwd_finalize_kernel(const float* __restrict__ partial, int nblocks, int C, int64_t M,
                                       const float* __restrict__ gamma, const float* __restrict__ invstd,
                                       float* __restrict__ dgamma, float* __restrict__ dbeta, float* __restrict__ coef) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f, q = 0.f;
  for (int b = 0; b < nblocks; ++b) { s += partial[((int64_t)b * 2) * C + c]; q += partial[((int64_t)b * 2 + 1) * C + c]; }
  dbeta[c] = s;
  dgamma[c] = q;
  coef[c] = gamma[c] * invstd[c];
  coef[C + c] = s / (float)M;
  coef[2 * C + c] = q / (float)M;
}

template <typename T, bool kRelu, bool kRes>
__global__ void __launch_bounds__(256)
bn_bwd_apply_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ y,
                    const float* __restrict__ mean, const float* __restrict__ invstd, const float* __restrict__ coef,
                    T* __restrict__ dx, T* __restrict__ dres, int64_t nvec, int L, int C) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    const int c0 = (int)(i % L) * 8;
    Vec16<T> a = ld16(x + i * 8), g = ld16(dy + i * 8), o, od, yy;
    if (kRelu) yy = ld16(y + i * 8);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = c0 + j;
      float d = Cvt<T>::to_f(g.v[j]);
      if (kRelu && !(Cvt<T>::to_f(yy.v[j]) > 0.f)) d = 0.f;
      float xh = (Cvt<T>::to_f(a.v[j]) - mean[c]) * invstd[c];
      o.v[j] = Cvt<T>::from_f(coef[c] * (d - coef[C + c] - xh * coef[2 * C + c]));
      if (kRes) od.v[j] = Cvt<T>::from_f(d);
    }
    st16(dx + i * 8, o);
    if (kRes) st16(dres + i * 8, od);
  }
}

inline int bn_grid(int64_t M, int C) {
  int R = kBnThreads / (C >> 3);
  int64_t need = (M + R - 1) / R;
  int64_t cap = (int64_t)sm_count() * 4;
  return (int)(need < cap ? (need < 1 ? 1 : need) : cap);
}

template <typename T>
int bn_forward_t(const T* x, const T* res, const float* gamma, const float* beta, float* rmean, float* rvar,
                 float* save_mean, float* save_invstd, float* scratch, T* y, int64_t M, int C, float eps, float momentum,
                 int training, int relu, cudaStream_t st) {
  const int grid = bn_grid(M, C);
  float* partial = scratch;                         // [grid][2][C]
  float* scale = scratch + (int64_t)grid * 2 * C;   // [C]
  float* shift = scale + C;                         // [C]
  if (training) bn_reduce_kernel<T, false, false><<<grid, kBnThreads, 0, st>>>(x, nullptr, nullptr, nullptr, nullptr, M, C, partial);
  bn_fwd_finalize_kernel<<<(C + 127) / 128, 128, 0, st>>>(partial, grid, C, M, eps, momentum, gamma, beta, rmean, rvar,
                                                          save_mean, save_invstd, scale, shift, training);
  const int64_t nvec = M * (C >> 3);
  int64_t blocks = (nvec + 255) / 256;
  int64_t cap = (int64_t)sm_count() * 8;
  int g2 = (int)(blocks < cap ? blocks : cap);
  const int L = C >> 3;
  if (relu && res) bn_fwd_apply_kernel<T, true, true><<<g2, 256, 0, st>>>(x, res, scale, shift, y, nvec, L);
  else if (relu) bn_fwd_apply_kernel<T, true, false><<<g2, 256, 0, st>>>(x, res, scale, shift, y, nvec, L);
  else if (res) bn_fwd_apply_kernel<T, false, true><<<g2, 256, 0, st>>>(x, res, scale, shift, y, nvec, L);
  else bn_fwd_apply_kernel<T, false, false><<<g2, 256, 0, st>>>(x, res, scale, shift, y, nvec, L);
  return (int)cudaGetLastError();
}

template <typename T>
int bn_backward_t(const T* x, const T* dy, const T* y, const float* gamma, const float* save_mean,
                  const float* save_invstd, float* scratch, T* dx, T* dres, float* dgamma, float* dbeta, int64_t M, int C,
                  int relu, cudaStream_t st) {
  const int grid = bn_grid(M, C);
  float* partial = scratch;
  float* coef = scratch + (int64_t)grid * 2 * C;    // [3][C]
  if (relu) bn_reduce_kernel<T, true, true><<<grid, kBnThreads, 0, st>>>(x, dy, y, save_mean, save_invstd, M, C, partial);
  else bn_reduce_kernel<T, true, false><<<grid, kBnThreads, 0, st>>>(x, dy, y, save_mean, save_invstd, M, C, partial);
  bn_bwd_finalize_kernel<<<(C + 127) / 128, 128, 0, st>>>(partial, grid, C, M, gamma, save_invstd, dgamma, dbeta, coef);
  const int64_t nvec = M * (C >> 3);
  int64_t blocks = (nvec + 255) / 256;
  int64_t cap = (int64_t)sm_count() * 8;
  int g2 = (int)(blocks < cap ? blocks : cap);
  const int L = C >> 3;
  if (relu && dres) bn_bwd_apply_kernel<T, true, true><<<g2, 256, 0, st>>>(x, dy, y, save_mean, save_invstd, coef, dx, dres, nvec, L, C);
  else if (relu) bn_bwd_apply_kernel<T, true, false><<<g2, 256, 0, st>>>(x, dy, y, save_mean, save_invstd, coef, dx, dres, nvec, L, C);
  else if (dres) bn_bwd_apply_kernel<T, false, true><<<g2, 256, 0, st>>>(x, dy, y, save_mean, save_invstd, coef, dx, dres, nvec, L, C);
  else bn_bwd_apply_kernel<T, false, false><<<g2, 256, 0, st>>>(x, dy, y, save_mean, save_invstd, coef, dx, dres, nvec, L, C);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// LayerNorm over the last axis: x [rows, C]
// ------------------------------------------------------------------------------------------------
constexpr int kLnThreads = 256;
constexpr int kLnMaxPerThread = 8;     // C <= 2048

template <typename T>
__global__ void __launch_bounds__(kLnThreads)
ln_fwd_kernel(const T* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
              T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out, int64_t rows, int C, float eps) {
  __shared__ float red[32];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * C;
    float v[kLnMaxPerThread];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < kLnMaxPerThread; ++k) {
      int c = threadIdx.x + k * kLnThreads;
      v[k] = c < C ? Cvt<T>::to_f(xr[c]) : 0.f;
      s += v[k];
    }
    const float mean = block_sum(s, red) / (float)C;
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < kLnMaxPerThread; ++k) {
      int c = threadIdx.x + k * kLnThreads;
      float d = c < C ? v[k] - mean : 0.f;
      q += d * d;
    }
    const float rstd = rsqrtf(block_sum(q, red) / (float)C + eps);
    if (threadIdx.x == 0) { mean_out[row] = mean; rstd_out[row] = rstd; }
    T* yr = y + row * C;
#pragma unroll
    for (int k = 0; k < kLnMaxPerThread; ++k) {
      int c = threadIdx.x + k * kLnThreads;
      if (c < C) yr[c] = Cvt<T>::from_f((v[k] - mean) * rstd * gamma[c] + beta[c]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kLnThreads)
ln_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy, const float* __restrict__ gamma,
              const float* __restrict__ mean, const float* __restrict__ rstd, T* __restrict__ dx,
              float* __restrict__ partial /*[grid][2][C]*/, int64_t rows, int C) {
  __shared__ float red[32];
  float dg[kLnMaxPerThread], db[kLnMaxPerThread];
#pragma unroll
  for (int k = 0; k < kLnMaxPerThread; ++k) { dg[k] = 0.f; db[k] = 0.f; }
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * C;
    const T* gr = dy + row * C;
    const float mu = mean[row], rs = rstd[row];
    float xh[kLnMaxPerThread], g[kLnMaxPerThread];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < kLnMaxPerThread; ++k) {
      int c = threadIdx.x + k * kLnThreads;
      if (c < C) {
        xh[k] = (Cvt<T>::to_f(xr[c]) - mu) * rs;
        float d = Cvt<T>::to_f(gr[c]);
        dg[k] += d * xh[k];
        db[k] += d;
        g[k] = d * gamma[c];
        s1 += g[k];
        s2 += g[k] * xh[k];
      } else { xh[k] = 0.f; g[k] = 0.f; }
    }
    s1 = block_sum(s1, red) / (float)C;
    s2 = block_sum(s2, red) / (float)C;
    T* dr = dx + row * C;
#pragma unroll
    for (int k = 0; k < kLnMaxPerThread; ++k) {
      int c = threadIdx.x + k * kLnThreads;
      if (c < C) dr[c] = Cvt<T>::from_f(rs * (g[k] - s1 - xh[k] * s2));
    }
  }
#pragma unroll
  for (int k = 0; k < kLnMaxPerThread; ++k) {
    int c = threadIdx.x + k * kLnThreads;
    if (c < C) {
      partial[((int64_t)blockIdx.x * 2 + 0) * C + c] = dg[k];
      partial[((int64_t)blockIdx.x * 2 + 1) * C + c] = db[k];
    }
  }
}

__global__ void ln_bwd_finalize_kernel(const float* __restrict__ partial, int nblocks, int C, float* __restrict__ dgamma,
                                       float* __restrict__ dbeta) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float a = 0.f, b = 0.f;
  for (int k = 0; k < nblocks; ++k) { a += partial[((int64_t)k * 2) * C + c]; b += partial[((int64_t)k * 2 + 1) * C + c]; }
  dgamma[c] = a;
  dbeta[c] = b;
}

inline int ln_grid(int64_t rows) {
  int64_t cap = (int64_t)sm_count() * 4;
  return (int)(rows < cap ? (rows < 1 ? 1 : rows) : cap);
}

}  // namespace mxb

using namespace mxb;

// Number of CTAs the BatchNorm reductions use for (M, C): the caller sizes the scratch buffer as
// (grid * 2 + 3) * C floats.
MXB_EXPORT int mxb_bn_grid(int64_t M, int C) { return bn_grid(M, C); }
MXB_EXPORT int mxb_ln_grid(int64_t rows) { return ln_grid(rows); }

MXB_EXPORT int mxb_bn_forward(int dtype, const void* x, const void* res, const float* gamma, const float* beta,
                              float* rmean, float* rvar, float* save_mean, float* save_invstd, float* scratch, void* y,
                              int64_t M, int C, float eps, float momentum, int training, int relu, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == kF16)
    return bn_forward_t<__half>((const __half*)x, (const __half*)res, gamma, beta, rmean, rvar, save_mean, save_invstd,
                                scratch, (__half*)y, M, C, eps, momentum, training, relu, st);
  if (dtype == kBF16)
    return bn_forward_t<__nv_bfloat16>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res, gamma, beta, rmean, rvar,
                                       save_mean, save_invstd, scratch, (__nv_bfloat16*)y, M, C, eps, momentum, training,
                                       relu, st);
  return -1;
}

MXB_EXPORT int mxb_bn_backward(int dtype, const void* x, const void* dy, const void* y, const float* gamma,
                               const float* save_mean, const float* save_invstd, float* scratch, void* dx, void* dres,
                               float* dgamma, float* dbeta, int64_t M, int C, int relu, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == kF16)
    return bn_backward_t<__half>((const __half*)x, (const __half*)dy, (const __half*)y, gamma, save_mean, save_invstd,
                                 scratch, (__half*)dx, (__half*)dres, dgamma, dbeta, M, C, relu, st);
  if (dtype == kBF16)
    return bn_backward_t<__nv_bfloat16>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)y, gamma,
                                        save_mean, save_invstd, scratch, (__nv_bfloat16*)dx, (__nv_bfloat16*)dres, dgamma,
                                        dbeta, M, C, relu, st);
  return -1;
}

template <typename T>
static int ln_fwd_t(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd, int64_t rows,
                    int C, float eps, cudaStream_t st) {
  ln_fwd_kernel<T><<<ln_grid(rows), kLnThreads, 0, st>>>((const T*)x, gamma, beta, (T*)y, mean, rstd, rows, C, eps);
  return (int)cudaGetLastError();
}
template <typename T>
static int ln_bwd_t(const void* x, const void* dy, const float* gamma, const float* mean, const float* rstd, void* dx,
                    float* dgamma, float* dbeta, float* scratch, int64_t rows, int C, cudaStream_t st) {
  int grid = ln_grid(rows);
  ln_bwd_kernel<T><<<grid, kLnThreads, 0, st>>>((const T*)x, (const T*)dy, gamma, mean, rstd, (T*)dx, scratch, rows, C);
  ln_bwd_finalize_kernel<<<(C + 127) / 128, 128, 0, st>>>(scratch, grid, C, dgamma, dbeta);
  return (int)cudaGetLastError();
}

MXB_EXPORT int mxb_ln_forward(int dtype, const void* x, const float* gamma, const float* beta, void* y, float* mean,
                              float* rstd, int64_t rows, int C, float eps, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (C > kLnThreads * kLnMaxPerThread) return -2;
  if (dtype == kF32) return ln_fwd_t<float>(x, gamma, beta, y, mean, rstd, rows, C, eps, st);
  if (dtype == kF16) return ln_fwd_t<__half>(x, gamma, beta, y, mean, rstd, rows, C, eps, st);
  if (dtype == kBF16) return ln_fwd_t<__nv_bfloat16>(x, gamma, beta, y, mean, rstd, rows, C, eps, st);
  return -1;
}

// scratch: ln_grid(rows) * 2 * C floats
MXB_EXPORT int mxb_ln_backward(int dtype, const void* x, const void* dy, const float* gamma, const float* mean,
                               const float* rstd, void* dx, float* dgamma, float* dbeta, float* scratch, int64_t rows,
                               int C, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (C > kLnThreads * kLnMaxPerThread) return -2;
  if (dtype == kF32) return ln_bwd_t<float>(x, dy, gamma, mean, rstd, dx, dgamma, dbeta, scratch, rows, C, st);
  if (dtype == kF16) return ln_bwd_t<__half>(x, dy, gamma, mean, rstd, dx, dgamma, dbeta, scratch, rows, C, st);
  if (dtype == kBF16) return ln_bwd_t<__nv_bfloat16>(x, dy, gamma, mean, rstd, dx, dgamma, dbeta, scratch, rows, C, st);
  return -1;
}

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
//
// Backward of BN+ReLU without a residual does not read y: the mask y > 0 is recomputed from x and the
// per-channel scale/shift.  With a residual the mask comes from y.  dx is evaluated as
// A[c]*dy' + B[c]*x + D[c] with three per-channel coefficients prepared by the finalize kernel.
#include "common.cuh"

namespace mxb {

constexpr int kBnThreads = 256;
enum BnRelu { kReluNone = 0, kReluFromX = 1, kReluFromY = 2 };

__device__ __forceinline__ float load_param(const void* p, int dtype, int c) {
  if (dtype == kF32) return static_cast<const float*>(p)[c];
  if (dtype == kF16) return __half2float(static_cast<const __half*>(p)[c]);
  return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[c]);
}
__device__ __forceinline__ void store_param(void* p, int dtype, int c, float v) {
  if (dtype == kF32) static_cast<float*>(p)[c] = v;
  else if (dtype == kF16) static_cast<__half*>(p)[c] = __float2half_rn(v);
  else static_cast<__nv_bfloat16*>(p)[c] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ void load8(const float* p, float* out) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w; out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}

// forward (kBackward = false): partial = {sum x, sum x^2}
// backward: partial = {sum dy', sum dy' * xhat} with dy' = dy masked by the ReLU
template <typename T, bool kBackward, int kRelu>
__global__ void __launch_bounds__(kBnThreads)
bn_reduce_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ y,
                 const float* __restrict__ mean, const float* __restrict__ invstd, const float* __restrict__ scale,
                 const float* __restrict__ shift, int64_t M, int C, float* __restrict__ partial) {
  __shared__ float sh[2][kBnThreads * 8];
  const int L = C >> 3;
  const int v = threadIdx.x % L, r = threadIdx.x / L, R = kBnThreads / L;
  float s[8], q[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { s[j] = 0.f; q[j] = 0.f; }
  float mu[8], is[8], sc[8], sf[8];
  if (kBackward) {
    load8(mean + v * 8, mu);
    load8(invstd + v * 8, is);
    if (kRelu == kReluFromX) { load8(scale + v * 8, sc); load8(shift + v * 8, sf); }
  }
  const int64_t stride = (int64_t)gridDim.x * R;
  for (int64_t row = (int64_t)blockIdx.x * R + r; row < M; row += 2 * stride) {
    // two rows per trip keep more 16-byte loads in flight per thread
    const int64_t off0 = row * C + v * 8;
    const bool two = row + stride < M;
    const int64_t off1 = two ? off0 + stride * C : off0;
    Vec16<T> a0 = ld16(x + off0), a1 = ld16(x + off1);
    if (!kBackward) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float f0 = Cvt<T>::to_f(a0.v[j]), f1 = two ? Cvt<T>::to_f(a1.v[j]) : 0.f;
        s[j] += f0 + f1;
        q[j] += f0 * f0 + f1 * f1;
      }
    } else {
      Vec16<T> g0 = ld16(dy + off0), g1 = ld16(dy + off1), o0, o1;
      if (kRelu == kReluFromY) { o0 = ld16(y + off0); o1 = ld16(y + off1); }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float x0 = Cvt<T>::to_f(a0.v[j]), x1 = Cvt<T>::to_f(a1.v[j]);
        float d0 = Cvt<T>::to_f(g0.v[j]), d1 = two ? Cvt<T>::to_f(g1.v[j]) : 0.f;
        if (kRelu == kReluFromY) {
          if (!(Cvt<T>::to_f(o0.v[j]) > 0.f)) d0 = 0.f;
          if (!(Cvt<T>::to_f(o1.v[j]) > 0.f)) d1 = 0.f;
        } else if (kRelu == kReluFromX) {
          if (!(x0 * sc[j] + sf[j] > 0.f)) d0 = 0.f;
          if (!(x1 * sc[j] + sf[j] > 0.f)) d1 = 0.f;
        }
        s[j] += d0 + d1;
        q[j] += d0 * ((x0 - mu[j]) * is[j]) + d1 * ((x1 - mu[j]) * is[j]);
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

// Sum the per-CTA partials of 8 channels with an (8 x 128) thread block: a few hundred partial rows are one or two
// independent loads per thread, so the kernel is one memory round trip instead of a dependent chain, and C / 8 blocks
// spread it over the SMs; fixed-order tree in shared memory (deterministic).
constexpr int kFinX = 8, kFinY = 128;
__device__ __forceinline__ bool finalize_sums(const float* __restrict__ partial, int nblocks, int C, float& s, float& q) {
  __shared__ float red[2][kFinY][kFinX];
  const int c = blockIdx.x * kFinX + threadIdx.x;
  float a = 0.f, b = 0.f;
  if (c < C) {
    // four independent loads per trip keep the L2 round trips overlapped; the order of additions is fixed
    int k = threadIdx.y;
    for (; k + 3 * kFinY < nblocks; k += 4 * kFinY) {
      const float a0 = partial[((int64_t)k * 2) * C + c], b0 = partial[((int64_t)k * 2 + 1) * C + c];
      const float a1 = partial[((int64_t)(k + kFinY) * 2) * C + c], b1 = partial[((int64_t)(k + kFinY) * 2 + 1) * C + c];
      const float a2 = partial[((int64_t)(k + 2 * kFinY) * 2) * C + c], b2 = partial[((int64_t)(k + 2 * kFinY) * 2 + 1) * C + c];
      const float a3 = partial[((int64_t)(k + 3 * kFinY) * 2) * C + c], b3 = partial[((int64_t)(k + 3 * kFinY) * 2 + 1) * C + c];
      a += (a0 + a1) + (a2 + a3);
      b += (b0 + b1) + (b2 + b3);
    }
    for (; k < nblocks; k += kFinY) {
      a += partial[((int64_t)k * 2) * C + c];
      b += partial[((int64_t)k * 2 + 1) * C + c];
    }
  }
  red[0][threadIdx.y][threadIdx.x] = a;
  red[1][threadIdx.y][threadIdx.x] = b;
  __syncthreads();
  // 128 -> 32 rows in parallel, then one thread per channel adds the 32 rows in order
  if (threadIdx.y < 32) {
    const int y = threadIdx.y;
    red[0][y][threadIdx.x] = (red[0][y][threadIdx.x] + red[0][y + 32][threadIdx.x]) +
                             (red[0][y + 64][threadIdx.x] + red[0][y + 96][threadIdx.x]);
    red[1][y][threadIdx.x] = (red[1][y][threadIdx.x] + red[1][y + 32][threadIdx.x]) +
                             (red[1][y + 64][threadIdx.x] + red[1][y + 96][threadIdx.x]);
  }
  __syncthreads();
  if (threadIdx.y != 0 || c >= C) return false;
  s = 0.f; q = 0.f;
#pragma unroll
  for (int k = 0; k < 32; ++k) { s += red[0][k][threadIdx.x]; q += red[1][k][threadIdx.x]; }
  return true;
}

// Forward finalize: statistics, running averages, fused scale/shift.
__global__ void __launch_bounds__(kFinX * kFinY)
bn_fwd_finalize_kernel(const float* __restrict__ partial, int nblocks, int C, int64_t M, float eps, float momentum,
                       const void* __restrict__ gamma, const void* __restrict__ beta, int pdtype,
                       float* __restrict__ running_mean, float* __restrict__ running_var, float* __restrict__ save_mean,
                       float* __restrict__ save_invstd, float* __restrict__ scale, float* __restrict__ shift, int training) {
  float s = 0.f, q = 0.f;
  float mean, var;
  const int c = blockIdx.x * kFinX + threadIdx.x;
  if (training) {
    if (!finalize_sums(partial, nblocks, C, s, q)) return;
    mean = s / (float)M;
    var = fmaxf(q / (float)M - mean * mean, 0.f);
    running_mean[c] = running_mean[c] * momentum + mean * (1.f - momentum);
    running_var[c] = running_var[c] * momentum + var * (1.f - momentum);
  } else {
    if (threadIdx.y != 0 || c >= C) return;
    mean = running_mean[c];
    var = running_var[c];
  }
  const float is = rsqrtf(var + eps);
  save_mean[c] = mean;
  save_invstd[c] = is;
  const float sc = load_param(gamma, pdtype, c) * is;
  scale[c] = sc;
  shift[c] = load_param(beta, pdtype, c) - mean * sc;
}

template <typename T, bool kRelu, bool kRes>
__global__ void __launch_bounds__(256)
bn_fwd_apply_kernel(const T* __restrict__ x, const T* __restrict__ res, const float* __restrict__ scale,
                    const float* __restrict__ shift, T* __restrict__ y, int64_t nvec, int L) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    const int c0 = (int)(i % L) * 8;
    Vec16<T> a = ld16(x + i * 8), o, rr;
    if (kRes) rr = ld16(res + i * 8);
    float sc[8], sf[8];
    load8(scale + c0, sc);
    load8(shift + c0, sf);
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

// Backward finalize: dgamma, dbeta and the per-channel coefficients of dx = A*dy' + B*x + D.
// coef layout: [A | B | D], each C floats.
__global__ void __launch_bounds__(kFinX * kFinY)
bn_bwd_finalize_kernel(const float* __restrict__ partial, int nblocks, int C, int64_t M, const void* __restrict__ gamma,
                       int pdtype, const float* __restrict__ mean, const float* __restrict__ invstd,
                       void* __restrict__ dgamma, void* __restrict__ dbeta, float* __restrict__ coef) {
  float s, q;
  if (!finalize_sums(partial, nblocks, C, s, q)) return;
  const int c = blockIdx.x * kFinX + threadIdx.x;
  store_param(dbeta, pdtype, c, s);
  store_param(dgamma, pdtype, c, q);
  const float is = invstd[c], mu = mean[c];
  const float A = load_param(gamma, pdtype, c) * is;
  const float ms = s / (float)M, mq = q / (float)M;
  coef[c] = A;
  coef[C + c] = -A * mq * is;
  coef[2 * C + c] = A * (mu * is * mq - ms);
}

template <typename T, int kRelu, bool kRes>
__global__ void __launch_bounds__(256)
bn_bwd_apply_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ y,
                    const float* __restrict__ scale, const float* __restrict__ shift, const float* __restrict__ coef,
                    T* __restrict__ dx, T* __restrict__ dres, int64_t nvec, int L, int C) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    const int c0 = (int)(i % L) * 8;
    Vec16<T> a = ld16(x + i * 8), g = ld16(dy + i * 8), o, od, yy;
    if (kRelu == kReluFromY) yy = ld16(y + i * 8);
    float A[8], B[8], D[8], sc[8], sf[8];
    load8(coef + c0, A);
    load8(coef + C + c0, B);
    load8(coef + 2 * C + c0, D);
    if (kRelu == kReluFromX) { load8(scale + c0, sc); load8(shift + c0, sf); }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float xv = Cvt<T>::to_f(a.v[j]);
      float d = Cvt<T>::to_f(g.v[j]);
      if (kRelu == kReluFromY) { if (!(Cvt<T>::to_f(yy.v[j]) > 0.f)) d = 0.f; }
      else if (kRelu == kReluFromX) { if (!(xv * sc[j] + sf[j] > 0.f)) d = 0.f; }
      o.v[j] = Cvt<T>::from_f(A[j] * d + B[j] * xv + D[j]);
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

inline int apply_grid(int64_t nvec) {
  int64_t blocks = (nvec + 255) / 256;
  int64_t cap = (int64_t)sm_count() * 8;
  return (int)(blocks < cap ? blocks : cap);
}

// scratch layout (floats): [grid][2][C] partials | scale[C] | shift[C] | coef[3][C]
template <typename T>
int bn_forward_t(const T* x, const T* res, const void* gamma, const void* beta, int pdtype, float* rmean, float* rvar,
                 float* save_mean, float* save_invstd, float* scale_shift, float* scratch, T* y, int64_t M, int C, float eps,
                 float momentum, int training, int relu, cudaStream_t st, const float* ext_partial = nullptr,
                 int ext_rows = 0) {
  const int grid = ext_partial ? ext_rows : bn_grid(M, C);
  float* scale = scale_shift;
  float* shift = scale_shift + C;
  // batch statistics: reduced here, or taken from partial sums that the producer of x already accumulated
  if (training && !ext_partial)
    bn_reduce_kernel<T, false, kReluNone><<<grid, kBnThreads, 0, st>>>(x, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                                                                       M, C, scratch);
  bn_fwd_finalize_kernel<<<(C + kFinX - 1) / kFinX, dim3(kFinX, kFinY), 0, st>>>(
      ext_partial ? ext_partial : scratch, grid, C, M, eps, momentum, gamma, beta, pdtype, rmean, rvar, save_mean, save_invstd,
      scale, shift, training);
  const int64_t nvec = M * (C >> 3);
  const int g2 = apply_grid(nvec);
  const int L = C >> 3;
  if (relu && res) bn_fwd_apply_kernel<T, true, true><<<g2, 256, 0, st>>>(x, res, scale, shift, y, nvec, L);
  else if (relu) bn_fwd_apply_kernel<T, true, false><<<g2, 256, 0, st>>>(x, res, scale, shift, y, nvec, L);
  else if (res) bn_fwd_apply_kernel<T, false, true><<<g2, 256, 0, st>>>(x, res, scale, shift, y, nvec, L);
  else bn_fwd_apply_kernel<T, false, false><<<g2, 256, 0, st>>>(x, res, scale, shift, y, nvec, L);
  return (int)cudaGetLastError();
}

template <typename T>
int bn_backward_t(const T* x, const T* dy, const T* y, const void* gamma, int pdtype, const float* save_mean,
                  const float* save_invstd, const float* scale_shift, float* scratch, T* dx, T* dres, void* dgamma,
                  void* dbeta, int64_t M, int C, int relu, cudaStream_t st) {
  const int grid = bn_grid(M, C);
  float* partial = scratch;
  float* coef = scratch + (int64_t)grid * 2 * C;    // [3][C]
  const float* scale = scale_shift;
  const float* shift = scale_shift + C;
  // a residual output means y = relu(bn(x) + res): the mask must come from y
  const int mode = !relu ? kReluNone : (dres ? kReluFromY : kReluFromX);
  if (mode == kReluFromY)
    bn_reduce_kernel<T, true, kReluFromY><<<grid, kBnThreads, 0, st>>>(x, dy, y, save_mean, save_invstd, scale, shift, M, C, partial);
  else if (mode == kReluFromX)
    bn_reduce_kernel<T, true, kReluFromX><<<grid, kBnThreads, 0, st>>>(x, dy, y, save_mean, save_invstd, scale, shift, M, C, partial);
  else
    bn_reduce_kernel<T, true, kReluNone><<<grid, kBnThreads, 0, st>>>(x, dy, y, save_mean, save_invstd, scale, shift, M, C, partial);
  bn_bwd_finalize_kernel<<<(C + kFinX - 1) / kFinX, dim3(kFinX, kFinY), 0, st>>>(partial, grid, C, M, gamma, pdtype, save_mean,
                                                                               save_invstd, dgamma, dbeta, coef);
  const int64_t nvec = M * (C >> 3);
  const int g2 = apply_grid(nvec);
  const int L = C >> 3;
  if (mode == kReluFromY && dres) bn_bwd_apply_kernel<T, kReluFromY, true><<<g2, 256, 0, st>>>(x, dy, y, scale, shift, coef, dx, dres, nvec, L, C);
  else if (mode == kReluFromX) bn_bwd_apply_kernel<T, kReluFromX, false><<<g2, 256, 0, st>>>(x, dy, y, scale, shift, coef, dx, dres, nvec, L, C);
  else if (dres) bn_bwd_apply_kernel<T, kReluNone, true><<<g2, 256, 0, st>>>(x, dy, y, scale, shift, coef, dx, dres, nvec, L, C);
  else bn_bwd_apply_kernel<T, kReluNone, false><<<g2, 256, 0, st>>>(x, dy, y, scale, shift, coef, dx, dres, nvec, L, C);
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

// Warp-per-row variants for half-precision rows of up to 1024 columns (C a multiple of 8): lane l owns the 16-byte
// vectors l, l + 32, ... of the row (NV of them), statistics are warp shuffles, so a row costs no block-wide barrier;
// eight rows are in flight per CTA.  The backward kernel keeps dgamma / dbeta per lane in registers over all rows of
// the warp and adds the eight warps of a CTA in a fixed order in shared memory before writing the CTA's partial row.
constexpr int kLnWarps = 8;

template <typename T, int NV>
__global__ void __launch_bounds__(kLnWarps * 32)
ln_fwd_warp_kernel(const T* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta, T* __restrict__ y,
                   float* __restrict__ mean_out, float* __restrict__ rstd_out, int64_t rows, int C, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = C >> 3;
  for (int64_t row = (int64_t)blockIdx.x * kLnWarps + warp; row < rows; row += (int64_t)gridDim.x * kLnWarps) {
    const T* xr = x + row * C;
    float v[NV][8];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int vi = lane + 32 * k;
      if (vi < nvec) {
        const Vec16<T> a = ld16(xr + vi * 8);
#pragma unroll
        for (int j = 0; j < 8; ++j) { v[k][j] = Cvt<T>::to_f(a.v[j]); s += v[k][j]; }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[k][j] = 0.f;
      }
    }
    const float mean = warp_sum(s) / (float)C;
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      if (lane + 32 * k < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { const float d = v[k][j] - mean; q += d * d; }
      }
    }
    const float rstd = rsqrtf(warp_sum(q) / (float)C + eps);
    if (lane == 0) { mean_out[row] = mean; rstd_out[row] = rstd; }
    T* yr = y + row * C;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int vi = lane + 32 * k;
      if (vi < nvec) {
        const float4 g0 = *reinterpret_cast<const float4*>(gamma + vi * 8), g1 = *reinterpret_cast<const float4*>(gamma + vi * 8 + 4);
        const float4 b0 = *reinterpret_cast<const float4*>(beta + vi * 8), b1 = *reinterpret_cast<const float4*>(beta + vi * 8 + 4);
        const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        Vec16<T> o;
#pragma unroll
        for (int j = 0; j < 8; ++j) o.v[j] = Cvt<T>::from_f((v[k][j] - mean) * rstd * gg[j] + bb[j]);
        st16(yr + vi * 8, o);
      }
    }
  }
}

template <typename T, int NV>
__global__ void __launch_bounds__(kLnWarps * 32, 2)
ln_bwd_warp_kernel(const T* __restrict__ x, const T* __restrict__ dy, const float* __restrict__ gamma,
                   const float* __restrict__ mean, const float* __restrict__ rstd, T* __restrict__ dx,
                   float* __restrict__ partial /*[grid][2][C]*/, int64_t rows, int C) {
  extern __shared__ float ln_acc[];          // [2][C]: dgamma | dbeta of this CTA
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = C >> 3;
  float dg[NV][8], db[NV][8];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
#pragma unroll
    for (int j = 0; j < 8; ++j) { dg[k][j] = 0.f; db[k][j] = 0.f; }
  }
  for (int64_t row = (int64_t)blockIdx.x * kLnWarps + warp; row < rows; row += (int64_t)gridDim.x * kLnWarps) {
    const T* xr = x + row * C;
    const T* gr = dy + row * C;
    const float mu = mean[row], rs = rstd[row];
    float xh[NV][8], g[NV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int vi = lane + 32 * k;
      if (vi < nvec) {
        const Vec16<T> a = ld16(xr + vi * 8), d = ld16(gr + vi * 8);
        const float4 g0 = *reinterpret_cast<const float4*>(gamma + vi * 8), g1 = *reinterpret_cast<const float4*>(gamma + vi * 8 + 4);
        const float gm[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[k][j] = (Cvt<T>::to_f(a.v[j]) - mu) * rs;
          const float dd = Cvt<T>::to_f(d.v[j]);
          dg[k][j] += dd * xh[k][j];
          db[k][j] += dd;
          g[k][j] = dd * gm[j];
          s1 += g[k][j];
          s2 += g[k][j] * xh[k][j];
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) { xh[k][j] = 0.f; g[k][j] = 0.f; }
      }
    }
    s1 = warp_sum(s1) / (float)C;
    s2 = warp_sum(s2) / (float)C;
    T* dr = dx + row * C;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int vi = lane + 32 * k;
      if (vi < nvec) {
        Vec16<T> o;
#pragma unroll
        for (int j = 0; j < 8; ++j) o.v[j] = Cvt<T>::from_f(rs * (g[k][j] - s1 - xh[k][j] * s2));
        st16(dr + vi * 8, o);
      }
    }
  }
  // the eight warps add their sums one after the other (fixed order) into the CTA's accumulators
  for (int i = threadIdx.x; i < 2 * C; i += blockDim.x) ln_acc[i] = 0.f;
  __syncthreads();
  for (int w = 0; w < kLnWarps; ++w) {
    if (warp == w) {
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int vi = lane + 32 * k;
        if (vi < nvec) {
#pragma unroll
          for (int j = 0; j < 8; ++j) { ln_acc[vi * 8 + j] += dg[k][j]; ln_acc[C + vi * 8 + j] += db[k][j]; }
        }
      }
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < 2 * C; i += blockDim.x) partial[(int64_t)blockIdx.x * 2 * C + i] = ln_acc[i];
}

__global__ void __launch_bounds__(kFinX * kFinY)
ln_bwd_finalize_kernel(const float* __restrict__ partial, int nblocks, int C, float* __restrict__ dgamma,
                       float* __restrict__ dbeta) {
  float a, b;
  if (!finalize_sums(partial, nblocks, C, a, b)) return;
  const int c = blockIdx.x * kFinX + threadIdx.x;
  dgamma[c] = a;
  dbeta[c] = b;
}

inline int ln_grid(int64_t rows) {
  int64_t cap = (int64_t)sm_count() * 4;
  return (int)(rows < cap ? (rows < 1 ? 1 : rows) : cap);
}

}  // namespace mxb

using namespace mxb;

// Number of CTAs the BatchNorm reductions use for (M, C); scratch sizes are stated at each entry point.
MXB_EXPORT int mxb_bn_grid(int64_t M, int C) { return bn_grid(M, C); }
MXB_EXPORT int mxb_ln_grid(int64_t rows) { return ln_grid(rows); }

// x, res, y: [M, C] of `dtype` (fp16 / bf16).  gamma, beta: C values of `pdtype`.  rmean, rvar, save_mean,
// save_invstd: C floats.  scale_shift: 2*C floats written here and read again by the backward pass.
// scratch: mxb_bn_grid(M, C) * 2 * C floats.
MXB_EXPORT int mxb_bn_forward(int dtype, const void* x, const void* res, const void* gamma, const void* beta, int pdtype,
                              float* rmean, float* rvar, float* save_mean, float* save_invstd, float* scale_shift,
                              float* scratch, void* y, int64_t M, int C, float eps, float momentum, int training, int relu,
                              void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (pdtype != kF32 && pdtype != kF16 && pdtype != kBF16) return -1;
  if (dtype == kF16)
    return bn_forward_t<__half>((const __half*)x, (const __half*)res, gamma, beta, pdtype, rmean, rvar, save_mean,
                                save_invstd, scale_shift, scratch, (__half*)y, M, C, eps, momentum, training, relu, st);
  if (dtype == kBF16)
    return bn_forward_t<__nv_bfloat16>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res, gamma, beta, pdtype, rmean, rvar,
                                       save_mean, save_invstd, scale_shift, scratch, (__nv_bfloat16*)y, M, C, eps, momentum,
                                       training, relu, st);
  return -1;
}

// Training-mode forward whose batch statistics come from `partial` ([rows][2][C] floats: per-channel sums of x and
// x*x, any split over the rows), e.g. from the epilogue of the convolution that produced x.
MXB_EXPORT int mxb_bn_forward_stats(int dtype, const void* x, const void* res, const void* gamma, const void* beta,
                                    int pdtype, float* rmean, float* rvar, float* save_mean, float* save_invstd,
                                    float* scale_shift, const float* partial, int rows, void* y, int64_t M, int C, float eps,
                                    float momentum, int relu, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (pdtype != kF32 && pdtype != kF16 && pdtype != kBF16) return -1;
  if (!partial || rows < 1) return -2;
  if (dtype == kF16)
    return bn_forward_t<__half>((const __half*)x, (const __half*)res, gamma, beta, pdtype, rmean, rvar, save_mean,
                                save_invstd, scale_shift, nullptr, (__half*)y, M, C, eps, momentum, 1, relu, st, partial, rows);
  if (dtype == kBF16)
    return bn_forward_t<__nv_bfloat16>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res, gamma, beta, pdtype, rmean, rvar,
                                       save_mean, save_invstd, scale_shift, nullptr, (__nv_bfloat16*)y, M, C, eps, momentum,
                                       1, relu, st, partial, rows);
  return -1;
}

// scratch: (mxb_bn_grid(M, C) * 2 + 3) * C floats.  dgamma, dbeta: C values of `pdtype`.  `y` is read only when
// relu != 0 and dres != nullptr (the mask of BN+add+ReLU); `dres` receives the gradient of the residual input.
MXB_EXPORT int mxb_bn_backward(int dtype, const void* x, const void* dy, const void* y, const void* gamma, int pdtype,
                               const float* save_mean, const float* save_invstd, const float* scale_shift, float* scratch,
                               void* dx, void* dres, void* dgamma, void* dbeta, int64_t M, int C, int relu, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (pdtype != kF32 && pdtype != kF16 && pdtype != kBF16) return -1;
  if (dtype == kF16)
    return bn_backward_t<__half>((const __half*)x, (const __half*)dy, (const __half*)y, gamma, pdtype, save_mean, save_invstd,
                                 scale_shift, scratch, (__half*)dx, (__half*)dres, dgamma, dbeta, M, C, relu, st);
  if (dtype == kBF16)
    return bn_backward_t<__nv_bfloat16>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)y, gamma,
                                        pdtype, save_mean, save_invstd, scale_shift, scratch, (__nv_bfloat16*)dx,
                                        (__nv_bfloat16*)dres, dgamma, dbeta, M, C, relu, st);
  return -1;
}

// rows of half-precision values with C % 8 == 0 and C <= 1024, 16-byte aligned: the warp-per-row kernels
template <typename T>
static bool ln_warp_ok(const void* x, const void* y, const float* gamma, const float* beta, int C) {
  return sizeof(T) == 2 && (C % 8) == 0 && C <= 1024 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)y % 16) == 0 &&
         ((uintptr_t)gamma % 16) == 0 && (beta == nullptr || ((uintptr_t)beta % 16) == 0);
}
inline int ln_warp_grid(int64_t rows) {
  const int64_t want = (rows + kLnWarps - 1) / kLnWarps, cap = (int64_t)sm_count() * 4;
  return (int)(want < cap ? (want < 1 ? 1 : want) : cap);
}

template <typename T>
static int ln_fwd_t(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd, int64_t rows,
                    int C, float eps, cudaStream_t st) {
  if constexpr (sizeof(T) == 2) if (ln_warp_ok<T>(x, y, gamma, beta, C)) {
    const int grid = ln_warp_grid(rows), nv = (C / 8 + 31) / 32;
#define MXB_LN_FWD(NV) ln_fwd_warp_kernel<T, NV><<<grid, kLnWarps * 32, 0, st>>>((const T*)x, gamma, beta, (T*)y, mean, rstd, rows, C, eps)
    if (nv == 1) MXB_LN_FWD(1); else if (nv == 2) MXB_LN_FWD(2); else if (nv == 3) MXB_LN_FWD(3); else MXB_LN_FWD(4);
#undef MXB_LN_FWD
    return (int)cudaGetLastError();
  }
  ln_fwd_kernel<T><<<ln_grid(rows), kLnThreads, 0, st>>>((const T*)x, gamma, beta, (T*)y, mean, rstd, rows, C, eps);
  return (int)cudaGetLastError();
}
template <typename T>
static int ln_bwd_t(const void* x, const void* dy, const float* gamma, const float* mean, const float* rstd, void* dx,
                    float* dgamma, float* dbeta, float* scratch, int64_t rows, int C, cudaStream_t st) {
  int grid = ln_grid(rows);
  bool warp_path = false;
  if constexpr (sizeof(T) == 2) warp_path = ln_warp_ok<T>(x, dx, gamma, nullptr, C) && ((uintptr_t)dy % 16) == 0;
  if constexpr (sizeof(T) == 2) if (warp_path) {
    // at most ln_grid(rows) CTAs, so the scratch sized for the block-per-row kernel is large enough
    const int wgrid = ln_warp_grid(rows) < grid ? ln_warp_grid(rows) : grid;
    const int nv = (C / 8 + 31) / 32;
    const size_t smem = (size_t)2 * C * sizeof(float);
#define MXB_LN_BWD(NV) ln_bwd_warp_kernel<T, NV><<<wgrid, kLnWarps * 32, smem, st>>>((const T*)x, (const T*)dy, gamma, mean, rstd, (T*)dx, scratch, rows, C)
    if (nv == 1) MXB_LN_BWD(1); else if (nv == 2) MXB_LN_BWD(2); else if (nv == 3) MXB_LN_BWD(3); else MXB_LN_BWD(4);
#undef MXB_LN_BWD
    grid = wgrid;
  }
  if (!warp_path)
    ln_bwd_kernel<T><<<grid, kLnThreads, 0, st>>>((const T*)x, (const T*)dy, gamma, mean, rstd, (T*)dx, scratch, rows, C);
  ln_bwd_finalize_kernel<<<(C + kFinX - 1) / kFinX, dim3(kFinX, kFinY), 0, st>>>(scratch, grid, C, dgamma, dbeta);
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

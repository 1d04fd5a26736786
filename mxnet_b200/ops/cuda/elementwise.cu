// Vectorised pointwise, gather and pooling kernels for sm_100a (all HBM-bound: 16-byte accesses, grid-stride loops).
//
// Reference behaviour:
//   GELU / bias + GELU           src/operator/leaky_relu-inl.h (erf form), src/operator/mshadow_op.h
//   Dropout (+ bias + residual)  src/operator/nn/dropout-inl.h:72-84 (Bernoulli keep mask scaled by 1/(1-p))
//   add_n                        src/operator/tensor/elemwise_sum.h
//   cast / amp_cast              src/operator/tensor/elemwise_unary_op.h, src/operator/tensor/amp_cast.h
//   Embedding / take             src/operator/tensor/indexing_op.cu:712-820 (sorted, segmented gradient)
//   avg / global avg pooling     src/operator/nn/pool.cuh
//   2-D transpose                src/operator/tensor/pseudo2DTranspose_op-inl.cuh
//
// Dropout keeps no mask tensor: an element is kept when a counter-based hash of (seed word, element index) passes a
// threshold, and the backward pass recomputes the same decision from the same device-resident seed word.
#include "common.cuh"

namespace mxb {

constexpr int kEwThreads = 256;

static inline int ew_grid(int64_t work_items) {
  int64_t b = (work_items + kEwThreads - 1) / kEwThreads;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (b > cap) b = cap;
  return (int)(b < 1 ? 1 : b);
}

__device__ __forceinline__ uint32_t ew_hash(uint32_t seed, uint32_t idx) {
  uint32_t x = idx * 0x9E3779B1u ^ seed;
  x ^= x >> 16; x *= 0x85EBCA6Bu; x ^= x >> 13; x *= 0xC2B2AE35u; x ^= x >> 16;
  return x;
}

__device__ __forceinline__ float gelu_f(float x) { return 0.5f * x * (1.f + erf_fast(x * 0.70710678118654752f)); }
__device__ __forceinline__ float gelu_grad_f(float x) {
  const float cdf = 0.5f * (1.f + erf_fast(x * 0.70710678118654752f));
  const float pdf = 0.3989422804014327f * __expf(-0.5f * x * x);
  return cdf + x * pdf;
}

// y = gelu(x + bias[col]),  n elements, C columns (bias may be null).  Vector path: n, C multiples of Vec16<T>::N.
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
gelu_fwd_kernel(const T* __restrict__ x, const T* __restrict__ bias, T* __restrict__ y, int64_t n, int C) {
  constexpr int V = Vec16<T>::N;
  const int64_t nvec = n / V;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    Vec16<T> a = ld16(x + i * V);
    if (bias) {
      const Vec16<T> b = ld16(bias + (i * V) % C);
#pragma unroll
      for (int j = 0; j < V; ++j) a.v[j] = Cvt<T>::from_f(gelu_f(Cvt<T>::to_f(a.v[j]) + Cvt<T>::to_f(b.v[j])));
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) a.v[j] = Cvt<T>::from_f(gelu_f(Cvt<T>::to_f(a.v[j])));
    }
    st16(y + i * V, a);
  }
}

// dx = dy * gelu'(x + bias[col])
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
gelu_bwd_kernel(const T* __restrict__ x, const T* __restrict__ bias, const T* __restrict__ dy, T* __restrict__ dx, int64_t n,
                int C) {
  constexpr int V = Vec16<T>::N;
  const int64_t nvec = n / V;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    const Vec16<T> a = ld16(x + i * V), g = ld16(dy + i * V);
    Vec16<T> b, o;
    if (bias) b = ld16(bias + (i * V) % C);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float v = Cvt<T>::to_f(a.v[j]) + (bias ? Cvt<T>::to_f(b.v[j]) : 0.f);
      o.v[j] = Cvt<T>::from_f(Cvt<T>::to_f(g.v[j]) * gelu_grad_f(v));
    }
    st16(dx + i * V, o);
  }
}

// y = res + keep(i) * scale * (x + bias[col])        (res, bias optional; threshold 0 keeps everything)
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
dropout_fwd_kernel(const T* __restrict__ x, const T* __restrict__ bias, const T* __restrict__ res, T* __restrict__ y, int64_t n,
                   int C, uint32_t threshold, float scale, const uint32_t* __restrict__ seed_ptr) {
  constexpr int V = Vec16<T>::N;
  const int64_t nvec = n / V;
  const uint32_t seed = threshold ? *seed_ptr : 0u;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    const Vec16<T> a = ld16(x + i * V);
    Vec16<T> b, r, o;
    if (bias) b = ld16(bias + (i * V) % C);
    if (res) r = ld16(res + i * V);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      float v = Cvt<T>::to_f(a.v[j]) + (bias ? Cvt<T>::to_f(b.v[j]) : 0.f);
      const bool keep = !threshold || ew_hash(seed, (uint32_t)(i * V + j)) >= threshold;
      v = keep ? v * scale : 0.f;
      if (res) v += Cvt<T>::to_f(r.v[j]);
      o.v[j] = Cvt<T>::from_f(v);
    }
    st16(y + i * V, o);
  }
}

// dx = keep(i) * scale * dy   (the gradient of the residual input is dy itself)
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
dropout_bwd_kernel(const T* __restrict__ dy, T* __restrict__ dx, int64_t n, uint32_t threshold, float scale,
                   const uint32_t* __restrict__ seed_ptr) {
  constexpr int V = Vec16<T>::N;
  const int64_t nvec = n / V;
  const uint32_t seed = threshold ? *seed_ptr : 0u;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    const Vec16<T> g = ld16(dy + i * V);
    Vec16<T> o;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const bool keep = !threshold || ew_hash(seed, (uint32_t)(i * V + j)) >= threshold;
      o.v[j] = Cvt<T>::from_f(keep ? Cvt<T>::to_f(g.v[j]) * scale : 0.f);
    }
    st16(dx + i * V, o);
  }
}

constexpr int kAddNMax = 8;
struct AddNArgs {
  const void* in[kAddNMax];
  int count;
};

// y = in[0] + ... + in[count-1], accumulated in fp32
template <typename T>
__global__ void __launch_bounds__(kEwThreads) add_n_kernel(const AddNArgs a, T* __restrict__ y, int64_t n) {
  constexpr int V = Vec16<T>::N;
  const int64_t nvec = n / V;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
    for (int k = 0; k < a.count; ++k) {
      const Vec16<T> v = ld16(reinterpret_cast<const T*>(a.in[k]) + i * V);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += Cvt<T>::to_f(v.v[j]);
    }
    Vec16<T> o;
#pragma unroll
    for (int j = 0; j < V; ++j) o.v[j] = Cvt<T>::from_f(acc[j]);
    st16(y + i * V, o);
  }
}

// dst = (D)src, 8 elements per thread
template <typename S, typename D>
__global__ void __launch_bounds__(kEwThreads) cast_kernel(const S* __restrict__ src, D* __restrict__ dst, int64_t n) {
  const int64_t n8 = n / 8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    alignas(16) S in[8];
    alignas(16) D out[8];
    if (sizeof(S) == 4) {
      *reinterpret_cast<uint4*>(&in[0]) = *reinterpret_cast<const uint4*>(src + i * 8);
      *reinterpret_cast<uint4*>(&in[4]) = *reinterpret_cast<const uint4*>(src + i * 8 + 4);
    } else {
      *reinterpret_cast<uint4*>(&in[0]) = *reinterpret_cast<const uint4*>(src + i * 8);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = Cvt<D>::from_f(Cvt<S>::to_f(in[j]));
    if (sizeof(D) == 4) {
      *reinterpret_cast<uint4*>(dst + i * 8) = *reinterpret_cast<const uint4*>(&out[0]);
      *reinterpret_cast<uint4*>(dst + i * 8 + 4) = *reinterpret_cast<const uint4*>(&out[4]);
    } else {
      *reinterpret_cast<uint4*>(dst + i * 8) = *reinterpret_cast<const uint4*>(&out[0]);
    }
  }
  // tail
  const int64_t base = n8 * 8;
  for (int64_t i = base + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    dst[i] = Cvt<D>::from_f(Cvt<S>::to_f(src[i]));
}


// ---------------------------------------------------------------------------------------------- embedding
// out[i, :] = weight[idx[i], :]; one warp-sized group of threads per row, 16-byte vectors.  Indices are clipped to
// [0, rows) like the reference's take(mode='clip').
template <typename T, typename I>
__global__ void __launch_bounds__(kEwThreads)
embedding_fwd_kernel(const I* __restrict__ idx, const T* __restrict__ weight, T* __restrict__ out, int64_t n, int D, int64_t rows) {
  constexpr int V = Vec16<T>::N;
  const int L = D / V;
  const int64_t total = n * L;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / L;
    const int c = (int)(i % L);
    int64_t k = (int64_t)idx[r];
    k = k < 0 ? 0 : (k >= rows ? rows - 1 : k);
    st16(out + r * D + c * V, ld16(weight + k * D + c * V));
  }
}

// Gradient of the gather: `sorted` holds the indices in ascending order and `perm` the position each came from.
// Stage 1: one warp per block of 32 sorted positions sums the rows of dy run by run (fp32, in order).  A run that lies
// inside its block is written to dw directly; a run that crosses a block boundary leaves a partial sum ([block][0] when
// it continues from the previous block, [block][1] when it starts here and continues into the next).  Stage 2: one warp
// per run that starts in one block and continues adds its partials block by block.  The order of additions is fixed by
// the sorted order, so the result does not depend on scheduling, and a table with a few distinct indices (a run of
// thousands of positions) is still spread over all warps.
constexpr int kEmbBlock = 32;

template <typename T, typename I>
__global__ void __launch_bounds__(kEwThreads)
embedding_bwd_stage1_kernel(const I* __restrict__ sorted, const int64_t* __restrict__ perm, const T* __restrict__ dy,
                            T* __restrict__ dw, float* __restrict__ partial, int64_t n, int D, int64_t rows, int accumulate) {
  constexpr int V = Vec16<T>::N;
  const int L = D / V;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t nblocks = (n + kEmbBlock - 1) / kEmbBlock;
  for (int64_t b = (int64_t)blockIdx.x * (kEwThreads / 32) + warp; b < nblocks; b += (int64_t)gridDim.x * (kEwThreads / 32)) {
    const int64_t p0 = b * kEmbBlock, p1 = (p0 + kEmbBlock < n) ? p0 + kEmbBlock : n;
    for (int c = lane; c < L; c += 32) {
      float acc[V];
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = 0.f;
      int64_t cur = (int64_t)sorted[p0], seg = p0;
      for (int64_t p = p0; p <= p1; ++p) {
        const bool end = p == p1;
        const int64_t k = end ? -1 : (int64_t)sorted[p];
        if (end || k != cur) {
          // flush the run [seg, p) of index `cur`
          const bool from_prev = seg == p0 && p0 > 0 && (int64_t)sorted[p0 - 1] == cur;
          const bool into_next = end && p1 < n && (int64_t)sorted[p1] == cur;
          if (!from_prev && !into_next) {
            int64_t kk = cur < 0 ? 0 : (cur >= rows ? rows - 1 : cur);
            if (accumulate) {
              const Vec16<T> w = ld16(dw + kk * D + c * V);
#pragma unroll
              for (int j = 0; j < V; ++j) acc[j] += Cvt<T>::to_f(w.v[j]);
            }
            Vec16<T> o;
#pragma unroll
            for (int j = 0; j < V; ++j) o.v[j] = Cvt<T>::from_f(acc[j]);
            st16(dw + kk * D + c * V, o);
          } else {
            float* dst = partial + ((b * 2 + (from_prev ? 0 : 1)) * (int64_t)D) + c * V;
#pragma unroll
            for (int j = 0; j < V; ++j) dst[j] = acc[j];
          }
#pragma unroll
          for (int j = 0; j < V; ++j) acc[j] = 0.f;
          cur = k;
          seg = p;
        }
        if (!end) {
          const Vec16<T> g = ld16(dy + perm[p] * D + c * V);
#pragma unroll
          for (int j = 0; j < V; ++j) acc[j] += Cvt<T>::to_f(g.v[j]);
        }
      }
    }
  }
}

template <typename T, typename I>
__global__ void __launch_bounds__(kEwThreads)
embedding_bwd_stage2_kernel(const I* __restrict__ sorted, const float* __restrict__ partial, T* __restrict__ dw, int64_t n,
                            int D, int64_t rows, int accumulate) {
  constexpr int V = Vec16<T>::N;
  const int L = D / V;
  const int groups = (L + 31) / 32;              // a warp handles 32 vectors of one run: `groups` warps per block
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t nblocks = (n + kEmbBlock - 1) / kEmbBlock;
  const int64_t items = nblocks * groups;
  for (int64_t it = (int64_t)blockIdx.x * (kEwThreads / 32) + warp; it < items; it += (int64_t)gridDim.x * (kEwThreads / 32)) {
    const int64_t b = it / groups;
    const int c = (int)(it % groups) * 32 + lane;
    const int64_t p0 = b * kEmbBlock, p1 = p0 + kEmbBlock;
    if (p1 >= n) continue;
    const int64_t k = (int64_t)sorted[p1 - 1];
    if ((int64_t)sorted[p1] != k) continue;                        // the last run of this block ends here
    // does that run start in this block?  (otherwise an earlier block owns it)
    if ((int64_t)sorted[p0] == k && p0 > 0 && (int64_t)sorted[p0 - 1] == k) continue;
    int64_t b_end = b + 1;                                           // blocks b+1 .. b_end-1 begin with this run
    while (b_end < nblocks && (int64_t)sorted[b_end * kEmbBlock] == k) ++b_end;
    if (c >= L) continue;
    const int64_t kk = k < 0 ? 0 : (k >= rows ? rows - 1 : k);
    float acc[V];
    const float* src = partial + (b * 2 + 1) * (int64_t)D + c * V;
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = src[j];
    // the following blocks' partials: independent loads, added in block order
    int64_t b2 = b + 1;
    for (; b2 + 3 < b_end; b2 += 4) {
      float t[4][V];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float* s2 = partial + ((b2 + u) * 2) * (int64_t)D + c * V;
#pragma unroll
        for (int j = 0; j < V; ++j) t[u][j] = s2[j];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] += t[u][j];
    }
    for (; b2 < b_end; ++b2) {
      const float* s2 = partial + (b2 * 2) * (int64_t)D + c * V;
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += s2[j];
    }
    if (accumulate) {
      const Vec16<T> w = ld16(dw + kk * D + c * V);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += Cvt<T>::to_f(w.v[j]);
    }
    Vec16<T> o;
#pragma unroll
    for (int j = 0; j < V; ++j) o.v[j] = Cvt<T>::from_f(acc[j]);
    st16(dw + kk * D + c * V, o);
  }
}

// ---------------------------------------------------------------------------------------------- average pooling
struct AvgPoolShape {
  int N, H, W, C, Ho, Wo, kh, kw, sh, sw, ph, pw, count_include_pad;
};

// NHWC average pooling; one thread per 16-byte channel vector of one output pixel.
template <typename T>
__global__ void __launch_bounds__(kEwThreads) avgpool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, const AvgPoolShape p) {
  constexpr int V = Vec16<T>::N;
  const int L = p.C / V;
  const int64_t nvec = (int64_t)p.N * p.Ho * p.Wo * L;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    const int cv = (int)(i % L);
    int64_t t = i / L;
    const int ow = (int)(t % p.Wo); t /= p.Wo;
    const int oh = (int)(t % p.Ho);
    const int n = (int)(t / p.Ho);
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
    int cnt = 0;
    for (int r = 0; r < p.kh; ++r) {
      const int ih = oh * p.sh - p.ph + r;
      for (int s = 0; s < p.kw; ++s) {
        const int iw = ow * p.sw - p.pw + s;
        const bool inside = ih >= 0 && ih < p.H && iw >= 0 && iw < p.W;
        // a padded position counts towards the divisor only with count_include_pad and only inside the padded extent
        if (inside || (p.count_include_pad && ih < p.H + p.ph && iw < p.W + p.pw)) ++cnt;
        if (!inside) continue;
        const Vec16<T> v = ld16(x + (((int64_t)n * p.H + ih) * p.W + iw) * p.C + cv * V);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] += Cvt<T>::to_f(v.v[j]);
      }
    }
    const float inv = cnt > 0 ? 1.f / (float)cnt : 0.f;
    Vec16<T> o;
#pragma unroll
    for (int j = 0; j < V; ++j) o.v[j] = Cvt<T>::from_f(acc[j] * inv);
    st16(y + i * V, o);
  }
}

// Gradient: gather over the windows that cover an input pixel (no atomics).
template <typename T>
__global__ void __launch_bounds__(kEwThreads) avgpool_bwd_kernel(const T* __restrict__ dy, T* __restrict__ dx, const AvgPoolShape p) {
  constexpr int V = Vec16<T>::N;
  const int L = p.C / V;
  const int64_t nvec = (int64_t)p.N * p.H * p.W * L;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    const int cv = (int)(i % L);
    int64_t t = i / L;
    const int iw = (int)(t % p.W); t /= p.W;
    const int ih = (int)(t % p.H);
    const int n = (int)(t / p.H);
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
    int oh0 = ih + p.ph - p.kh + 1;
    oh0 = oh0 <= 0 ? 0 : (oh0 + p.sh - 1) / p.sh;
    int oh1 = (ih + p.ph) / p.sh;
    if (oh1 > p.Ho - 1) oh1 = p.Ho - 1;
    int ow0 = iw + p.pw - p.kw + 1;
    ow0 = ow0 <= 0 ? 0 : (ow0 + p.sw - 1) / p.sw;
    int ow1 = (iw + p.pw) / p.sw;
    if (ow1 > p.Wo - 1) ow1 = p.Wo - 1;
    for (int oh = oh0; oh <= oh1; ++oh) {
      for (int ow = ow0; ow <= ow1; ++ow) {
        int cnt = 0;
        for (int r = 0; r < p.kh; ++r) {
          const int h2 = oh * p.sh - p.ph + r;
          for (int s = 0; s < p.kw; ++s) {
            const int w2 = ow * p.sw - p.pw + s;
            const bool inside = h2 >= 0 && h2 < p.H && w2 >= 0 && w2 < p.W;
            if (inside || (p.count_include_pad && h2 < p.H + p.ph && w2 < p.W + p.pw)) ++cnt;
          }
        }
        const float inv = cnt > 0 ? 1.f / (float)cnt : 0.f;
        const Vec16<T> g = ld16(dy + (((int64_t)n * p.Ho + oh) * p.Wo + ow) * p.C + cv * V);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] += Cvt<T>::to_f(g.v[j]) * inv;
      }
    }
    Vec16<T> o;
#pragma unroll
    for (int j = 0; j < V; ++j) o.v[j] = Cvt<T>::from_f(acc[j]);
    st16(dx + i * V, o);
  }
}

// ---------------------------------------------------------------------------------------------- column sums
// out[c] = sum over rows of x[r, c] (the bias gradient of a FullyConnected layer; the reference's two-phase
// AddBiasGradKernelPhase1/2, src/operator/nn/fully_connected-inl.h).  Stage 1: CTA (bx, by) sums a chunk of rows for 32
// vector columns (8 row lanes x 32 column lanes, 16-byte loads, fp32 accumulation) into partial[by][c]; stage 2 adds the
// partials in order.  Deterministic.
constexpr int kColRowsLanes = 8;

template <typename T>
__global__ void __launch_bounds__(256)
colsum_stage1_kernel(const T* __restrict__ x, float* __restrict__ partial, int64_t rows, int C, int64_t rows_per_cta) {
  constexpr int V = Vec16<T>::N;
  __shared__ float red[kColRowsLanes][32][V + 1];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int L = C / V;
  const int cv = blockIdx.x * 32 + tx;
  const int64_t r0 = (int64_t)blockIdx.y * rows_per_cta, r1 = (r0 + rows_per_cta < rows) ? r0 + rows_per_cta : rows;
  float acc[V];
#pragma unroll
  for (int j = 0; j < V; ++j) acc[j] = 0.f;
  if (cv < L) {
    for (int64_t r = r0 + ty; r < r1; r += kColRowsLanes) {
      const Vec16<T> a = ld16(x + r * C + cv * V);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += Cvt<T>::to_f(a.v[j]);
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j) red[ty][tx][j] = acc[j];
  __syncthreads();
  if (ty == 0 && cv < L) {
#pragma unroll
    for (int j = 0; j < V; ++j) {
      float t = 0.f;
#pragma unroll
      for (int k = 0; k < kColRowsLanes; ++k) t += red[k][tx][j];
      partial[(int64_t)blockIdx.y * C + cv * V + j] = t;
    }
  }
}

__global__ void __launch_bounds__(256) colsum_stage2_kernel(const float* __restrict__ partial, float* __restrict__ out, int C, int ny) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float t = 0.f;
  for (int k = 0; k < ny; ++k) t += partial[(int64_t)k * C + c];
  out[c] = t;
}

// ---------------------------------------------------------------------------------------------- transpose
// out[b, c, r] = in[b, r, c] through a padded 32x32 shared-memory tile (coalesced on both sides).
template <typename T>
__global__ void __launch_bounds__(256) transpose_kernel(const T* __restrict__ in, T* __restrict__ out, int R, int C) {
  __shared__ T tile[32][33];
  const int64_t base = (int64_t)blockIdx.z * R * C;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int r = r0 + j, c = c0 + threadIdx.x;
    if (r < R && c < C) tile[j][threadIdx.x] = in[base + (int64_t)r * C + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int c = c0 + j, r = r0 + threadIdx.x;
    if (r < R && c < C) out[base + (int64_t)c * R + r] = tile[threadIdx.x][j];
  }
}

}  // namespace mxb

using namespace mxb;

#define MXB_DISPATCH_FLOAT(dtype, ...)                                   \
  [&]() -> int {                                                         \
    if (dtype == kF32) { using T = float; __VA_ARGS__ }                  \
    if (dtype == kF16) { using T = __half; __VA_ARGS__ }                 \
    if (dtype == kBF16) { using T = __nv_bfloat16; __VA_ARGS__ }         \
    return -1;                                                           \
  }()

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
static inline int vec_of(int dtype) { return dtype == kF32 ? 4 : 8; }

// y = gelu(x + bias[col]); n elements in rows of C (bias may be null).  n and C multiples of 16 bytes worth of elements.
MXB_EXPORT int mxb_gelu_forward(int dtype, const void* x, const void* bias, void* y, int64_t n, int C, void* stream) {
  if (n < 1 || C < 1 || n % vec_of(dtype) || C % vec_of(dtype) || !aligned16(x) || !aligned16(y) || !aligned16(bias)) return -3;
  cudaStream_t st = (cudaStream_t)stream;
  return MXB_DISPATCH_FLOAT(dtype, {
    gelu_fwd_kernel<T><<<ew_grid(n / Vec16<T>::N), kEwThreads, 0, st>>>((const T*)x, (const T*)bias, (T*)y, n, C);
    return (int)cudaGetLastError();
  });
}

MXB_EXPORT int mxb_gelu_backward(int dtype, const void* x, const void* bias, const void* dy, void* dx, int64_t n, int C,
                                 void* stream) {
  if (n < 1 || C < 1 || n % vec_of(dtype) || C % vec_of(dtype) || !aligned16(x) || !aligned16(dy) || !aligned16(dx) ||
      !aligned16(bias))
    return -3;
  cudaStream_t st = (cudaStream_t)stream;
  return MXB_DISPATCH_FLOAT(dtype, {
    gelu_bwd_kernel<T><<<ew_grid(n / Vec16<T>::N), kEwThreads, 0, st>>>((const T*)x, (const T*)bias, (const T*)dy, (T*)dx, n, C);
    return (int)cudaGetLastError();
  });
}

static inline uint32_t drop_threshold(float p) {
  const double t = (double)p * 4294967296.0;
  return t >= 4294967295.0 ? 4294967295u : (uint32_t)t;
}

// y = res + dropout(x + bias[col], p); bias, res optional; `seed` is a device word (required when p > 0).
MXB_EXPORT int mxb_dropout_forward(int dtype, const void* x, const void* bias, const void* res, void* y, int64_t n, int C,
                                   float p, const uint32_t* seed, void* stream) {
  if (n < 1 || C < 1 || n % vec_of(dtype) || C % vec_of(dtype) || p < 0.f || p >= 1.f || (p > 0.f && !seed)) return -3;
  if (!aligned16(x) || !aligned16(y) || !aligned16(bias) || !aligned16(res) || n > 0xffffffffLL) return -3;
  cudaStream_t st = (cudaStream_t)stream;
  const uint32_t thr = p > 0.f ? drop_threshold(p) : 0u;
  const float scale = 1.f / (1.f - p);
  return MXB_DISPATCH_FLOAT(dtype, {
    dropout_fwd_kernel<T><<<ew_grid(n / Vec16<T>::N), kEwThreads, 0, st>>>((const T*)x, (const T*)bias, (const T*)res, (T*)y, n, C,
                                                                         thr, scale, seed);
    return (int)cudaGetLastError();
  });
}

MXB_EXPORT int mxb_dropout_backward(int dtype, const void* dy, void* dx, int64_t n, float p, const uint32_t* seed, void* stream) {
  if (n < 1 || n % vec_of(dtype) || p < 0.f || p >= 1.f || (p > 0.f && !seed) || !aligned16(dy) || !aligned16(dx) ||
      n > 0xffffffffLL)
    return -3;
  cudaStream_t st = (cudaStream_t)stream;
  const uint32_t thr = p > 0.f ? drop_threshold(p) : 0u;
  const float scale = 1.f / (1.f - p);
  return MXB_DISPATCH_FLOAT(dtype, {
    dropout_bwd_kernel<T><<<ew_grid(n / Vec16<T>::N), kEwThreads, 0, st>>>((const T*)dy, (T*)dx, n, thr, scale, seed);
    return (int)cudaGetLastError();
  });
}

MXB_EXPORT int mxb_add_n_max() { return kAddNMax; }

// y = sum of `count` tensors (1..mxb_add_n_max()) of n elements each; y may alias in[0].
MXB_EXPORT int mxb_add_n(int dtype, const void* const* in, int count, void* y, int64_t n, void* stream) {
  if (count < 1 || count > kAddNMax || n < 1 || n % vec_of(dtype) || !aligned16(y)) return -3;
  AddNArgs a;
  a.count = count;
  for (int k = 0; k < count; ++k) {
    if (!in[k] || !aligned16(in[k])) return -3;
    a.in[k] = in[k];
  }
  cudaStream_t st = (cudaStream_t)stream;
  return MXB_DISPATCH_FLOAT(dtype, {
    add_n_kernel<T><<<ew_grid(n / Vec16<T>::N), kEwThreads, 0, st>>>(a, (T*)y, n);
    return (int)cudaGetLastError();
  });
}

// dst[i] = (dst type) src[i] between fp32, fp16 and bf16.
MXB_EXPORT int mxb_cast(int src_dtype, int dst_dtype, const void* src, void* dst, int64_t n, void* stream) {
  if (n < 1 || !aligned16(src) || !aligned16(dst)) return -3;
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = ew_grid((n + 7) / 8);
#define MXB_CAST(S, D) \
  { cast_kernel<S, D><<<grid, kEwThreads, 0, st>>>((const S*)src, (D*)dst, n); return (int)cudaGetLastError(); }
  if (src_dtype == kF32 && dst_dtype == kF16) MXB_CAST(float, __half)
  if (src_dtype == kF32 && dst_dtype == kBF16) MXB_CAST(float, __nv_bfloat16)
  if (src_dtype == kF16 && dst_dtype == kF32) MXB_CAST(__half, float)
  if (src_dtype == kBF16 && dst_dtype == kF32) MXB_CAST(__nv_bfloat16, float)
  if (src_dtype == kF16 && dst_dtype == kBF16) MXB_CAST(__half, __nv_bfloat16)
  if (src_dtype == kBF16 && dst_dtype == kF16) MXB_CAST(__nv_bfloat16, __half)
#undef MXB_CAST
  return -1;
}

// out[n, D] = weight[idx[i], :]; idx_is_64: indices are int64 (else int32).  D a multiple of 16 bytes worth of elements.
MXB_EXPORT int mxb_embedding_forward(int dtype, const void* idx, int idx_is_64, const void* weight, void* out, int64_t n, int D,
                                     int64_t rows, void* stream) {
  if (n < 1 || D < 1 || rows < 1 || D % vec_of(dtype) || !aligned16(weight) || !aligned16(out)) return -3;
  cudaStream_t st = (cudaStream_t)stream;
  return MXB_DISPATCH_FLOAT(dtype, {
    const int grid = ew_grid(n * (D / Vec16<T>::N));
    if (idx_is_64) embedding_fwd_kernel<T, int64_t><<<grid, kEwThreads, 0, st>>>((const int64_t*)idx, (const T*)weight, (T*)out, n, D, rows);
    else embedding_fwd_kernel<T, int32_t><<<grid, kEwThreads, 0, st>>>((const int32_t*)idx, (const T*)weight, (T*)out, n, D, rows);
    return (int)cudaGetLastError();
  });
}

// dw[rows, D] (+)= scatter of dy[n, D] by the indices; `sorted` ascending with `perm` (int64) the original positions;
// `partial`: ceil(n / 32) * 2 * D floats of scratch.
MXB_EXPORT int mxb_embedding_backward(int dtype, const void* sorted, int idx_is_64, const int64_t* perm, const void* dy, void* dw,
                                      float* partial, int64_t n, int D, int64_t rows, int accumulate, void* stream) {
  if (n < 1 || D < 1 || rows < 1 || D % vec_of(dtype) || !aligned16(dy) || !aligned16(dw) || !partial || !aligned16(partial))
    return -3;
  cudaStream_t st = (cudaStream_t)stream;
  return MXB_DISPATCH_FLOAT(dtype, {
    const int64_t nblocks = (n + kEmbBlock - 1) / kEmbBlock;
    const int grid = ew_grid(nblocks * 32);
    const int grid2 = ew_grid(nblocks * 32 * ((D / Vec16<T>::N + 31) / 32));
    if (idx_is_64) {
      embedding_bwd_stage1_kernel<T, int64_t><<<grid, kEwThreads, 0, st>>>((const int64_t*)sorted, perm, (const T*)dy, (T*)dw, partial, n, D, rows, accumulate);
      embedding_bwd_stage2_kernel<T, int64_t><<<grid2, kEwThreads, 0, st>>>((const int64_t*)sorted, partial, (T*)dw, n, D, rows, accumulate);
    } else {
      embedding_bwd_stage1_kernel<T, int32_t><<<grid, kEwThreads, 0, st>>>((const int32_t*)sorted, perm, (const T*)dy, (T*)dw, partial, n, D, rows, accumulate);
      embedding_bwd_stage2_kernel<T, int32_t><<<grid2, kEwThreads, 0, st>>>((const int32_t*)sorted, partial, (T*)dw, n, D, rows, accumulate);
    }
    return (int)cudaGetLastError();
  });
}

static int fill_avg(AvgPoolShape* p, int N, int H, int W, int C, int Ho, int Wo, int kh, int kw, int sh, int sw, int ph, int pw,
                    int count_include_pad, int dtype) {
  if (N < 1 || H < 1 || W < 1 || C < 1 || Ho < 1 || Wo < 1 || kh < 1 || kw < 1 || sh < 1 || sw < 1 || ph < 0 || pw < 0) return -2;
  if (C % vec_of(dtype)) return -3;
  *p = AvgPoolShape{N, H, W, C, Ho, Wo, kh, kw, sh, sw, ph, pw, count_include_pad};
  return 0;
}

// NHWC average pooling (a global pool is kernel = input extent, stride 1, no padding).
MXB_EXPORT int mxb_avgpool_forward(int dtype, const void* x, void* y, int N, int H, int W, int C, int Ho, int Wo, int kh, int kw,
                                   int sh, int sw, int ph, int pw, int count_include_pad, void* stream) {
  AvgPoolShape p;
  int rc = fill_avg(&p, N, H, W, C, Ho, Wo, kh, kw, sh, sw, ph, pw, count_include_pad, dtype);
  if (rc) return rc;
  if (!aligned16(x) || !aligned16(y)) return -3;
  cudaStream_t st = (cudaStream_t)stream;
  return MXB_DISPATCH_FLOAT(dtype, {
    avgpool_fwd_kernel<T><<<ew_grid((int64_t)N * Ho * Wo * (C / Vec16<T>::N)), kEwThreads, 0, st>>>((const T*)x, (T*)y, p);
    return (int)cudaGetLastError();
  });
}

MXB_EXPORT int mxb_avgpool_backward(int dtype, const void* dy, void* dx, int N, int H, int W, int C, int Ho, int Wo, int kh, int kw,
                                    int sh, int sw, int ph, int pw, int count_include_pad, void* stream) {
  AvgPoolShape p;
  int rc = fill_avg(&p, N, H, W, C, Ho, Wo, kh, kw, sh, sw, ph, pw, count_include_pad, dtype);
  if (rc) return rc;
  if (!aligned16(dy) || !aligned16(dx)) return -3;
  cudaStream_t st = (cudaStream_t)stream;
  return MXB_DISPATCH_FLOAT(dtype, {
    avgpool_bwd_kernel<T><<<ew_grid((int64_t)N * H * W * (C / Vec16<T>::N)), kEwThreads, 0, st>>>((const T*)dy, (T*)dx, p);
    return (int)cudaGetLastError();
  });
}

// out[b, c, r] = in[b, r, c] for `batch` matrices of R x C elements of `elem_bytes` (2 or 4) each.
MXB_EXPORT int mxb_transpose(int elem_bytes, const void* in, void* out, int batch, int R, int C, void* stream) {
  if (batch < 1 || R < 1 || C < 1 || batch > 65535 || (R + 31) / 32 > 65535) return -2;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((C + 31) / 32, (R + 31) / 32, batch), block(32, 8);
  if (elem_bytes == 2) transpose_kernel<uint16_t><<<grid, block, 0, st>>>((const uint16_t*)in, (uint16_t*)out, R, C);
  else if (elem_bytes == 4) transpose_kernel<uint32_t><<<grid, block, 0, st>>>((const uint32_t*)in, (uint32_t*)out, R, C);
  else return -1;
  return (int)cudaGetLastError();
}

// Row chunks used by mxb_colsum for (rows, C): the partial buffer holds that many rows of C floats.
MXB_EXPORT int mxb_colsum_chunks(int dtype, int64_t rows, int C) {
  const int L = C / vec_of(dtype);
  const int nx = (L + 31) / 32;
  int64_t ny = ((int64_t)sm_count() * 4 + nx - 1) / nx;
  if (ny > (rows + 63) / 64) ny = (rows + 63) / 64;          // at least 64 rows per chunk
  return (int)(ny < 1 ? 1 : ny);
}

// out[C] (fp32) = column sums of x[rows, C]; partial: mxb_colsum_chunks(...) * C floats.
MXB_EXPORT int mxb_colsum(int dtype, const void* x, float* partial, float* out, int64_t rows, int C, void* stream) {
  if (rows < 1 || C < 1 || C % vec_of(dtype) || !aligned16(x) || !partial || !out) return -3;
  cudaStream_t st = (cudaStream_t)stream;
  const int ny = mxb_colsum_chunks(dtype, rows, C);
  const int64_t per = (rows + ny - 1) / ny;
  return MXB_DISPATCH_FLOAT(dtype, {
    const int L = C / Vec16<T>::N;
    dim3 grid((L + 31) / 32, ny);
    colsum_stage1_kernel<T><<<grid, 256, 0, st>>>((const T*)x, partial, rows, C, per);
    colsum_stage2_kernel<<<(C + 255) / 256, 256, 0, st>>>(partial, out, C, ny);
    return (int)cudaGetLastError();
  });
}

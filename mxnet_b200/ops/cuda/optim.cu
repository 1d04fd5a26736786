// Multi-tensor optimizer and reduction kernels for sm_100a.
//
// Reference behaviour: MultiSGDKernel (src/operator/optimizer_op-inl.h:201-250, at most 60 tensors
// per launch), multi_all_finite (src/operator/all_finite.cu), multi_sum_sq
// (src/operator/contrib/multi_sum_sq.cu).  The tensor table travels as a kernel argument (no
// per-call host-to-device table copy, so launches are CUDA-graph capturable); work is split into
// fixed-size chunks and every CTA walks chunks with a grid-stride loop, finding the owning tensor by
// binary search over the chunk prefix sums.
#include "common.cuh"

namespace mxb {

constexpr int kMaxTensors = 48;
constexpr int kChunk = 8192;          // elements per chunk

struct TensorTable {
  void* w[kMaxTensors];               // weights (out)
  const void* g[kMaxTensors];         // gradients
  float* m[kMaxTensors];              // momentum (or null)
  float* w32[kMaxTensors];            // fp32 master weights (or null)
  float lr[kMaxTensors];
  float wd[kMaxTensors];
  int64_t n[kMaxTensors];
  int chunk_start[kMaxTensors + 1];   // prefix sums of chunk counts
  int count;
};

__device__ __forceinline__ int find_tensor(const int* chunk_start, int count, int chunk) {
  int lo = 0, hi = count - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (chunk_start[mid] <= chunk) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// T: storage type of weights/gradients; master weights and momentum are fp32.
template <typename T, bool kMom, bool kMP>
__global__ void __launch_bounds__(256)
multi_sgd_kernel(const __grid_constant__ TensorTable tab, float momentum, float rescale, float clip) {
  const int total = tab.chunk_start[tab.count];
  for (int chunk = blockIdx.x; chunk < total; chunk += gridDim.x) {
    const int t = find_tensor(tab.chunk_start, tab.count, chunk);
    const int64_t base = (int64_t)(chunk - tab.chunk_start[t]) * kChunk;
    const int64_t n = tab.n[t];
    T* w = (T*)tab.w[t];
    const T* g = (const T*)tab.g[t];
    float* m = tab.m[t];
    float* w32 = tab.w32[t];
    const float lr = tab.lr[t], wd = tab.wd[t];
    for (int64_t i = base + threadIdx.x; i < base + kChunk && i < n; i += blockDim.x) {
      float gr = Cvt<T>::to_f(g[i]) * rescale;
      if (clip >= 0.f) gr = fminf(fmaxf(gr, -clip), clip);
      float wv = kMP ? w32[i] : Cvt<T>::to_f(w[i]);
      gr += wd * wv;
      if (kMom) {
        float mv = momentum * m[i] - lr * gr;
        m[i] = mv;
        wv += mv;
      } else {
        wv -= lr * gr;
      }
      if (kMP) w32[i] = wv;
      w[i] = Cvt<T>::from_f(wv);
    }
  }
}

struct AdamTable {
  void* w[kMaxTensors];
  const void* g[kMaxTensors];
  float* mean[kMaxTensors];
  float* var[kMaxTensors];
  float* w32[kMaxTensors];            // fp32 master weights (or null)
  float lr[kMaxTensors];
  float wd[kMaxTensors];
  float eta[kMaxTensors];
  int64_t n[kMaxTensors];
  int chunk_start[kMaxTensors + 1];
  int count;
};

// Adam (kDecoupled = false: weight decay folded into the gradient, optimizer_op-inl.h AdamUpdate) and AdamW
// (kDecoupled = true: w -= eta * (lr * m / (sqrt(v) + eps) + wd * w), src/operator/contrib/adamw-inl.h) over a table of
// tensors.  `rescale_ptr` is a device float (the reference passes rescale_grad as a tensor so that the loss scaler never
// synchronises with the host): a zero or non-finite value skips the whole update.
template <typename T, bool kMP, bool kDecoupled>
__global__ void __launch_bounds__(256)
multi_adam_kernel(const __grid_constant__ AdamTable tab, float beta1, float beta2, float eps, float clip,
                  const float* __restrict__ rescale_ptr, float rescale_host) {
  const float rescale = rescale_ptr ? *rescale_ptr : rescale_host;
  if (!(fabsf(rescale) <= 3.0e38f) || rescale == 0.f) return;
  const int total = tab.chunk_start[tab.count];
  for (int chunk = blockIdx.x; chunk < total; chunk += gridDim.x) {
    const int t = find_tensor(tab.chunk_start, tab.count, chunk);
    const int64_t base = (int64_t)(chunk - tab.chunk_start[t]) * kChunk;
    const int64_t n = tab.n[t];
    T* w = (T*)tab.w[t];
    const T* g = (const T*)tab.g[t];
    float* mean = tab.mean[t];
    float* var = tab.var[t];
    float* w32 = tab.w32[t];
    const float lr = tab.lr[t], wd = tab.wd[t], eta = tab.eta[t];
    for (int64_t i = base + threadIdx.x; i < base + kChunk && i < n; i += blockDim.x) {
      float gr = Cvt<T>::to_f(g[i]) * rescale;
      if (clip >= 0.f) gr = fminf(fmaxf(gr, -clip), clip);
      float wv = kMP ? w32[i] : Cvt<T>::to_f(w[i]);
      if (!kDecoupled) gr += wd * wv;
      const float m = beta1 * mean[i] + (1.f - beta1) * gr;
      const float v = beta2 * var[i] + (1.f - beta2) * gr * gr;
      mean[i] = m;
      var[i] = v;
      const float step = lr * m / (sqrtf(v) + eps);
      wv -= kDecoupled ? eta * (step + wd * wv) : step;
      if (kMP) w32[i] = wv;
      w[i] = Cvt<T>::from_f(wv);
    }
  }
}

struct PtrTable {
  const void* p[kMaxTensors];
  int64_t n[kMaxTensors];
  int dtype[kMaxTensors];
  int chunk_start[kMaxTensors + 1];
  int count;
};

__device__ __forceinline__ float load_as_float(const void* p, int dtype, int64_t i) {
  if (dtype == kF32) return ((const float*)p)[i];
  if (dtype == kF16) return __half2float(((const __half*)p)[i]);
  return __bfloat162float(((const __nv_bfloat16*)p)[i]);
}

// out[0] is multiplied towards 0 when any element is inf/nan (caller initialises it to 1).
__global__ void __launch_bounds__(256) multi_all_finite_kernel(const __grid_constant__ PtrTable tab, float* out) {
  const int total = tab.chunk_start[tab.count];
  bool bad = false;
  for (int chunk = blockIdx.x; chunk < total; chunk += gridDim.x) {
    const int t = find_tensor(tab.chunk_start, tab.count, chunk);
    const int64_t base = (int64_t)(chunk - tab.chunk_start[t]) * kChunk;
    const int64_t n = tab.n[t];
    for (int64_t i = base + threadIdx.x; i < base + kChunk && i < n; i += blockDim.x) {
      float v = load_as_float(tab.p[t], tab.dtype[t], i);
      bad |= !isfinite(v);
    }
  }
  if (__syncthreads_or(bad) && threadIdx.x == 0) out[0] = 0.f;
}

// Stage 1 of sum of squares: one partial per (chunk); stage 2 sums the partials of each tensor in
// chunk order, so the result does not depend on the grid size.
__global__ void __launch_bounds__(256) multi_sum_sq_partial_kernel(const __grid_constant__ PtrTable tab, float* partial) {
  __shared__ float red[32];
  const int total = tab.chunk_start[tab.count];
  for (int chunk = blockIdx.x; chunk < total; chunk += gridDim.x) {
    const int t = find_tensor(tab.chunk_start, tab.count, chunk);
    const int64_t base = (int64_t)(chunk - tab.chunk_start[t]) * kChunk;
    const int64_t n = tab.n[t];
    float s = 0.f;
    for (int64_t i = base + threadIdx.x; i < base + kChunk && i < n; i += blockDim.x) {
      float v = load_as_float(tab.p[t], tab.dtype[t], i);
      s += v * v;
    }
    s = block_sum(s, red);
    if (threadIdx.x == 0) partial[chunk] = s;
  }
}

__global__ void multi_sum_sq_final_kernel(const __grid_constant__ PtrTable tab, const float* partial, float* out, int out_offset) {
  __shared__ float red[32];
  const int t = blockIdx.x;
  float s = 0.f;
  for (int c = tab.chunk_start[t] + threadIdx.x; c < tab.chunk_start[t + 1]; c += blockDim.x) s += partial[c];
  s = block_sum(s, red);
  if (threadIdx.x == 0) out[out_offset + t] = s;
}

__global__ void set_float_kernel(float* p, float v) { *p = v; }

inline int chunks_of(int64_t n) { return (int)((n + kChunk - 1) / kChunk); }

}  // namespace mxb

using namespace mxb;

// dst[t] += src[t] for up to kMaxTensors tensors of one dtype in one launch (16-byte vectors where both pointers allow
// it).  Used where many small accumulations follow each other: the parameter-gradient accumulation at the end of a
// captured backward pass (one tensor library launch per parameter otherwise).
struct AddTable {
  void* dst[kMaxTensors];
  const void* src[kMaxTensors];
  int64_t n[kMaxTensors];
  int chunk_start[kMaxTensors + 1];
  int count;
};

template <typename T>
__global__ void __launch_bounds__(256) multi_add_inplace_kernel(const __grid_constant__ AddTable tab) {
  constexpr int N = Vec16<T>::N;
  const int total = tab.chunk_start[tab.count];
  for (int chunk = blockIdx.x; chunk < total; chunk += gridDim.x) {
    const int t = find_tensor(tab.chunk_start, tab.count, chunk);
    const int64_t base = (int64_t)(chunk - tab.chunk_start[t]) * kChunk;
    const int64_t n = tab.n[t];
    const int64_t end = base + kChunk < n ? base + kChunk : n;
    T* d = (T*)tab.dst[t];
    const T* s = (const T*)tab.src[t];
    const bool vec = (((uintptr_t)d | (uintptr_t)s) & 15) == 0;      // chunk starts are multiples of 8192 elements
    int64_t i = base + (int64_t)threadIdx.x * N;
    if (vec) {
      for (; i + N <= end; i += (int64_t)blockDim.x * N) {
        Vec16<T> a = ld16(d + i);
        const Vec16<T> b = ld16(s + i);
#pragma unroll
        for (int j = 0; j < N; ++j) a.v[j] = Cvt<T>::from_f(Cvt<T>::to_f(a.v[j]) + Cvt<T>::to_f(b.v[j]));
        st16(d + i, a);
      }
      // the ragged tail of the last chunk: the first lanes past the last whole vector
      const int64_t tail = base + ((end - base) / N) * N;
      const int64_t k = tail + threadIdx.x;
      if (k < end) d[k] = Cvt<T>::from_f(Cvt<T>::to_f(d[k]) + Cvt<T>::to_f(s[k]));
    } else {
      for (int64_t k = base + threadIdx.x; k < end; k += blockDim.x) d[k] = Cvt<T>::from_f(Cvt<T>::to_f(d[k]) + Cvt<T>::to_f(s[k]));
    }
  }
}

MXB_EXPORT int mxb_max_tensors() { return kMaxTensors; }
MXB_EXPORT int mxb_chunk_elems() { return kChunk; }

MXB_EXPORT int mxb_multi_add_inplace(int dtype, int count, void** dst, void** src, const int64_t* sizes, void* stream) {
  if (count > kMaxTensors || count <= 0) return -2;
  AddTable tab;
  tab.count = count;
  int acc = 0;
  for (int i = 0; i < count; ++i) {
    if (sizes[i] < 0) return -2;
    tab.dst[i] = dst[i]; tab.src[i] = src[i]; tab.n[i] = sizes[i];
    tab.chunk_start[i] = acc;
    acc += chunks_of(sizes[i]);
  }
  tab.chunk_start[count] = acc;
  int grid = acc < sm_count() * 8 ? acc : sm_count() * 8;
  if (grid < 1) grid = 1;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == kF32) multi_add_inplace_kernel<float><<<grid, 256, 0, st>>>(tab);
  else if (dtype == kF16) multi_add_inplace_kernel<__half><<<grid, 256, 0, st>>>(tab);
  else if (dtype == kBF16) multi_add_inplace_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(tab);
  else return -1;
  return (int)cudaGetLastError();
}

// dtype: storage type of weights and gradients.  moms / w32 may be null arrays.
MXB_EXPORT int mxb_multi_sgd(int dtype, int count, void** w, void** g, float** m, float** w32, const float* lrs,
                             const float* wds, const int64_t* sizes, float momentum, float rescale, float clip,
                             void* stream) {
  if (count > kMaxTensors || count <= 0) return -2;
  TensorTable tab;
  tab.count = count;
  int acc = 0;
  for (int i = 0; i < count; ++i) {
    tab.w[i] = w[i]; tab.g[i] = g[i];
    tab.m[i] = m ? m[i] : nullptr;
    tab.w32[i] = w32 ? w32[i] : nullptr;
    tab.lr[i] = lrs[i]; tab.wd[i] = wds[i]; tab.n[i] = sizes[i];
    tab.chunk_start[i] = acc;
    acc += chunks_of(sizes[i]);
  }
  tab.chunk_start[count] = acc;
  int grid = acc < sm_count() * 8 ? acc : sm_count() * 8;
  if (grid < 1) grid = 1;
  cudaStream_t st = (cudaStream_t)stream;
  const bool mom = m != nullptr, mp = w32 != nullptr;
#define LAUNCH(T)                                                                                         \
  if (mom && mp) multi_sgd_kernel<T, true, true><<<grid, 256, 0, st>>>(tab, momentum, rescale, clip);        \
  else if (mom) multi_sgd_kernel<T, true, false><<<grid, 256, 0, st>>>(tab, momentum, rescale, clip);        \
  else if (mp) multi_sgd_kernel<T, false, true><<<grid, 256, 0, st>>>(tab, momentum, rescale, clip);         \
  else multi_sgd_kernel<T, false, false><<<grid, 256, 0, st>>>(tab, momentum, rescale, clip);
  if (dtype == kF32) { LAUNCH(float) }
  else if (dtype == kF16) { LAUNCH(__half) }
  else if (dtype == kBF16) { LAUNCH(__nv_bfloat16) }
  else return -1;
#undef LAUNCH
  return (int)cudaGetLastError();
}

// Adam / AdamW over up to mxb_max_tensors() tensors in one launch.  mean, var: fp32 states; w32: fp32 masters or null;
// rescale_ptr: device float or null (then rescale_host is used); decoupled: 0 = Adam, 1 = AdamW (etas used).
MXB_EXPORT int mxb_multi_adam(int dtype, int count, void** w, void** g, float** mean, float** var, float** w32,
                              const float* lrs, const float* wds, const float* etas, const int64_t* sizes, float beta1,
                              float beta2, float eps, float clip, const float* rescale_ptr, float rescale_host,
                              int decoupled, void* stream) {
  if (count > kMaxTensors || count <= 0 || !mean || !var) return -2;
  AdamTable tab;
  tab.count = count;
  int acc = 0;
  for (int i = 0; i < count; ++i) {
    tab.w[i] = w[i]; tab.g[i] = g[i]; tab.mean[i] = mean[i]; tab.var[i] = var[i];
    tab.w32[i] = w32 ? w32[i] : nullptr;
    tab.lr[i] = lrs[i]; tab.wd[i] = wds[i]; tab.eta[i] = etas ? etas[i] : 1.f; tab.n[i] = sizes[i];
    tab.chunk_start[i] = acc;
    acc += chunks_of(sizes[i]);
  }
  tab.chunk_start[count] = acc;
  int grid = acc < sm_count() * 8 ? acc : sm_count() * 8;
  if (grid < 1) grid = 1;
  cudaStream_t st = (cudaStream_t)stream;
  const bool mp = w32 != nullptr;
#define LAUNCH(T)                                                                                                              \
  if (mp && decoupled) multi_adam_kernel<T, true, true><<<grid, 256, 0, st>>>(tab, beta1, beta2, eps, clip, rescale_ptr, rescale_host);   \
  else if (mp) multi_adam_kernel<T, true, false><<<grid, 256, 0, st>>>(tab, beta1, beta2, eps, clip, rescale_ptr, rescale_host);          \
  else if (decoupled) multi_adam_kernel<T, false, true><<<grid, 256, 0, st>>>(tab, beta1, beta2, eps, clip, rescale_ptr, rescale_host);   \
  else multi_adam_kernel<T, false, false><<<grid, 256, 0, st>>>(tab, beta1, beta2, eps, clip, rescale_ptr, rescale_host);
  if (dtype == kF32) { LAUNCH(float) }
  else if (dtype == kF16) { LAUNCH(__half) }
  else if (dtype == kBF16) { LAUNCH(__nv_bfloat16) }
  else return -1;
#undef LAUNCH
  return (int)cudaGetLastError();
}

static int fill_ptr_table(PtrTable* tab, int count, void** p, const int64_t* sizes, const int* dtypes) {
  tab->count = count;
  int acc = 0;
  for (int i = 0; i < count; ++i) {
    tab->p[i] = p[i]; tab->n[i] = sizes[i]; tab->dtype[i] = dtypes[i];
    tab->chunk_start[i] = acc;
    acc += chunks_of(sizes[i]);
  }
  tab->chunk_start[count] = acc;
  return acc;
}

// out: one float, set to 1 by this call and cleared to 0 by the kernel when a non-finite value is found.
MXB_EXPORT int mxb_multi_all_finite(int count, void** p, const int64_t* sizes, const int* dtypes, float* out, int init,
                                    void* stream) {
  if (count > kMaxTensors || count <= 0) return -2;
  PtrTable tab;
  int acc = fill_ptr_table(&tab, count, p, sizes, dtypes);
  cudaStream_t st = (cudaStream_t)stream;
  if (init) set_float_kernel<<<1, 1, 0, st>>>(out, 1.f);
  int grid = acc < sm_count() * 8 ? acc : sm_count() * 8;
  if (grid < 1) grid = 1;
  multi_all_finite_kernel<<<grid, 256, 0, st>>>(tab, out);
  return (int)cudaGetLastError();
}

// Total chunk count for a set of sizes: the caller provides a scratch buffer of that many floats.
MXB_EXPORT int mxb_sum_sq_chunks(int count, const int64_t* sizes) {
  int acc = 0;
  for (int i = 0; i < count; ++i) acc += chunks_of(sizes[i]);
  return acc;
}

MXB_EXPORT int mxb_multi_sum_sq(int count, void** p, const int64_t* sizes, const int* dtypes, float* scratch, float* out,
                                int out_offset, void* stream) {
  if (count > kMaxTensors || count <= 0) return -2;
  PtrTable tab;
  int acc = fill_ptr_table(&tab, count, p, sizes, dtypes);
  cudaStream_t st = (cudaStream_t)stream;
  int grid = acc < sm_count() * 8 ? acc : sm_count() * 8;
  if (grid < 1) grid = 1;
  multi_sum_sq_partial_kernel<<<grid, 256, 0, st>>>(tab, scratch);
  multi_sum_sq_final_kernel<<<count, 128, 0, st>>>(tab, scratch, out, out_offset);
  return (int)cudaGetLastError();
}

// ---- sum of squares with a fixed scratch array (see optim_noalloc.h) ---------------------------------------
#include <mutex>

#include "optim_noalloc.h"

static_assert(MXB_SUM_SQ_CHUNK_ELEMS == mxb::kChunk, "header and kernels disagree on the chunk size");

// Stage-1 partial sums of mxb_multi_sum_sq_static: one slot per chunk, shared by every call on the device.
static __device__ __align__(256) float g_sum_sq_static_scratch[MXB_SUM_SQ_STATIC_MAX_CHUNKS];

namespace {
constexpr int kMaxDevices = 64;
float* g_static_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_static_scratch_mutex;

// Device address of the array on the current device, looked up once per device.
int static_scratch(float** out) {
  int dev = 0;
  cudaError_t rc = cudaGetDevice(&dev);
  if (rc != cudaSuccess) return (int)rc;
  if (dev < 0 || dev >= kMaxDevices) return MXB_SUM_SQ_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (!g_static_scratch_ptr[dev]) {
    float* ptr = nullptr;
    rc = cudaGetSymbolAddress((void**)&ptr, g_sum_sq_static_scratch);
    if (rc != cudaSuccess) return (int)rc;
    g_static_scratch_ptr[dev] = ptr;
  }
  *out = g_static_scratch_ptr[dev];
  return 0;
}
}  // namespace

MXB_EXPORT int mxb_multi_sum_sq_static(int count, void** p, const int64_t* sizes, const int* dtypes, float* out,
                                       int out_offset, void* stream) {
  if (count > kMaxTensors || count <= 0) return MXB_SUM_SQ_ERR_BAD_COUNT;
  int64_t chunks = 0;
  for (int i = 0; i < count; ++i) {
    if (sizes[i] < 0) return MXB_SUM_SQ_ERR_TOO_LARGE;
    chunks += sizes[i] / kChunk + (sizes[i] % kChunk != 0);      // no rounding-up addition: it would overflow near INT64_MAX
    if (chunks > MXB_SUM_SQ_STATIC_MAX_CHUNKS) return MXB_SUM_SQ_ERR_TOO_LARGE;
  }
  float* scratch = nullptr;
  int rc = static_scratch(&scratch);
  if (rc != 0) return rc;
  PtrTable tab;
  int acc = fill_ptr_table(&tab, count, p, sizes, dtypes);
  cudaStream_t st = (cudaStream_t)stream;
  int grid = acc < sm_count() * 8 ? acc : sm_count() * 8;
  if (grid < 1) grid = 1;
  multi_sum_sq_partial_kernel<<<grid, 256, 0, st>>>(tab, scratch);
  multi_sum_sq_final_kernel<<<count, 128, 0, st>>>(tab, scratch, out, out_offset);
  return (int)cudaGetLastError();
}

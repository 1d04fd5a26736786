// Fused gradient reduce-scatter + AMP unscale + inf/nan check + sharded optimizer update + weight
// all-gather over NVLink peer memory, as two kernel launches per training step.
//
// What the reference does per step (python/mxnet/gluon/trainer.py:392-486, src/kvstore/kvstore_nccl.h:212-425,
// src/kvstore/comm.h:535-654): one pushpull per parameter (ncclReduce to a root GPU, or P2P gather +
// ElementwiseSum), a multi_all_finite pass with a blocking host read, multi_mp_sgd_mom_update launches of
// at most 60 tensors, then ncclBcast / P2P copies of the weights.
//
// Here all parameters of a process live in one flat arena per GPU (weights, and gradients with the same
// layout).  Rank r owns the contiguous shard r of the arena together with the fp32 master weights and
// optimizer state of that shard only.
//   kernel A (reduce):  waits until every rank has finished its backward pass, then each rank sums ITS
//                       shard of the gradients by loading it from all ranks' arenas (plain 16-byte peer
//                       loads over NVSwitch), scales by rescale/loss_scale, records inf/nan and the sum of
//                       squares, keeps the reduced shard in fp32, and publishes {nonfinite, sumsq} to all ranks.
//   kernel B (update):  waits for all ranks' results, decides the step globally (skip on overflow, global-norm
//                       clipping coefficient), applies SGD-momentum / NAG on the fp32 master shard, writes the
//                       new low-precision weights into EVERY rank's weight arena (peer stores = all-gather),
//                       clears the local gradient arena, adapts the loss scale on the device, and returns
//                       only after all ranks have finished writing.
// Synchronisation is by step-numbered flags in a control block of every rank that peers write with
// st.release.sys and the owner polls with ld.acquire.sys.  Every wait is bounded by a wall-clock budget; when
// it expires the kernel records an error code in the control block, publishes "nonfinite" so that no rank
// applies a partial update, and returns normally (no trap, the context stays usable).
// Ranks run as separate processes on separate GPUs; the kernels never wait on another launch of the same GPU.
#include "common.cuh"

namespace mxb {

constexpr int kMaxRanks = 8;

enum StepMode { kModeSGD = 0, kModeNAG = 1, kModePlain = 2, kModeAdam = 3, kModeAdamW = 4, kModeLamb = 5 };
enum StepError { kOk = 0, kErrWaitReady = 1, kErrWaitReduced = 2, kErrWaitGather = 3, kErrWaitNorms = 4 };

struct __align__(256) Ctrl {
  // written by peers (index = sender rank)
  uint32_t ready[kMaxRanks];
  uint32_t reduced[kMaxRanks];
  uint32_t agdone[kMaxRanks];
  uint32_t normed[kMaxRanks];
  float payload[kMaxRanks][4];
  // local
  uint32_t ticket_a, ticket_b, ticket_c, pad0;
  uint32_t nonfinite;
  float sumsq;
  uint32_t status;          // first StepError seen (sticky until the host clears it)
  uint32_t status_step;
  float scale_state[4];     // [loss scale, clean steps, skipped steps total, last global grad norm]
};

struct StepParams {
  const void* grads[kMaxRanks];     // gradient arenas of all ranks (own entry = local pointer)
  void* weights[kMaxRanks];         // weight arenas of all ranks
  Ctrl* ctrl[kMaxRanks];
  int rank, nranks;
  int64_t total;                    // arena length in elements (multiple of 8)
  int64_t shard_begin, shard_end;   // this rank's shard [begin, end) in elements (multiples of 8)
  float* gred;                      // fp32 reduced gradient of the shard
  float* master;                    // fp32 master weights of the shard (null when weights are fp32)
  float* mom;                       // momentum of the shard (null when momentum == 0)
  const int64_t* seg_end;           // per-parameter end offsets in the arena (sorted)
  const float* lr_mult;             // per-parameter multipliers
  const float* wd_mult;
  int nseg;
  uint32_t step;
  float rescale;                    // host part of the gradient scale (1 / batch size ...)
  int use_loss_scale;               // 0 off, 1 divide by scale_state[0] and adapt it, 2 adapt only
  float lr, wd, momentum, clip_gradient, max_norm;
  float scale_window, scale_max;
  int mode;
  unsigned long long timeout_ns;
  // Adam / AdamW / LAMB
  float* var;                       // second moment of the shard (`mom` holds the first moment)
  float beta1, beta2, epsilon;
  float coef1, coef2;               // 1 - beta1^t, 1 - beta2^t of this step (1 when bias correction is off)
  float lower_bound, upper_bound;   // LAMB clamps of ||w|| (negative = off)
  float* norm_acc;                  // local [2][nseg]: per-parameter partial sums of w^2 and u^2 over this shard
  float* norm_in[kMaxRanks];        // every rank's receive area [kMaxRanks][2][nseg] (own entry = local pointer)
  const int* seg_skip;              // per-parameter flag: 1 = leave this parameter and its state untouched (stale gradient); may be null
  const float* seg_coef;            // per-parameter bias corrections [2][nseg] when the update counts differ; null = coef1 / coef2
  // NVLink-switch multicast (NVLS) addresses of the gradient and weight arenas: one address that stands for the same
  // offset in every rank's arena.  A multimem.ld_reduce on it returns the sum over all ranks, formed inside the switch
  // (one load instead of nranks peer loads); a multimem.st on it writes every rank's copy with one store.  Null = plain
  // peer loads and stores.
  const void* grads_mc;
  void* weights_mc;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---- multimem (NVLS) accesses: 16 bytes per instruction ---------------------------------------------------------------
template <typename T> __device__ __forceinline__ Vec16<T> mc_ld_reduce(const T* p);
template <> __device__ __forceinline__ Vec16<float> mc_ld_reduce<float>(const float* p) {
  Vec16<float> r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]) : "l"(p) : "memory");
  return r;
}
template <> __device__ __forceinline__ Vec16<__half> mc_ld_reduce<__half>(const __half* p) {
  uint32_t a, b, c, d;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "l"(p) : "memory");
  Vec16<__half> r;
  *reinterpret_cast<uint4*>(&r) = make_uint4(a, b, c, d);
  return r;
}
template <> __device__ __forceinline__ Vec16<__nv_bfloat16> mc_ld_reduce<__nv_bfloat16>(const __nv_bfloat16* p) {
  uint32_t a, b, c, d;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "l"(p) : "memory");
  Vec16<__nv_bfloat16> r;
  *reinterpret_cast<uint4*>(&r) = make_uint4(a, b, c, d);
  return r;
}
template <typename T>
__device__ __forceinline__ void mc_st16(T* p, const Vec16<T>& v) {
  const uint4 u = *reinterpret_cast<const uint4*>(&v);
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(p), "f"(__uint_as_float(u.x)), "f"(__uint_as_float(u.y)), "f"(__uint_as_float(u.z)), "f"(__uint_as_float(u.w))
               : "memory");
}
// One value for every rank's arena at element offset e: through the switch when a multicast address is known.
template <typename T>
__device__ __forceinline__ void store_all(void* const* arenas, void* mc, int nranks, int64_t e, const Vec16<T>& v) {
  if (mc) {
    mc_st16((T*)mc + e, v);
  } else {
    for (int r = 0; r < nranks; ++r) st16((T*)arenas[r] + e, v);
  }
}

// Threads 0..n-1 of the CTA each poll one flag until it reaches `step`; returns false on time-out.
__device__ bool wait_flags(const uint32_t* flags, int n, uint32_t step, unsigned long long timeout_ns) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < n) {
    const unsigned long long t0 = now_ns();
    unsigned spins = 0;
    while ((int32_t)(ld_acquire_sys(flags + threadIdx.x) - step) < 0) {
      if ((++spins & 63u) == 0) {
        if (now_ns() - t0 > timeout_ns) { ok = 0; break; }
        __nanosleep(200);
      }
    }
  }
  __syncthreads();
  return ok != 0;
}

template <typename T>
__global__ void __launch_bounds__(256) fused_reduce_kernel(const __grid_constant__ StepParams p) {
  __shared__ float red[32];
  Ctrl* me = p.ctrl[p.rank];
  bool alive = true;
  if (p.nranks > 1) {
    if (blockIdx.x == 0 && threadIdx.x < p.nranks) st_release_sys(&p.ctrl[threadIdx.x]->ready[p.rank], p.step);
    alive = wait_flags(me->ready, p.nranks, p.step, p.timeout_ns);
    if (!alive && threadIdx.x == 0) { atomicCAS(&me->status, (uint32_t)kOk, (uint32_t)kErrWaitReady); me->status_step = p.step; }
  }
  float sumsq = 0.f;
  bool bad = !alive;
  if (alive) {
    float scale = p.rescale;
    if (p.use_loss_scale == 1) scale /= me->scale_state[0];   // 2: the host already folded 1/scale into rescale
    constexpr int N = Vec16<T>::N;
    const int64_t v0 = p.shard_begin / N, v1 = p.shard_end / N;
    for (int64_t v = v0 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < v1; v += (int64_t)gridDim.x * blockDim.x) {
      float acc[N];
      if (p.grads_mc) {
        // the switch adds the ranks' values (fp32 accumulation) and returns the sum in the element type
        const Vec16<T> sum = mc_ld_reduce<T>((const T*)p.grads_mc + v * N);
#pragma unroll
        for (int j = 0; j < N; ++j) acc[j] = Cvt<T>::to_f(sum.v[j]);
      } else {
        Vec16<T> in[kMaxRanks];
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
          if (r < p.nranks) in[r] = ld16((const T*)p.grads[r] + v * N);
#pragma unroll
        for (int j = 0; j < N; ++j) acc[j] = 0.f;
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
          if (r < p.nranks) {
#pragma unroll
            for (int j = 0; j < N; ++j) acc[j] += Cvt<T>::to_f(in[r].v[j]);
          }
      }
      float* out = p.gred + (v * N - p.shard_begin);
#pragma unroll
      for (int j = 0; j < N; ++j) {
        acc[j] *= scale;
        bad |= !isfinite(acc[j]);
        sumsq += acc[j] * acc[j];
      }
#pragma unroll
      for (int j = 0; j < N; j += 4) *reinterpret_cast<float4*>(out + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
    }
  }
  sumsq = block_sum(sumsq, red);
  const int any_bad = __syncthreads_or(bad ? 1 : 0);
  if (threadIdx.x == 0) {
    if (any_bad) atomicOr(&me->nonfinite, 1u);
    atomicAdd(&me->sumsq, sumsq);
    __threadfence();
    const uint32_t ticket = atomicAdd(&me->ticket_a, 1u);
    if (ticket == gridDim.x - 1) {           // last CTA of this rank: publish the shard's summary
      __threadfence();
      const float nf = (float)atomicOr(&me->nonfinite, 0u);
      const float sq = atomicAdd(&me->sumsq, 0.f);
      for (int r = 0; r < p.nranks; ++r) {
        volatile float* dst = p.ctrl[r]->payload[p.rank];
        dst[0] = nf;
        dst[1] = sq;
      }
      __threadfence_system();
      for (int r = 0; r < p.nranks; ++r) st_release_sys(&p.ctrl[r]->reduced[p.rank], p.step);
      me->nonfinite = 0u;
      me->sumsq = 0.f;
      me->ticket_a = 0u;
    }
  }
}

__device__ __forceinline__ int find_segment(const int64_t* seg_end, int nseg, int64_t elem) {
  int lo = 0, hi = nseg - 1;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (seg_end[mid] > elem) hi = mid; else lo = mid + 1;
  }
  return lo;
}

// Common end of an optimizer step: clear the local gradient arena, adapt the loss scale, and leave only after every
// rank's stores into this GPU's weight arena have landed.
template <typename T>
__device__ void finish_step(const StepParams& p, Ctrl* me, bool skip, float sumsq) {
  constexpr int N = Vec16<T>::N;
  if (p.mode != kModePlain) {
    // every rank has finished reading this arena (all `reduced` flags seen): clear it for the next backward
    const uint4 z = make_uint4(0, 0, 0, 0);
    T* ga = (T*)p.grads[p.rank];
    const int64_t nv = p.total / N;
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < nv; v += (int64_t)gridDim.x * blockDim.x)
      *reinterpret_cast<uint4*>(ga + v * N) = z;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t ticket = atomicAdd(&me->ticket_b, 1u);
    if (ticket == gridDim.x - 1) {
      __threadfence();
      me->scale_state[3] = sqrtf(sumsq);
      if (p.use_loss_scale && p.mode != kModePlain) {
        float s = me->scale_state[0], good = me->scale_state[1];
        if (skip) { s = fmaxf(s * 0.5f, 1.f); good = 0.f; me->scale_state[2] += 1.f; }
        else {
          good += 1.f;
          if (good >= p.scale_window) { s = fminf(s * 2.f, p.scale_max); good = 0.f; }
        }
        me->scale_state[0] = s;
        me->scale_state[1] = good;
      } else if (skip && p.mode != kModePlain) {
        me->scale_state[2] += 1.f;
      }
      me->ticket_b = 0u;
      if (p.nranks > 1) {
        __threadfence_system();
        for (int r = 0; r < p.nranks; ++r) st_release_sys(&p.ctrl[r]->agdone[p.rank], p.step);
        // do not return before every rank's stores into this GPU's arena have landed
        const unsigned long long t0 = now_ns();
        for (int r = 0; r < p.nranks; ++r) {
          unsigned spins = 0;
          while ((int32_t)(ld_acquire_sys(&me->agdone[r]) - p.step) < 0) {
            if ((++spins & 63u) == 0) {
              if (now_ns() - t0 > p.timeout_ns) {
                atomicCAS(&me->status, (uint32_t)kOk, (uint32_t)kErrWaitGather);
                me->status_step = p.step;
                r = p.nranks;
                break;
              }
              __nanosleep(200);
            }
          }
        }
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) fused_update_kernel(const __grid_constant__ StepParams p) {
  Ctrl* me = p.ctrl[p.rank];
  constexpr int N = Vec16<T>::N;
  bool alive = wait_flags(me->reduced, p.nranks, p.step, p.timeout_ns);
  if (!alive && threadIdx.x == 0) { atomicCAS(&me->status, (uint32_t)kOk, (uint32_t)kErrWaitReduced); me->status_step = p.step; }
  float nonfinite = 0.f, sumsq = 0.f;
  for (int r = 0; r < p.nranks; ++r) {
    volatile float* src = me->payload[r];
    nonfinite += src[0];
    sumsq += src[1];
  }
  // a plain all-reduce passes inf/nan through like any sum; only an optimizer step is skipped on overflow
  const bool skip = !alive || (nonfinite != 0.f && p.mode != kModePlain);
  float coef = 1.f;
  if (p.max_norm > 0.f) coef = fminf(1.f, p.max_norm / (sqrtf(sumsq) + 1e-8f));
  if (!skip) {
    const int64_t v0 = p.shard_begin / N, v1 = p.shard_end / N;
    for (int64_t v = v0 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < v1; v += (int64_t)gridDim.x * blockDim.x) {
      const int64_t e = v * N, le = e - p.shard_begin;
      float g[N];
#pragma unroll
      for (int j = 0; j < N; j += 4) {
        float4 t = *reinterpret_cast<const float4*>(p.gred + le + j);
        g[j] = t.x; g[j + 1] = t.y; g[j + 2] = t.z; g[j + 3] = t.w;
      }
      Vec16<T> out;
      if (p.mode == kModePlain) {
#pragma unroll
        for (int j = 0; j < N; ++j) out.v[j] = Cvt<T>::from_f(g[j]);
        store_all<T>((void* const*)p.grads, const_cast<void*>(p.grads_mc), p.nranks, e, out);     // all-gather of the reduced gradient
        continue;
      }
      const int seg = find_segment(p.seg_end, p.nseg, e);
      if (p.seg_skip && p.seg_skip[seg]) continue;      // weights, master copy and state stay as they are on every rank
      const float lr = p.lr * p.lr_mult[seg], wd = p.wd * p.wd_mult[seg];
      float w[N], m[N];
      if (p.master) {
#pragma unroll
        for (int j = 0; j < N; j += 4) {
          float4 t = *reinterpret_cast<const float4*>(p.master + le + j);
          w[j] = t.x; w[j + 1] = t.y; w[j + 2] = t.z; w[j + 3] = t.w;
        }
      } else {
        Vec16<T> cur = ld16((const T*)p.weights[p.rank] + e);
#pragma unroll
        for (int j = 0; j < N; ++j) w[j] = Cvt<T>::to_f(cur.v[j]);
      }
      if (p.mom) {
#pragma unroll
        for (int j = 0; j < N; j += 4) {
          float4 t = *reinterpret_cast<const float4*>(p.mom + le + j);
          m[j] = t.x; m[j + 1] = t.y; m[j + 2] = t.z; m[j + 3] = t.w;
        }
      }
      const bool adam = p.mode == kModeAdam || p.mode == kModeAdamW;
      float s2[N];
      if (adam) {
#pragma unroll
        for (int j = 0; j < N; j += 4) {
          float4 t = *reinterpret_cast<const float4*>(p.var + le + j);
          s2[j] = t.x; s2[j + 1] = t.y; s2[j + 2] = t.z; s2[j + 3] = t.w;
        }
      }
      // Adam folds the bias correction into the step size (python/mxnet/optimizer/adam.py: lr *= sqrt(c2) / c1)
      const float c1 = p.seg_coef ? p.seg_coef[seg] : p.coef1, c2 = p.seg_coef ? p.seg_coef[p.nseg + seg] : p.coef2;
      const float lr_t = adam ? lr * sqrtf(c2) / c1 : lr;
#pragma unroll
      for (int j = 0; j < N; ++j) {
        float gr = g[j] * coef;
        if (p.clip_gradient >= 0.f) gr = fminf(fmaxf(gr, -p.clip_gradient), p.clip_gradient);
        if (adam) {
          if (p.mode == kModeAdam) gr += wd * w[j];
          m[j] = p.beta1 * m[j] + (1.f - p.beta1) * gr;
          s2[j] = p.beta2 * s2[j] + (1.f - p.beta2) * gr * gr;
          w[j] -= lr_t * m[j] / (sqrtf(s2[j]) + p.epsilon);
          if (p.mode == kModeAdamW && wd > 0.f) w[j] -= lr_t * wd * w[j];    // decoupled decay on the updated weight
        } else {
          gr += wd * w[j];
          if (p.mom) {
            m[j] = p.momentum * m[j] - lr * gr;
            w[j] += (p.mode == kModeNAG) ? (p.momentum * m[j] - lr * gr) : m[j];
          } else {
            w[j] -= lr * gr;
          }
        }
        out.v[j] = Cvt<T>::from_f(w[j]);
      }
      if (adam) {
#pragma unroll
        for (int j = 0; j < N; j += 4) *reinterpret_cast<float4*>(p.var + le + j) = make_float4(s2[j], s2[j + 1], s2[j + 2], s2[j + 3]);
      }
      if (p.master) {
#pragma unroll
        for (int j = 0; j < N; j += 4) *reinterpret_cast<float4*>(p.master + le + j) = make_float4(w[j], w[j + 1], w[j + 2], w[j + 3]);
      }
      if (p.mom) {
#pragma unroll
        for (int j = 0; j < N; j += 4) *reinterpret_cast<float4*>(p.mom + le + j) = make_float4(m[j], m[j + 1], m[j + 2], m[j + 3]);
      }
      store_all<T>(p.weights, p.weights_mc, p.nranks, e, out);       // all-gather of the new weights
    }
  }
  finish_step<T>(p, me, skip, sumsq);
}

// ---- LAMB (python/mxnet/optimizer/lamb.py; src/operator/contrib/multi_lamb.cu) -----------------------------------
// Phase 1: moments and the raw update u = m_hat / (sqrt(v_hat) + eps) + wd * w for this rank's shard (u replaces the
// reduced gradient in `gred`), plus per-parameter partial sums of w^2 and u^2; the partial sums of every rank are
// exchanged through peer stores.  Phase 2: trust ratio per parameter from the summed norms, weight update, all-gather.
__device__ __forceinline__ void load_f(const float* p, float* out, int n) {
  for (int j = 0; j < n; j += 4) {
    const float4 t = *reinterpret_cast<const float4*>(p + j);
    out[j] = t.x; out[j + 1] = t.y; out[j + 2] = t.z; out[j + 3] = t.w;
  }
}
__device__ __forceinline__ void store_f(float* p, const float* in, int n) {
  for (int j = 0; j < n; j += 4) *reinterpret_cast<float4*>(p + j) = make_float4(in[j], in[j + 1], in[j + 2], in[j + 3]);
}

__device__ __forceinline__ bool step_verdict(const StepParams& p, Ctrl* me, bool alive, float* sumsq_out) {
  float nonfinite = 0.f, sumsq = 0.f;
  for (int r = 0; r < p.nranks; ++r) {
    volatile float* src = me->payload[r];
    nonfinite += src[0];
    sumsq += src[1];
  }
  *sumsq_out = sumsq;
  return !alive || nonfinite != 0.f;
}

template <typename T>
__global__ void __launch_bounds__(256) fused_lamb1_kernel(const __grid_constant__ StepParams p) {
  Ctrl* me = p.ctrl[p.rank];
  constexpr int N = Vec16<T>::N;
  const bool alive = wait_flags(me->reduced, p.nranks, p.step, p.timeout_ns);
  if (!alive && threadIdx.x == 0) { atomicCAS(&me->status, (uint32_t)kOk, (uint32_t)kErrWaitReduced); me->status_step = p.step; }
  float sumsq;
  const bool skip = step_verdict(p, me, alive, &sumsq);
  float coef = 1.f;
  if (p.max_norm > 0.f) coef = fminf(1.f, p.max_norm / (sqrtf(sumsq) + 1e-8f));
  // Every CTA takes one contiguous chunk of the shard, so it meets few parameters (segments): the per-parameter sums
  // are collected in shared memory and reach the global accumulators once per CTA and segment.  (One global atomic per
  // warp and vector, all warps of a large parameter on the same two addresses, made this kernel several times slower
  // than its memory traffic.)
  constexpr int kSpan = 64;
  __shared__ float sacc[2][kSpan];
  const int64_t v0 = p.shard_begin / N, v1 = p.shard_end / N;
  const int64_t chunk = (v1 - v0 + gridDim.x - 1) / gridDim.x;
  const int64_t c0 = v0 + (int64_t)blockIdx.x * chunk, c1 = (c0 + chunk < v1) ? c0 + chunk : v1;
  int seg_first = 0, span = 0;
  if (c0 < c1) {
    seg_first = find_segment(p.seg_end, p.nseg, c0 * N);
    span = find_segment(p.seg_end, p.nseg, c1 * N - 1) - seg_first + 1;
  }
  const bool in_smem = span <= kSpan;
  for (int i = threadIdx.x; i < 2 * kSpan; i += blockDim.x) (&sacc[0][0])[i] = 0.f;
  __syncthreads();
  if (!skip) {
    int seg = seg_first;                   // positions of a thread only grow: the segment index is advanced, not searched
    for (int64_t v = c0 + threadIdx.x; v < c1; v += blockDim.x) {
      const int64_t e = v * N, le = e - p.shard_begin;
      while (seg < p.nseg - 1 && e >= p.seg_end[seg]) ++seg;
      const bool stale = p.seg_skip && p.seg_skip[seg];      // nothing of this parameter changes; phase 2 skips it as well
      const float wd = p.wd * p.wd_mult[seg];
      const float c1 = p.seg_coef ? p.seg_coef[seg] : p.coef1, c2 = p.seg_coef ? p.seg_coef[p.nseg + seg] : p.coef2;
      float g[N], w[N], m[N], s2[N];
      load_f(p.gred + le, g, N);
      load_f(p.mom + le, m, N);
      load_f(p.var + le, s2, N);
      if (p.master) {
        load_f(p.master + le, w, N);
      } else {
        const Vec16<T> cur = ld16((const T*)p.weights[p.rank] + e);
#pragma unroll
        for (int j = 0; j < N; ++j) w[j] = Cvt<T>::to_f(cur.v[j]);
      }
      float w2 = 0.f, u2 = 0.f;
#pragma unroll
      for (int j = 0; j < N; ++j) {
        float gr = g[j] * coef;
        if (p.clip_gradient >= 0.f) gr = fminf(fmaxf(gr, -p.clip_gradient), p.clip_gradient);
        m[j] = p.beta1 * m[j] + (1.f - p.beta1) * gr;
        s2[j] = p.beta2 * s2[j] + (1.f - p.beta2) * gr * gr;
        const float u = (m[j] / c1) / (sqrtf(s2[j] / c2) + p.epsilon) + wd * w[j];
        g[j] = u;
        w2 += w[j] * w[j];
        u2 += u * u;
      }
      if (!stale) {
        store_f(p.gred + le, g, N);
        store_f(p.mom + le, m, N);
        store_f(p.var + le, s2, N);
      } else {
        w2 = 0.f;
        u2 = 0.f;
      }
      // lanes of a warp that work on the same parameter combine their sums before the atomic
      const unsigned peers = __match_any_sync(__activemask(), seg);
      const int leader = __ffs(peers) - 1, lane = threadIdx.x & 31;
      float a = w2, b = u2;
      for (int o = 16; o > 0; o >>= 1) {
        const float a2 = __shfl_down_sync(peers, a, o), b2 = __shfl_down_sync(peers, b, o);
        if (lane + o < 32 && ((peers >> (lane + o)) & 1u)) { a += a2; b += b2; }
      }
      if (lane == leader) {
        if (in_smem) { atomicAdd(&sacc[0][seg - seg_first], a); atomicAdd(&sacc[1][seg - seg_first], b); }
        else { atomicAdd(p.norm_acc + seg, a); atomicAdd(p.norm_acc + p.nseg + seg, b); }
      }
    }
  }
  __syncthreads();
  if (!skip && in_smem) {
    for (int i = threadIdx.x; i < span; i += blockDim.x) {
      atomicAdd(p.norm_acc + seg_first + i, sacc[0][i]);
      atomicAdd(p.norm_acc + p.nseg + seg_first + i, sacc[1][i]);
    }
  }
  __threadfence();
  __syncthreads();
  __shared__ int last;
  if (threadIdx.x == 0) last = atomicAdd(&me->ticket_c, 1u) == gridDim.x - 1;
  __syncthreads();
  if (last) {                                  // last CTA of this rank: publish the partial norms to every rank
    __threadfence();
    const int n2 = 2 * p.nseg;
    for (int i = threadIdx.x; i < n2; i += blockDim.x) {
      const float val = __ldcg(p.norm_acc + i);
      for (int r = 0; r < p.nranks; ++r) p.norm_in[r][(int64_t)p.rank * n2 + i] = val;
      p.norm_acc[i] = 0.f;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < p.nranks) st_release_sys(&p.ctrl[threadIdx.x]->normed[p.rank], p.step);
    if (threadIdx.x == 0) me->ticket_c = 0u;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) fused_lamb2_kernel(const __grid_constant__ StepParams p) {
  Ctrl* me = p.ctrl[p.rank];
  constexpr int N = Vec16<T>::N;
  bool alive = wait_flags(me->reduced, p.nranks, p.step, p.timeout_ns);
  const bool normed = wait_flags(me->normed, p.nranks, p.step, p.timeout_ns);
  if (!normed && threadIdx.x == 0) { atomicCAS(&me->status, (uint32_t)kOk, (uint32_t)kErrWaitNorms); me->status_step = p.step; }
  alive = alive && normed;
  float sumsq;
  const bool skip = step_verdict(p, me, alive, &sumsq);
  if (!skip) {
    const int n2 = 2 * p.nseg;
    const float* recv = p.norm_in[p.rank];
    const int64_t v0 = p.shard_begin / N, v1 = p.shard_end / N;
    for (int64_t v = v0 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < v1; v += (int64_t)gridDim.x * blockDim.x) {
      const int64_t e = v * N, le = e - p.shard_begin;
      const int seg = find_segment(p.seg_end, p.nseg, e);
      if (p.seg_skip && p.seg_skip[seg]) continue;
      float w2 = 0.f, u2 = 0.f;
      for (int r = 0; r < p.nranks; ++r) {       // fixed order: every rank computes the same ratio
        w2 += __ldcg(recv + (int64_t)r * n2 + seg);
        u2 += __ldcg(recv + (int64_t)r * n2 + p.nseg + seg);
      }
      float r1 = sqrtf(w2);
      const float r2 = sqrtf(u2);
      if (p.lower_bound >= 0.f) r1 = fmaxf(r1, p.lower_bound);
      if (p.upper_bound >= 0.f) r1 = fminf(r1, p.upper_bound);
      const float ratio = (r1 == 0.f || r2 == 0.f) ? 1.f : r1 / r2;
      const float lr = p.lr * p.lr_mult[seg] * ratio;
      float u[N], w[N];
      load_f(p.gred + le, u, N);
      if (p.master) {
        load_f(p.master + le, w, N);
      } else {
        const Vec16<T> cur = ld16((const T*)p.weights[p.rank] + e);
#pragma unroll
        for (int j = 0; j < N; ++j) w[j] = Cvt<T>::to_f(cur.v[j]);
      }
      Vec16<T> out;
#pragma unroll
      for (int j = 0; j < N; ++j) { w[j] -= lr * u[j]; out.v[j] = Cvt<T>::from_f(w[j]); }
      if (p.master) store_f(p.master + le, w, N);
      store_all<T>(p.weights, p.weights_mc, p.nranks, e, out);
    }
  }
  finish_step<T>(p, me, skip, sumsq);
}

// A wait that nothing satisfies: used by tests of the time-out path (flag index `slot` of `ready`).
__global__ void wait_probe_kernel(Ctrl* me, int slot, uint32_t step, unsigned long long timeout_ns) {
  bool ok = wait_flags(me->ready + slot, 1, step, timeout_ns);
  if (!ok && threadIdx.x == 0) { atomicCAS(&me->status, (uint32_t)kOk, (uint32_t)kErrWaitReady); me->status_step = step; }
}

}  // namespace mxb

using namespace mxb;

MXB_EXPORT int mxb_step_ctrl_bytes() { return (int)sizeof(Ctrl); }
MXB_EXPORT int mxb_step_params_bytes() { return (int)sizeof(StepParams); }
MXB_EXPORT int mxb_step_max_ranks() { return kMaxRanks; }
// byte offsets inside Ctrl the host needs: status, status_step, scale_state
MXB_EXPORT int mxb_step_ctrl_offset(int which) {
  switch (which) {
    case 0: return (int)offsetof(Ctrl, status);
    case 1: return (int)offsetof(Ctrl, status_step);
    case 2: return (int)offsetof(Ctrl, scale_state);
    default: return -1;
  }
}

static int step_grid(int64_t shard_elems, int64_t total, int n_per_vec) {
  int64_t vecs = (shard_elems > total / 4 ? shard_elems : total / 4) / n_per_vec;
  int64_t blocks = (vecs + 255) / 256;
  int cap = sm_count() * 2;
  if (blocks < 1) blocks = 1;
  return (int)(blocks < cap ? blocks : cap);
}

// `params` is a host copy of StepParams filled by the caller.  dtype: storage type of the arenas.
MXB_EXPORT int mxb_fused_reduce(int dtype, const void* params, void* stream) {
  StepParams p = *static_cast<const StepParams*>(params);
  cudaStream_t st = (cudaStream_t)stream;
  if (p.nranks < 1 || p.nranks > kMaxRanks) return -2;
  if (dtype == kF32) fused_reduce_kernel<float><<<step_grid(p.shard_end - p.shard_begin, 0, 4), 256, 0, st>>>(p);
  else if (dtype == kF16) fused_reduce_kernel<__half><<<step_grid(p.shard_end - p.shard_begin, 0, 8), 256, 0, st>>>(p);
  else if (dtype == kBF16) fused_reduce_kernel<__nv_bfloat16><<<step_grid(p.shard_end - p.shard_begin, 0, 8), 256, 0, st>>>(p);
  else return -1;
  return (int)cudaGetLastError();
}

MXB_EXPORT int mxb_fused_update(int dtype, const void* params, void* stream) {
  StepParams p = *static_cast<const StepParams*>(params);
  cudaStream_t st = (cudaStream_t)stream;
  if (p.nranks < 1 || p.nranks > kMaxRanks) return -2;
  if (dtype == kF32) fused_update_kernel<float><<<step_grid(p.shard_end - p.shard_begin, p.total, 4), 256, 0, st>>>(p);
  else if (dtype == kF16) fused_update_kernel<__half><<<step_grid(p.shard_end - p.shard_begin, p.total, 8), 256, 0, st>>>(p);
  else if (dtype == kBF16) fused_update_kernel<__nv_bfloat16><<<step_grid(p.shard_end - p.shard_begin, p.total, 8), 256, 0, st>>>(p);
  else return -1;
  return (int)cudaGetLastError();
}

// LAMB: phase 1 (moments, raw update, partial norms) and phase 2 (trust ratio, update, all-gather) after mxb_fused_reduce.
MXB_EXPORT int mxb_fused_lamb(int dtype, const void* params, void* stream) {
  StepParams p = *static_cast<const StepParams*>(params);
  cudaStream_t st = (cudaStream_t)stream;
  if (p.nranks < 1 || p.nranks > kMaxRanks) return -2;
  if (!p.mom || !p.var || !p.norm_acc || !p.norm_in[p.rank] || p.nseg < 1) return -3;
#define MXB_LAMB(T, n)                                                                                   \
  fused_lamb1_kernel<T><<<step_grid(p.shard_end - p.shard_begin, 0, n), 256, 0, st>>>(p);                  \
  fused_lamb2_kernel<T><<<step_grid(p.shard_end - p.shard_begin, p.total, n), 256, 0, st>>>(p);
  if (dtype == kF32) { MXB_LAMB(float, 4) }
  else if (dtype == kF16) { MXB_LAMB(__half, 8) }
  else if (dtype == kBF16) { MXB_LAMB(__nv_bfloat16, 8) }
  else return -1;
#undef MXB_LAMB
  return (int)cudaGetLastError();
}

MXB_EXPORT int mxb_wait_probe(void* ctrl, int slot, uint32_t step, unsigned long long timeout_ns, void* stream) {
  wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(static_cast<Ctrl*>(ctrl), slot, step, timeout_ns);
  return (int)cudaGetLastError();
}

// ---- peer-memory plumbing -------------------------------------------------------------------------------
MXB_EXPORT int mxb_dev_alloc(void** ptr, uint64_t bytes) {
  int rc = (int)cudaMalloc(ptr, bytes);
  if (rc == 0) rc = (int)cudaMemset(*ptr, 0, bytes);
  return rc;
}
MXB_EXPORT int mxb_dev_free(void* ptr) { return (int)cudaFree(ptr); }
MXB_EXPORT int mxb_ipc_handle_bytes() { return (int)sizeof(cudaIpcMemHandle_t); }
MXB_EXPORT int mxb_ipc_get_handle(void* ptr, void* out) {
  cudaIpcMemHandle_t h;
  int rc = (int)cudaIpcGetMemHandle(&h, ptr);
  if (rc == 0) memcpy(out, &h, sizeof(h));
  return rc;
}
MXB_EXPORT int mxb_ipc_open(const void* handle, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}
MXB_EXPORT int mxb_ipc_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }
// Lets kernels and copies of device `dev` address the memory of device `peer` (both of this process).  Returns 0 also
// when the access was enabled before; the caller's current device is left as it was.
MXB_EXPORT int mxb_enable_peer_access(int dev, int peer) {
  int prev = 0, can = 0;
  cudaGetDevice(&prev);
  cudaError_t rc = cudaDeviceCanAccessPeer(&can, dev, peer);
  if (rc == cudaSuccess && !can) rc = cudaErrorPeerAccessUnsupported;
  if (rc == cudaSuccess) rc = cudaSetDevice(dev);
  if (rc == cudaSuccess) {
    rc = cudaDeviceEnablePeerAccess(peer, 0);
    if (rc == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); rc = cudaSuccess; }
  }
  cudaSetDevice(prev);
  return (int)rc;
}
MXB_EXPORT int mxb_memcpy_d2h(void* dst, const void* src, uint64_t bytes, void* stream) {
  return (int)cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
}
MXB_EXPORT int mxb_memcpy_d2d(void* dst, const void* src, uint64_t bytes, void* stream) {
  return (int)cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
}
MXB_EXPORT int mxb_memcpy_h2d(void* dst, const void* src, uint64_t bytes, void* stream) {
  return (int)cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream);
}
MXB_EXPORT const char* mxb_error_string(int code) { return cudaGetErrorString((cudaError_t)code); }

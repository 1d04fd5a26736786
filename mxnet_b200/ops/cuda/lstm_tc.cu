// LSTM recurrence on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), forward and backward.
//
// Reference behaviour: the `RNN` operator in lstm mode (src/operator/rnn-inl.h: cudnnRNNForwardTraining /
// cudnnRNNBackwardData; CPU math in src/operator/rnn_impl.h, LstmForwardTraining and LstmBackward).  Gate order i, f, g, o.
//
// The input projection of all time steps is one GEMM done before this kernel; what remains per step is
//     a_t = xproj_t + h_{t-1} W_hh^T,  i,f,o = sigmoid(a), g = tanh(a),  c_t = f c_{t-1} + i g,  h_t = o tanh(c_t)
// a (batch x H) by (H x 4H) product whose cost is latency, not FLOPs.  One cooperative launch covers all time steps:
//   * CTA c owns U consecutive hidden units.  The 4U rows of W_hh that produce their gates stay in shared memory for the
//     whole sequence as the B operand of the MMA ([4U, H] K-major, 128-byte swizzle, loaded once by TMA).
//   * h_{t-1} lives in a row-major exchange buffer [batch, H] in global memory (L2).  Per step the producer lane streams
//     it through a ring of TMA boxes (batch rows x 128 bytes of K) as the A operand, the MMA lane issues
//     tcgen05.mma (M = 128 batch rows, N = 4U gate columns) into a TMEM accumulator.
//   * TMEM lane b then holds all four gates of the CTA's units for batch row b, so epilogue thread b does the whole cell
//     update in registers (c never leaves the thread), writes y_t and the new h slice into the other half of the exchange
//     buffer, and all CTAs meet at a grid barrier (arrival counter, bounded spin).
// fp32 models run kind::tf32 (U = 8), half-precision models kind::f16 (U = 16).
// Backward walks the steps in reverse with the same ownership: thread b turns dh_t (upstream + recurrent part read from
// TMEM) and the carried dc into the four gate gradients of its units, publishes them in an exchange buffer
// [batch, 4H'] (columns grouped per CTA), and after the barrier each CTA contracts ALL gate gradients with its U columns
// of W_hh (resident in shared memory, [U, 4H'] K-major) to get dh_{t-1} for its units, again lane b = batch row b.
// Weight and input gradients are large GEMMs over the saved gate gradients, done outside.
// Every wait is bounded; a CTA that gives up sets the error word, all CTAs leave at the next barrier, TMEM is freed.
#include "tcgen05.cuh"

namespace mxb {

constexpr int kTcThreads = 192;                 // warp 0: TMA producer, warp 1: MMA issuer, warps 2..5: epilogue
constexpr int kTcMaxStages = 16;
constexpr unsigned long long kTcBarrierNs = 2000000000ull;

struct LstmTcParams {
  const void* xproj;     // [T, B, KK]  x W_ih^T + b_ih + b_hh, columns in the per-CTA order c*4U + g*U + u
  const void* h0;        // [B, H]
  const void* c0;        // [B, H]
  void* y;               // [T, B, H]
  void* hT;              // [B, H]
  void* cT;              // [B, H]
  void* gates;           // [T, B, KK] activated gates, column c*4U + g*U + u (saved for backward; may be null)
  float* cs;             // [T, B, Hc] cell states (saved for backward; may be null)
  void* hbuf;            // [2, Bp, Hp] exchange buffer of h in the MMA operand type, zero-initialised
  unsigned int* bar;     // [2] arrival counter, error flag (zero-initialised)
  int T, B, H;
  int Bp;                // batch rounded up to 8
  int Hp;                // H rounded up to whole 128-byte chunks (row length of hbuf and of the packed weights)
  int Hc;                // units rounded up to whole CTAs (C * U)
  int KK;                // 4 * Hc: gate columns in per-CTA order
  int stages;            // ring depth
  int yalign;            // bytes to which every row of y / dy is aligned (a divisor of 16 given by H)
  // backward
  const void* dy;        // [T, B, H]
  const void* dhT;       // [B, H] or null
  const void* dcT;       // [B, H] or null
  void* dgates;          // [T, B, KK] gate gradients, columns in the per-CTA order: the saved result for the GEMMs outside
                         // and, step by step, the operand that the product of that step streams
  void* dh0;             // [B, H]
  void* dc0;             // [B, H]
};

template <typename X> struct TcType;
template <> struct TcType<float> {            // kind::tf32
  static constexpr int KC = 32;               // elements per 128-byte chunk
  static constexpr uint32_t FMT = 2;          // tf32 operand code of the instruction descriptor
};
template <> struct TcType<__half> { static constexpr int KC = 64; static constexpr uint32_t FMT = 0; };
template <> struct TcType<__nv_bfloat16> { static constexpr int KC = 64; static constexpr uint32_t FMT = 1; };

__host__ __device__ constexpr uint32_t tc_idesc(uint32_t fmt, int n) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

template <typename X>
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if constexpr (sizeof(X) == 4) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    umma(tmem_d, adesc, bdesc, idesc, accumulate);
  }
}

__device__ __forceinline__ unsigned long long tc_now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// The error word keeps the first failure: 1 = grid barrier, 2 = producer waiting for a free stage, 3 = MMA lane waiting for
// a load, 4 = epilogue waiting for the accumulator, 5 = resident weights not loaded,
// 6 = a wait inside this CTA failed earlier.
__device__ __forceinline__ void tc_fail(unsigned int* bar, unsigned int code) { atomicCAS(bar + 1, 0u, code); }

// Thread 0 of every CTA: arrive and wait until `target` arrivals; false when the others did not show up in time or an
// error was flagged.  The caller brackets it with __syncthreads.
__device__ bool tc_grid_arrive_wait(unsigned int* bar, unsigned int target) {
  __threadfence();
  atomicAdd(bar, 1u);
  const unsigned long long t0 = tc_now_ns();
  unsigned spins = 0;
  bool ok = true;
  while ((int)(*(volatile unsigned int*)bar - target) < 0) {
    if (*(volatile unsigned int*)(bar + 1) != 0u) { ok = false; break; }
    if ((++spins & 63u) == 0 && tc_now_ns() - t0 > kTcBarrierNs) {
      tc_fail(bar, 1u);
      ok = false;
      break;
    }
  }
  __threadfence();
  return ok;
}

// mbarrier wait bounded by wall time (one second): false when the phase did not complete.
__device__ __forceinline__ bool tc_mbar_wait(uint64_t* bar, uint32_t parity) {
  const unsigned long long t0 = tc_now_ns();
  unsigned spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 63u) == 0 && tc_now_ns() - t0 > 1000000000ull) return false;
  }
  return true;
}
__device__ __forceinline__ bool tc_mbar_wait_warp(uint64_t* bar, uint32_t parity) {
  return __all_sync(0xffffffffu, tc_mbar_wait(bar, parity) ? 1 : 0) != 0;
}

__device__ __forceinline__ float tc_sigmoid(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float tc_tanh(float x) { return 2.f / (1.f + __expf(-2.f * x)) - 1.f; }

__device__ __forceinline__ void tc_fence_async_global() { asm volatile("fence.proxy.async;" ::: "memory"); }

// N consecutive elements through accesses of W bytes (the pointer is W-byte aligned; N * sizeof(T) is a multiple of W).
template <typename T, int N, int W>
__device__ __forceinline__ void tc_ld_w(const T* p, float* v) {
  constexpr int E = W / (int)sizeof(T);
  struct alignas(W) Chunk { T e[E]; };
#pragma unroll
  for (int i = 0; i < N; i += E) {
    const Chunk c = *reinterpret_cast<const Chunk*>(p + i);
#pragma unroll
    for (int j = 0; j < E; ++j) v[i + j] = Cvt<T>::to_f(c.e[j]);
  }
}
template <typename T, int N, int W>
__device__ __forceinline__ void tc_st_w(T* p, const float* v) {
  constexpr int E = W / (int)sizeof(T);
  struct alignas(W) Chunk { T e[E]; };
#pragma unroll
  for (int i = 0; i < N; i += E) {
    Chunk c;
#pragma unroll
    for (int j = 0; j < E; ++j) c.e[j] = Cvt<T>::from_f(v[i + j]);
    *reinterpret_cast<Chunk*>(p + i) = c;
  }
}
// A row of N elements whose alignment (`align` bytes, the same for every thread) depends on the row pitch; `nvalid`
// elements exist (fewer than N only in the last CTA).
template <typename T, int N>
__device__ __forceinline__ void tc_ld_row(const T* p, float* v, int align, int nvalid) {
  if (nvalid >= N && align >= 16) tc_ld_w<T, N, 16>(p, v);
  else if (nvalid >= N && align >= 8) tc_ld_w<T, N, 8>(p, v);
  else if (nvalid >= N && align >= 4) tc_ld_w<T, N, 4>(p, v);
  else {
#pragma unroll
    for (int j = 0; j < N; ++j) v[j] = j < nvalid ? Cvt<T>::to_f(p[j]) : 0.f;
  }
}
template <typename T, int N>
__device__ __forceinline__ void tc_st_row(T* p, const float* v, int align, int nvalid) {
  if (nvalid >= N && align >= 16) tc_st_w<T, N, 16>(p, v);
  else if (nvalid >= N && align >= 8) tc_st_w<T, N, 8>(p, v);
  else if (nvalid >= N && align >= 4) tc_st_w<T, N, 4>(p, v);
  else {
#pragma unroll
    for (int j = 0; j < N; ++j)
      if (j < nvalid) p[j] = Cvt<T>::from_f(v[j]);
  }
}

template <int NCOL>
__device__ __forceinline__ void tc_tmem_load(uint32_t taddr, float* v) {
  uint32_t r[32];
#pragma unroll
  for (int c0 = 0; c0 < NCOL; c0 += 32) {
    tmem_ld32(taddr + (uint32_t)c0, r);
    tmem_wait_ld32(r);
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (c0 + j < NCOL) v[c0 + j] = __uint_as_float(r[j]);
  }
}

// Shared bookkeeping at the start of both kernels' dynamic shared memory (after the 1024-byte alignment).
struct TcShared {
  uint64_t full[kTcMaxStages];
  uint64_t empty[kTcMaxStages];
  uint64_t acc_full;
  uint64_t w_full;
  uint32_t tmem_slot;
  volatile int abort_flag;
  volatile int issued_it;
  volatile int consumed_it;
};

// Producer and MMA lanes of one product phase: stream `nk` chunks of the exchange buffer (rows y0 .. y0+Bp of `map_x`)
// against the resident operand whose chunk `kc` starts at `w_base + kc * w_chunk_bytes`.
template <typename X>
__device__ __forceinline__ void tc_produce(TcShared* sh, unsigned int* bar, uint8_t* ring, uint32_t stage_bytes, int stages,
                                           const CUtensorMap* map_x, int y0, int nk, int& st, uint32_t& ph, int& it) {
  constexpr int KC = TcType<X>::KC;
  for (int kc = 0; kc < nk; ++kc) {
    if (!tc_mbar_wait(&sh->empty[st], ph ^ 1u)) { sh->abort_flag = 1; tc_fail(bar, 2u); return; }
    mbar_expect_tx(&sh->full[st], stage_bytes);
    tma_load_2d(ring + (size_t)st * stage_bytes, map_x, kc * KC, y0, &sh->full[st]);
    ++it;
    if (++st == stages) { st = 0; ph ^= 1u; }
  }
}

template <typename X>
__device__ __forceinline__ void tc_consume(TcShared* sh, unsigned int* bar, uint8_t* ring, uint32_t stage_bytes, int stages, uint8_t* w_base,
                                           uint32_t w_chunk_bytes, int nk, uint32_t tmem_d, uint32_t idesc, int& st, uint32_t& ph,
                                           int& it) {
  const uint64_t adesc0 = make_desc(smem_u32(ring)), bdesc0 = make_desc(smem_u32(w_base));
  for (int kc = 0; kc < nk; ++kc) {
    if (!tc_mbar_wait(&sh->full[st], ph)) { sh->abort_flag = 1; tc_fail(bar, 3u); return; }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint64_t adesc = adesc0 + (uint64_t)((uint32_t)st * (stage_bytes >> 4));
    const uint64_t bdesc = bdesc0 + (uint64_t)((uint32_t)kc * (w_chunk_bytes >> 4));
#pragma unroll
    for (int k = 0; k < 4; ++k)                 // 32 bytes of K per instruction inside the 128-byte swizzle row
      tc_mma<X>(tmem_d, adesc + 2 * (uint64_t)k, bdesc + 2 * (uint64_t)k, idesc, (kc > 0 || k > 0) ? 1u : 0u);
    umma_commit(&sh->empty[st]);
    ++it;
    if (++st == stages) { st = 0; ph ^= 1u; }
  }
  umma_commit(&sh->acc_full);
}

// ---- forward -----------------------------------------------------------------------------------------------------------
// Dynamic shared memory: [ring: stages x Bp x 128][W: Hp/KC chunks x 4U x 128][TcShared].  The MMA reads 128 rows from a
// stage; rows beyond Bp are whatever follows in shared memory and only reach accumulator lanes that nobody reads.
template <typename T, typename X, int U>
__global__ void __launch_bounds__(kTcThreads, 1)
lstm_tc_fwd_kernel(const __grid_constant__ CUtensorMap map_h, const __grid_constant__ CUtensorMap map_w, const LstmTcParams p) {
  constexpr int KC = TcType<X>::KC;
  constexpr int NG = 4 * U;
  constexpr uint32_t W_CHUNK = NG * 128;
  constexpr uint32_t TMEM_COLS = NG < 32 ? 32 : NG;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int nk = p.Hp / KC;
  const uint32_t stage_bytes = (uint32_t)p.Bp * 128u;
  uint8_t* ring = smem;
  uint8_t* sW = ring + (size_t)p.stages * stage_bytes;
  TcShared* sh = reinterpret_cast<TcShared*>(sW + (size_t)nk * W_CHUNK);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  const unsigned int nctas = gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&sh->full[s], 1); mbar_init(&sh->empty[s], 1); }
    mbar_init(&sh->acc_full, 1);
    mbar_init(&sh->w_full, 1);
    sh->abort_flag = 0;
    sh->issued_it = 0;
    sh->consumed_it = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = sh->tmem_slot;

  // resident weights: one TMA box per chunk, all on one barrier
  if (threadIdx.x == 0) {
    mbar_expect_tx(&sh->w_full, (uint32_t)nk * W_CHUNK);
    for (int kc = 0; kc < nk; ++kc) tma_load_2d(sW + (size_t)kc * W_CHUNK, &map_w, kc * KC, cta * NG, &sh->w_full);
  }

  // epilogue threads: batch row b, units cta*U .. cta*U+U-1; c stays in registers for the whole sequence
  const int q = warp & 3;
  const int b = q * 32 + lane;
  const bool epi = warp >= 2;
  const bool row_ok = epi && b < p.B;
  const int unit0 = cta * U;
  float c[U];
  X* hbuf = static_cast<X*>(p.hbuf);
  if (row_ok) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const bool ok = unit0 + u < p.H;
      c[u] = ok ? Cvt<T>::to_f(static_cast<const T*>(p.c0)[(size_t)b * p.H + unit0 + u]) : 0.f;
      if (ok) hbuf[(size_t)b * p.Hp + unit0 + u] = Cvt<X>::from_f(Cvt<T>::to_f(static_cast<const T*>(p.h0)[(size_t)b * p.H + unit0 + u]));
    }
    tc_fence_async_global();
  }
  __syncthreads();
  __shared__ int step_ok;
  if (threadIdx.x == 0) {
    bool ok = tc_grid_arrive_wait(p.bar, nctas);
    if (ok && !tc_mbar_wait(&sh->w_full, 0)) { ok = false; tc_fail(p.bar, 5u); }
    tc_fence_async_global();
    step_ok = ok ? 1 : 0;
  }
  __syncthreads();
  bool alive = step_ok != 0;

  int pst = 0, pit = 0, cst = 0, cit = 0;
  uint32_t pph = 0, cph = 0;
  const uint32_t idesc = tc_idesc(TcType<X>::FMT, NG);
  for (int t = 0; t < p.T && alive; ++t) {
    const int par = t & 1;
    if (warp == 0) {
      if (lane == 0) {
        tc_produce<X>(sh, p.bar, ring, stage_bytes, p.stages, &map_h, par * p.Bp, nk, pst, pph, pit);
        sh->issued_it = pit;
      }
    } else if (warp == 1) {
      if (lane == 0) {
        tc_consume<X>(sh, p.bar, ring, stage_bytes, p.stages, sW, W_CHUNK, nk, tmem_base, idesc, cst, cph, cit);
        sh->consumed_it = cit;
      }
    } else {
      // this step's input projection (4U consecutive values per thread), fetched while the product runs
      float a[NG];
      if (row_ok) tc_ld_w<T, NG, 16>(static_cast<const T*>(p.xproj) + ((size_t)t * p.B + b) * p.KK + (size_t)cta * NG, a);
      const bool ready = tc_mbar_wait_warp(&sh->acc_full, (uint32_t)t & 1u);
      if (!ready) { sh->abort_flag = 1; tc_fail(p.bar, 4u); }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float v[NG];
      if (ready) tc_tmem_load<NG>(tmem_base + ((uint32_t)(q * 32) << 16), v);      // warp-wide: tcgen05.ld is .sync.aligned
      if (ready && row_ok) {
        float hv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const float ig = tc_sigmoid(v[u] + a[u]);
          const float fg = tc_sigmoid(v[U + u] + a[U + u]);
          const float gg = tc_tanh(v[2 * U + u] + a[2 * U + u]);
          const float og = tc_sigmoid(v[3 * U + u] + a[3 * U + u]);
          c[u] = fg * c[u] + ig * gg;
          hv[u] = unit0 + u < p.H ? og * tc_tanh(c[u]) : 0.f;
          a[u] = ig;
          a[U + u] = fg;
          a[2 * U + u] = gg;
          a[3 * U + u] = og;
        }
        const int nvalid = p.H - unit0 < U ? p.H - unit0 : U;
        tc_st_w<X, U, 16>(hbuf + ((size_t)(par ^ 1) * p.Bp + b) * p.Hp + unit0, hv);       // columns >= H stay zero
        tc_st_row<T, U>(static_cast<T*>(p.y) + ((size_t)t * p.B + b) * p.H + unit0, hv, p.yalign, nvalid);
        if (p.gates) tc_st_w<T, NG, 16>(static_cast<T*>(p.gates) + ((size_t)t * p.B + b) * p.KK + (size_t)cta * NG, a);
        if (p.cs) tc_st_w<float, U, 16>(p.cs + ((size_t)t * p.B + b) * p.Hc + unit0, c);
        if (t == p.T - 1) {
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (unit0 + u < p.H) {
              static_cast<T*>(p.hT)[(size_t)b * p.H + unit0 + u] = Cvt<T>::from_f(hv[u]);
              static_cast<T*>(p.cT)[(size_t)b * p.H + unit0 + u] = Cvt<T>::from_f(c[u]);
            }
        }
        tc_fence_async_global();          // the next step's TMA loads (async proxy) read what these stores wrote
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      bool ok = sh->abort_flag == 0;
      if (!ok) tc_fail(p.bar, 6u);
      if (ok && t + 1 < p.T) ok = tc_grid_arrive_wait(p.bar, (unsigned int)(t + 2) * nctas);
      tc_fence_async_global();
      step_ok = ok ? 1 : 0;
    }
    __syncthreads();
    alive = step_ok != 0;
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && sh->abort_flag) {
    for (int it = sh->consumed_it; it < sh->issued_it; ++it) tc_mbar_wait(&sh->full[it % p.stages], (uint32_t)(it / p.stages) & 1u);
    tc_fail(p.bar, 6u);
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

#include "lstm_tc_bwd.inl"
#include "lstm_tc_bwdc.inl"
#include "gru_tc.inl"

}  // namespace mxb

#include "lstm_tc_host.inl"

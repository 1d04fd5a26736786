// Fused multi-head self-attention for sm_100a: QKᵀ, masked softmax, dropout and PV in one kernel on the tcgen05
// tensor cores, forward and backward.
//
// Reference behaviour: the interleaved_matmul_selfatt_qk → softmax → Dropout → interleaved_matmul_selfatt_valatt chain
// (src/operator/contrib/transformer.cu: strided-batched cuBLAS GEMMs with the [T, T] score matrix written to and read
// back from HBM three times in the forward pass alone).
//
// Shapes: packed projection qkv [N, T, 3C] = [Q | K | V], C = heads * 64, T <= 128; optional key mask [N, T];
// output [N, T, C].  One CTA handles one (sample, head): the whole [T, T] score tile lives in TMEM and shared memory.
//   warp 0     : TMA loads of the Q, K, V (and dO) tiles straight out of the packed tensors (3-D tensor maps, rows
//                beyond T read as zeros).
//   warp 1     : one lane issues the tcgen05.mma chains: S = Q·Kᵀ (K-major operands), then O = P·V with P read from
//                shared memory and V used as an MN-major operand (no transposed copy); backward: S, dP = dO·Vᵀ,
//                dV = P̃ᵀ·dO, dQ = dS·K, dK = dSᵀ·Q, where the transposed operands are MN-major views of the same
//                shared-memory tiles.
//   warps 2..5 : one thread per query row: reads its row of S from TMEM, applies scale and key mask, max / exp / sum
//                in registers, dropout by a counter-based hash (recomputed in backward, no mask tensor), writes
//                P (fp16/bf16) into shared memory in the 128-byte-swizzled operand layout, later normalises and
//                stores the output rows.
// Every mbarrier wait is bounded; on expiry the CTA sets an error flag, skips the rest, frees its TMEM and exits.
#include "tcgen05.cuh"

namespace mxb {

constexpr int kAttT = 128, kAttD = 64;
constexpr int kAttThreads = 192;
constexpr uint32_t kTileBytes = kAttT * kAttD * 2;     // 16 KB: one [128 x 64] half tile

struct AttnParams {
  const void* mask;        // [N, T] float, 0 = masked key (or null)
  void* out;               // forward: [N, T, C]
  float* lse;              // [N, heads, T] log-sum-exp of the scaled, masked scores
  const void* o;           // backward: forward output [N, T, C]
  const void* dout;        // backward: [N, T, C]
  void* dqkv;              // backward: [N, T, 3C]
  int N, T, C, heads;
  float scale;             // 1 / sqrt(D)
  float keep_scale;        // 1 / (1 - p)
  uint32_t drop_threshold; // keep an element when hash >= threshold (0 = no dropout)
  const uint32_t* seed;    // device word: the dropout pattern of this call (read at run time, so a captured graph
                           // that advances the word before each launch draws a new pattern on every replay)
  int* error_flag;
};

__device__ __forceinline__ uint32_t att_hash(uint32_t seed, uint32_t idx) {
  uint32_t x = idx * 0x9E3779B1u ^ seed;
  x ^= x >> 16; x *= 0x85EBCA6Bu; x ^= x >> 13; x *= 0xC2B2AE35u; x ^= x >> 16;
  return x;
}

// Byte offset of element (row, col) of a [128 rows x 64 cols] half tile in the 128-byte-swizzled operand layout.
__device__ __forceinline__ uint32_t swz_chunk_offset(int row, int chunk16 /* 0..7 */) {
  return (uint32_t)row * 128u + (uint32_t)((chunk16 ^ (row & 7)) << 4);
}

template <typename T>
__device__ __forceinline__ void store8_swz(uint8_t* tile, int row, int chunk16, const float* v) {
  Vec16<T> o;
#pragma unroll
  for (int j = 0; j < 8; ++j) o.v[j] = Cvt<T>::from_f(v[j]);
  *reinterpret_cast<uint4*>(tile + swz_chunk_offset(row, chunk16)) = *reinterpret_cast<const uint4*>(&o);
}

// ------------------------------------------------------------------------------------------------ forward
// shared memory: Q | K | V | P0 | P1 tiles (16 KB each, 1024-byte aligned), key bias [128] floats, barriers.
constexpr uint32_t kFwdSmem = 5 * kTileBytes + 128 * 4 + 1024 + 256;

template <typename T>
__global__ void __launch_bounds__(kAttThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_qkv, const AttnParams p, int bf16) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kTileBytes;
  uint8_t* sV = smem + 2 * kTileBytes;
  uint8_t* sP = smem + 3 * kTileBytes;                 // two k-stages of P: keys 0..63, 64..127
  float* kbias = reinterpret_cast<float*>(smem + 5 * kTileBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(kbias + 128);
  uint64_t* bar_qk = bars, *bar_v = bars + 1, *bar_s = bars + 2, *bar_p = bars + 3, *bar_o = bars + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x / p.heads, h = blockIdx.x % p.heads;
  constexpr uint32_t kTmemCols = 256;                  // S: columns [0, 128), O: [128, 192)

  if (threadIdx.x == 0) {
    mbar_init(bar_qk, 1); mbar_init(bar_v, 1); mbar_init(bar_s, 1); mbar_init(bar_p, 4); mbar_init(bar_o, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // additive key bias: 0 for valid keys, -inf for masked keys and keys beyond T
  if (threadIdx.x >= 64 && threadIdx.x < 192) {
    const int k = threadIdx.x - 64;
    bool valid = k < p.T;
    if (valid && p.mask) valid = static_cast<const float*>(p.mask)[(int64_t)b * p.T + k] != 0.f;
    kbias[k] = valid ? 0.f : -INFINITY;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar_qk, 2 * kTileBytes);
      tma_load_3d(sQ, &map_qkv, h * kAttD, 0, b, bar_qk);
      tma_load_3d(sK, &map_qkv, p.C + h * kAttD, 0, b, bar_qk);
      mbar_expect_tx(bar_v, kTileBytes);
      tma_load_3d(sV, &map_qkv, 2 * p.C + h * kAttD, 0, b, bar_v);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(bar_qk, 0);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t idesc = make_idesc(bf16, 128, 0, 0);
        const uint64_t qd = make_desc(smem_u32(sQ)), kd = make_desc(smem_u32(sK));
#pragma unroll
        for (int k = 0; k < kAttD / 16; ++k) umma(tmem_base, qd + 2 * k, kd + 2 * k, idesc, k > 0 ? 1u : 0u);
        umma_commit(bar_s);
        ok = mbar_wait(bar_p, 0) && mbar_wait(bar_v, 0);
      }
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t idesc2 = make_idesc(bf16, kAttD, 0, 1);           // A = P K-major, B = V MN-major, N = 64
        const uint32_t v_addr = smem_u32(sV);
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          const uint64_t pd = make_desc(smem_u32(sP + s * kTileBytes));
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // keys 64 s + 16 k .. +15: 16 rows of 128 bytes further down the V tile
            const uint64_t vd = make_desc_mn(v_addr + (uint32_t)(s * 64 + k * 16) * 128u);
            umma(tmem_base + 128, pd + 2 * k, vd, idesc2, (s > 0 || k > 0) ? 1u : 0u);
          }
        }
        umma_commit(bar_o);
      } else {
        *abort_flag = 1;
      }
    }
  } else {
    // softmax / epilogue: thread = query row
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    bool ok = mbar_wait(bar_s, 0);
    if (!ok) *abort_flag = 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const float sc = p.scale * 1.4426950408889634f;       // scores in log2 units
    float m = -INFINITY;
    if (ok) {
#pragma unroll 1
      for (int c0 = 0; c0 < kAttT; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(lane_addr + (uint32_t)c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 32; ++j) m = fmaxf(m, __uint_as_float(r[j]) * sc + kbias[c0 + j]);
      }
    }
    float sum = 0.f;
    const float mm = (m == -INFINITY) ? 0.f : m;           // a fully masked row produces zeros, not NaN
    if (ok) {
      const uint32_t drop_base = ((uint32_t)blockIdx.x * kAttT + (uint32_t)row) * kAttT;
      const uint32_t seed = p.drop_threshold ? *p.seed : 0u;
#pragma unroll 1
      for (int c0 = 0; c0 < kAttT; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(lane_addr + (uint32_t)c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        float pv[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float e = exp2f(__uint_as_float(r[j]) * sc + kbias[c0 + j] - mm);
          sum += e;
          float keep = 1.f;
          if (p.drop_threshold) keep = att_hash(seed, drop_base + (uint32_t)(c0 + j)) >= p.drop_threshold ? p.keep_scale : 0.f;
          pv[j] = e * keep;
        }
        uint8_t* tile = sP + (c0 >> 6) * kTileBytes;
#pragma unroll
        for (int v = 0; v < 4; ++v) store8_swz<T>(tile, row, ((c0 & 63) >> 3) + v, pv + v * 8);
      }
    }
    fence_async_smem();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_p);
    ok = ok && mbar_wait(bar_o, 0);
    if (!ok) *abort_flag = 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok && !*abort_flag) {
      const float inv = sum > 0.f ? 1.f / sum : 0.f;
      T* orow = static_cast<T*>(p.out) + ((int64_t)b * p.T + row) * p.C + h * kAttD;
#pragma unroll 1
      for (int c0 = 0; c0 < kAttD; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(lane_addr + (uint32_t)(128 + c0), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < p.T) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            Vec16<T> o;
#pragma unroll
            for (int j = 0; j < 8; ++j) o.v[j] = Cvt<T>::from_f(__uint_as_float(r[v * 8 + j]) * inv);
            st16(orow + c0 + v * 8, o);
          }
        }
      }
      if (row < p.T && p.lse) p.lse[((int64_t)b * p.heads + h) * p.T + row] = (mm + log2f(fmaxf(sum, 1e-30f))) * 0.6931471805599453f;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) {
    // wait (bounded) for the bulk copies that may still be in flight before the shared memory is released
    mbar_wait(bar_qk, 0);
    mbar_wait(bar_v, 0);
    if (p.error_flag) atomicExch(p.error_flag, 1);
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------ backward
// shared memory: Q | K | V | dO | P~ (2 stages) | dS (2 stages), key bias, barriers.
// TMEM columns: S [0,128)  dP [128,256)  dV [256,320)  dQ [320,384)  dK [384,448).
constexpr uint32_t kBwdSmem = 8 * kTileBytes + 128 * 4 + 1024 + 256;

template <typename T>
__global__ void __launch_bounds__(kAttThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_do, const AttnParams p,
                int bf16) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kTileBytes;
  uint8_t* sV = smem + 2 * kTileBytes;
  uint8_t* sDO = smem + 3 * kTileBytes;
  uint8_t* sPt = smem + 4 * kTileBytes;                // P after dropout, two key stages
  uint8_t* sDS = smem + 6 * kTileBytes;                // dS, two key stages
  float* kbias = reinterpret_cast<float*>(smem + 8 * kTileBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(kbias + 128);
  uint64_t* bar_qk = bars, *bar_vdo = bars + 1, *bar_s = bars + 2, *bar_dp = bars + 3, *bar_pd = bars + 4, *bar_out = bars + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x / p.heads, h = blockIdx.x % p.heads;
  constexpr uint32_t kTmemCols = 512;

  if (threadIdx.x == 0) {
    mbar_init(bar_qk, 1); mbar_init(bar_vdo, 1); mbar_init(bar_s, 1); mbar_init(bar_dp, 1); mbar_init(bar_pd, 4);
    mbar_init(bar_out, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (threadIdx.x >= 64 && threadIdx.x < 192) {
    const int k = threadIdx.x - 64;
    bool valid = k < p.T;
    if (valid && p.mask) valid = static_cast<const float*>(p.mask)[(int64_t)b * p.T + k] != 0.f;
    kbias[k] = valid ? 0.f : -INFINITY;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar_qk, 2 * kTileBytes);
      tma_load_3d(sQ, &map_qkv, h * kAttD, 0, b, bar_qk);
      tma_load_3d(sK, &map_qkv, p.C + h * kAttD, 0, b, bar_qk);
      mbar_expect_tx(bar_vdo, 2 * kTileBytes);
      tma_load_3d(sV, &map_qkv, 2 * p.C + h * kAttD, 0, b, bar_vdo);
      tma_load_3d(sDO, &map_do, h * kAttD, 0, b, bar_vdo);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(bar_qk, 0);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t idesc = make_idesc(bf16, 128, 0, 0);
        const uint64_t qd = make_desc(smem_u32(sQ)), kd = make_desc(smem_u32(sK));
#pragma unroll
        for (int k = 0; k < 4; ++k) umma(tmem_base, qd + 2 * k, kd + 2 * k, idesc, k > 0 ? 1u : 0u);      // S = Q Kt
        umma_commit(bar_s);
        ok = mbar_wait(bar_vdo, 0);
      }
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t idesc = make_idesc(bf16, 128, 0, 0);
        const uint64_t dd = make_desc(smem_u32(sDO)), vd = make_desc(smem_u32(sV));
#pragma unroll
        for (int k = 0; k < 4; ++k) umma(tmem_base + 128, dd + 2 * k, vd + 2 * k, idesc, k > 0 ? 1u : 0u);  // dP = dO Vt
        umma_commit(bar_dp);
        ok = mbar_wait(bar_pd, 0);
      }
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t pt = smem_u32(sPt), ds = smem_u32(sDS), qa = smem_u32(sQ), ka = smem_u32(sK), doa = smem_u32(sDO);
        const uint32_t id_tt = make_idesc(bf16, kAttD, 1, 1);     // A MN-major (transposed view), B MN-major, N = 64
        const uint32_t id_nt = make_idesc(bf16, kAttD, 0, 1);     // A K-major, B MN-major
        // dV[key, d] = sum_q P~[q, key] dO[q, d]: contraction over the 128 query rows, 16 at a time
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma(tmem_base + 256, make_desc_mn(pt + k * 2048u, kTileBytes), make_desc_mn(doa + k * 2048u), id_tt, k > 0 ? 1u : 0u);
        // dQ[q, d] = sum_key dS[q, key] K[key, d]
#pragma unroll
        for (int s2 = 0; s2 < 2; ++s2) {
          const uint64_t dsd = make_desc(ds + s2 * kTileBytes);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma(tmem_base + 320, dsd + 2 * k, make_desc_mn(ka + (uint32_t)(s2 * 64 + k * 16) * 128u), id_nt,
                 (s2 > 0 || k > 0) ? 1u : 0u);
        }
        // dK[key, d] = sum_q dS[q, key] Q[q, d]
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma(tmem_base + 384, make_desc_mn(ds + k * 2048u, kTileBytes), make_desc_mn(qa + k * 2048u), id_tt, k > 0 ? 1u : 0u);
        umma_commit(bar_out);
      } else {
        *abort_flag = 1;
      }
    }
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const bool live = row < p.T;
    // D = rowsum(dO * O) and the row's log-sum-exp, fetched while the tensor cores work
    float Dr = 0.f, lse2 = 0.f;
    if (live) {
      const T* orow = static_cast<const T*>(p.o) + ((int64_t)b * p.T + row) * p.C + h * kAttD;
      const T* drow = static_cast<const T*>(p.dout) + ((int64_t)b * p.T + row) * p.C + h * kAttD;
#pragma unroll
      for (int v = 0; v < kAttD / 8; ++v) {
        const Vec16<T> a = ld16(orow + v * 8), g = ld16(drow + v * 8);
#pragma unroll
        for (int j = 0; j < 8; ++j) Dr += Cvt<T>::to_f(a.v[j]) * Cvt<T>::to_f(g.v[j]);
      }
      lse2 = p.lse[((int64_t)b * p.heads + h) * p.T + row] * 1.4426950408889634f;
    }
    bool ok = mbar_wait(bar_s, 0) && mbar_wait(bar_dp, 0);
    if (!ok) *abort_flag = 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
      const float sc = p.scale * 1.4426950408889634f;
      const uint32_t drop_base = ((uint32_t)blockIdx.x * kAttT + (uint32_t)row) * kAttT;
      const uint32_t seed = p.drop_threshold ? *p.seed : 0u;
#pragma unroll 1
      for (int c0 = 0; c0 < kAttT; c0 += 32) {
        uint32_t rs[32], rd[32];
        tmem_ld32(lane_addr + (uint32_t)c0, rs);
        tmem_ld32(lane_addr + (uint32_t)(128 + c0), rd);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        float pt[32], dsv[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float e = live ? exp2f(__uint_as_float(rs[j]) * sc + kbias[c0 + j] - lse2) : 0.f;
          float keep = 1.f;
          if (p.drop_threshold) keep = att_hash(seed, drop_base + (uint32_t)(c0 + j)) >= p.drop_threshold ? p.keep_scale : 0.f;
          pt[j] = e * keep;
          dsv[j] = e * (__uint_as_float(rd[j]) * keep - Dr) * p.scale;
        }
        uint8_t* t1 = sPt + (c0 >> 6) * kTileBytes;
        uint8_t* t2 = sDS + (c0 >> 6) * kTileBytes;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          store8_swz<T>(t1, row, ((c0 & 63) >> 3) + v, pt + v * 8);
          store8_swz<T>(t2, row, ((c0 & 63) >> 3) + v, dsv + v * 8);
        }
      }
    }
    fence_async_smem();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_pd);
    ok = ok && mbar_wait(bar_out, 0);
    if (!ok) *abort_flag = 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok && !*abort_flag) {
      // accumulator rows: dQ row = query, dK / dV row = key; all three go to the packed gradient tensor
      T* base = static_cast<T*>(p.dqkv) + ((int64_t)b * p.T + row) * 3 * p.C + h * kAttD;
#pragma unroll 1
      for (int part = 0; part < 3; ++part) {
        const uint32_t col = part == 0 ? 320u : (part == 1 ? 384u : 256u);     // dQ, dK, dV
        T* dst = base + (int64_t)part * p.C;
#pragma unroll 1
        for (int c0 = 0; c0 < kAttD; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(lane_addr + col + (uint32_t)c0, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (live) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              Vec16<T> o;
#pragma unroll
              for (int j = 0; j < 8; ++j) o.v[j] = Cvt<T>::from_f(__uint_as_float(r[v * 8 + j]));
              st16(dst + c0 + v * 8, o);
            }
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) {
    mbar_wait(bar_qk, 0);
    mbar_wait(bar_vdo, 0);
    if (p.error_flag) atomicExch(p.error_flag, 1);
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

#include "attention_long.inl"

// 3-D tensor map over a packed [N, T, W] half tensor: box = 64 columns x 128 rows x 1 sample, 128-byte swizzle;
// rows beyond T are filled with zeros.
static int make_map_ntc(CUtensorMap* map, const void* base, int bf16, int64_t N, int64_t T, int64_t W) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  cuuint64_t dims[3] = {(cuuint64_t)W, (cuuint64_t)T, (cuuint64_t)N};
  cuuint64_t strides[2] = {(cuuint64_t)W * 2, (cuuint64_t)T * W * 2};
  cuuint32_t box[3] = {(cuuint32_t)kAttD, (cuuint32_t)kAttT, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult rc = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base),
                   dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? 0 : -(1000 + (int)rc);
}

static bool attn_shape_ok(int N, int T, int C, int heads) {
  return N >= 1 && T >= 1 && T <= kAttLongMaxT && heads >= 1 && C == heads * kAttD;
}

}  // namespace mxb

using namespace mxb;

// 1 when the fused kernels take the shape: head size 64, T up to 1024 (one tile up to 128, the streaming kernels beyond).
MXB_EXPORT int mxb_attn_supported(int T, int C, int heads) { return attn_shape_ok(1, T, C, heads) ? 1 : 0; }

// Number of fp32 elements of the dQ workspace the backward call needs (0 for T <= 128).
MXB_EXPORT long long mxb_attn_backward_workspace(int N, int T, int C) {
  if (T <= kAttT) return 0;
  return (long long)((T + kAttT - 1) / kAttT) * N * T * C;
}

// qkv: [N, T, 3C] (fp16 / bf16), mask: [N, T] float or null, out: [N, T, C], lse: [N, heads, T] floats.
// dropout: probability of dropping an attention weight (0 = none); `seed`: device word that selects the pattern.
MXB_EXPORT int mxb_attn_forward(int dtype, const void* qkv, const float* mask, void* out, float* lse, int N, int T, int C,
                                int heads, float dropout, const uint32_t* seed, int* error_flag, void* stream) {
  if (dtype != kF16 && dtype != kBF16) return -1;
  if (!attn_shape_ok(N, T, C, heads) || dropout < 0.f || dropout >= 1.f || (dropout > 0.f && !seed)) return -2;
  if (((uintptr_t)qkv % 16) || ((uintptr_t)out % 16)) return -3;
  const int bf16 = dtype == kBF16;
  CUtensorMap map;
  int rc = make_map_ntc(&map, qkv, bf16, N, T, 3 * (int64_t)C);
  if (rc) return rc;
  AttnParams p{};
  p.mask = mask; p.out = out; p.lse = lse; p.N = N; p.T = T; p.C = C; p.heads = heads;
  p.scale = 1.f / sqrtf((float)kAttD);
  p.keep_scale = 1.f / (1.f - dropout);
  p.drop_threshold = dropout > 0.f ? (uint32_t)((double)dropout * 4294967296.0) : 0u;
  p.seed = seed; p.error_flag = error_flag;
  cudaStream_t st = (cudaStream_t)stream;
  static unsigned long long attr_seen = 0;
  if (first_on_device(&attr_seen)) {
    cudaFuncSetAttribute(attn_fwd_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwdSmem);
    cudaFuncSetAttribute(attn_fwd_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwdSmem);
  }
  if (T > kAttT) {
    static unsigned long long long_seen = 0;
    if (first_on_device(&long_seen)) {
      cudaFuncSetAttribute(attn_fwd_long_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwdLongSmem);
      cudaFuncSetAttribute(attn_fwd_long_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwdLongSmem);
    }
    const int64_t grid = (int64_t)N * heads * ((T + kAttT - 1) / kAttT);
    if (grid > 0x7fffffff) return -2;
    if (bf16) attn_fwd_long_kernel<__nv_bfloat16><<<(unsigned)grid, kAttThreads, kFwdLongSmem, st>>>(map, p, 1);
    else attn_fwd_long_kernel<__half><<<(unsigned)grid, kAttThreads, kFwdLongSmem, st>>>(map, p, 0);
    return (int)cudaGetLastError();
  }
  if (bf16) attn_fwd_kernel<__nv_bfloat16><<<N * heads, kAttThreads, kFwdSmem, st>>>(map, p, 1);
  else attn_fwd_kernel<__half><<<N * heads, kAttThreads, kFwdSmem, st>>>(map, p, 0);
  return (int)cudaGetLastError();
}

// dqkv: [N, T, 3C] receives dQ | dK | dV.  o, dout: [N, T, C]; lse from the forward call; same dropout and seed.
// `workspace`: mxb_attn_backward_workspace(N, T, C) floats (may be null when that is 0).
MXB_EXPORT int mxb_attn_backward(int dtype, const void* qkv, const float* mask, const void* o, const void* dout,
                                 const float* lse, void* dqkv, float* workspace, int N, int T, int C, int heads, float dropout,
                                 const uint32_t* seed, int* error_flag, void* stream) {
  if (dtype != kF16 && dtype != kBF16) return -1;
  if (!attn_shape_ok(N, T, C, heads) || dropout < 0.f || dropout >= 1.f || (dropout > 0.f && !seed)) return -2;
  if (((uintptr_t)qkv % 16) || ((uintptr_t)o % 16) || ((uintptr_t)dout % 16) || ((uintptr_t)dqkv % 16)) return -3;
  const int bf16 = dtype == kBF16;
  CUtensorMap map, map_do;
  int rc = make_map_ntc(&map, qkv, bf16, N, T, 3 * (int64_t)C);
  if (rc) return rc;
  rc = make_map_ntc(&map_do, dout, bf16, N, T, C);
  if (rc) return rc - 100000;
  AttnParams p{};
  p.mask = mask; p.lse = const_cast<float*>(lse); p.o = o; p.dout = dout; p.dqkv = dqkv;
  p.N = N; p.T = T; p.C = C; p.heads = heads;
  p.scale = 1.f / sqrtf((float)kAttD);
  p.keep_scale = 1.f / (1.f - dropout);
  p.drop_threshold = dropout > 0.f ? (uint32_t)((double)dropout * 4294967296.0) : 0u;
  p.seed = seed; p.error_flag = error_flag;
  cudaStream_t st = (cudaStream_t)stream;
  static unsigned long long attr_seen = 0;
  if (first_on_device(&attr_seen)) {
    cudaFuncSetAttribute(attn_bwd_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmem);
    cudaFuncSetAttribute(attn_bwd_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmem);
  }
  if (T > kAttT) {
    if (!workspace || ((uintptr_t)workspace % 16)) return -3;
    static unsigned long long long_seen = 0;
    if (first_on_device(&long_seen)) {
      cudaFuncSetAttribute(attn_bwd_long_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdLongSmem);
      cudaFuncSetAttribute(attn_bwd_long_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdLongSmem);
    }
    const int nblk = (T + kAttT - 1) / kAttT;
    const int64_t grid = (int64_t)N * heads * nblk;
    if (grid > 0x7fffffff) return -2;
    if (bf16) attn_bwd_long_kernel<__nv_bfloat16><<<(unsigned)grid, kAttThreads, kBwdLongSmem, st>>>(map, map_do, p, workspace, 1);
    else attn_bwd_long_kernel<__half><<<(unsigned)grid, kAttThreads, kBwdLongSmem, st>>>(map, map_do, p, workspace, 0);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    const int64_t rows = (int64_t)N * T, vecs = rows * (C / 8);
    const int fgrid = (int)((vecs + 255) / 256 < 148 * 16 ? (vecs + 255) / 256 : 148 * 16);
    if (bf16) attn_dq_finish_kernel<__nv_bfloat16><<<fgrid, 256, 0, st>>>(workspace, static_cast<__nv_bfloat16*>(dqkv), nblk, rows, C);
    else attn_dq_finish_kernel<__half><<<fgrid, 256, 0, st>>>(workspace, static_cast<__half*>(dqkv), nblk, rows, C);
    return (int)cudaGetLastError();
  }
  if (bf16) attn_bwd_kernel<__nv_bfloat16><<<N * heads, kAttThreads, kBwdSmem, st>>>(map, map_do, p, 1);
  else attn_bwd_kernel<__half><<<N * heads, kAttThreads, kBwdSmem, st>>>(map, map_do, p, 0);
  return (int)cudaGetLastError();
}

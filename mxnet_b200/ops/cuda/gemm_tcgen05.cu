// Dense GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) fed by TMA, for sm_100a.
//
//   D[M, N] = act( op(A) · op(B) + bias[N] )        A, B, D: fp16 or bf16, accumulation in fp32
//
// Each operand is either "K-major" (A stored [M, K], B stored [N, K]: the contraction axis is contiguous) or
// "MN-major" (A stored [K, M], B stored [K, N]).  The four combinations cover the forward product of a
// FullyConnected layer (K, K), its data gradient dY·W (K, MN), its weight gradient dYᵀ·X (MN, MN) and a plain
// row-major matmul A·B (K, MN) without any transposed copy.
//
// This is the contraction behind FullyConnected / dot / batch_dot and 1x1 NHWC convolutions; the
// reference sends all of them to cuBLAS (src/operator/linalg_impl.h: cublasGemmEx, pseudo-fp16 with fp32
// accumulation) followed by a separate add_bias_kernel (src/operator/nn/fully_connected-inl.h:165-367).
//
// Persistent, warp-specialised kernel: one CTA per SM walks output tiles of 128 x BN (BN = 64, 128 or 256).
//   warp 0     : TMA producer.  One elected lane issues cp.async.bulk.tensor.2d loads of a 128x64 A tile and a
//                BNx64 B tile per k-step into a shared-memory ring (128-byte swizzle); completion is signalled
//                on an mbarrier with the transaction byte count.  It runs ahead across tile boundaries, so the
//                ring is already full of the next tile's operands when the tensor cores finish the current one.
//   warp 1     : MMA issuer.  One elected lane issues four tcgen05.mma (M128 x N(BN) x K16, kind::f16) per k-step
//                from shared-memory matrix descriptors into one of TWO TMEM accumulators (128 lanes x BN fp32
//                columns each) and hands each ring stage back to the producer with tcgen05.commit.
//   warps 2..5 : epilogue.  They drain accumulator `t & 1` with tcgen05.ld (32 columns at a time), add the bias,
//                apply ReLU/GELU, convert and store, while the MMA warp already fills the other accumulator.
// No cluster features and no multicast loads are used, so the same binary runs in multi-GPU jobs.
// Every mbarrier wait is bounded; on expiry the CTA raises an error flag for the host, every role leaves its
// loop, copies still in flight are waited for (bounded), the TMEM columns are freed and the CTA exits.
#include "tcgen05.cuh"

namespace mxb {

constexpr int BM = 128, BK = 64, UMMA_K = 16;
// kernel selection: 0 = per shape, 1 = always the single-CTA kernel, 2 = the CTA-pair kernel wherever it applies
static int g_gemm_variant = 0;
static int g_gemm_streamk = 1;      // 0: never cut a last round of tiles by k-steps
constexpr int kGemmThreads = 192;
constexpr uint32_t A_BYTES = BM * BK * 2;
constexpr int kMaxStages = 8;

// ring depth that fits the 227 KB shared-memory budget for a given tile width
template <int BN> struct TileCfg {
  static constexpr uint32_t B_BYTES = BN * BK * 2;
  static constexpr int STAGES = BN == 256 ? 4 : (BN == 192 ? 5 : (BN == 128 ? 6 : 8));
  // TMEM columns between the two accumulators and the (power-of-two) allocation that holds both
  static constexpr int ACC_STRIDE = BN == 192 ? 256 : BN;
  static constexpr uint32_t TMEM_COLS = 2 * ACC_STRIDE < 32 ? 32 : 2 * ACC_STRIDE;
  static constexpr uint32_t STG_BYTES = 4 * 4096;   // per epilogue warp: two staging tiles of 32 rows x 64 bytes for the TMA stores
  static constexpr uint32_t SMEM_BYTES = STAGES * (A_BYTES + B_BYTES) + STG_BYTES + 1024 /*alignment slack*/ + 512 /*barriers*/;
};

enum Act { kActNone = 0, kActRelu = 1, kActGelu = 2 };

__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.f + erf_fast(x * 0.70710678118654752f)); }

// fp32 slot of a stream-K tile: [BN / 32 column chunks][8 float4 per chunk][128 rows] float4, so that the 32 lanes of a
// warp (32 consecutive rows) touch 512 contiguous bytes per access.
__device__ __forceinline__ float4* sk_slot_ptr(float* slot, int c0, int v, int row_in_tile) {
  return reinterpret_cast<float4*>(slot) + ((size_t)((c0 >> 5) * 8 + v) * 128 + (size_t)row_in_tile);
}

// Epilogue of one warp: drains 32 accumulator rows (TMEM lanes) by BN columns starting at TMEM address `taddr`, adds
// the bias, applies the activation and stores rows [row0, row0 + 32) x columns [tile_col0, tile_col0 + BN) of D, either
// through the copy engine (32 x 32 blocks staged in `stg`; `zb` = matrix of a batch, D is then that matrix's base for the
// per-thread path) or with per-thread stores.
// Stream-K pieces: with `slot` set, the fp32 partial products of this k-range are stored into that slot (this warp's
// rows at `part_row0`) and nothing else is written; gemm_sk_finish_kernel adds the pieces of a tile up afterwards.
template <typename T, int BN>
__device__ __forceinline__ void drain_quarter(uint32_t taddr, uint8_t* stg, const CUtensorMap* map_d, int use_tma_store,
                                              T* __restrict__ D, const T* __restrict__ bias, int M, int N, int ldd, int act,
                                              int row0, int tile_col0, int lane, int zb, float* __restrict__ slot = nullptr,
                                              int part_row0 = 0) {
  const int row = row0 + lane;
  const bool bias_vec = bias != nullptr && ((reinterpret_cast<uintptr_t>(bias) & 15) == 0);
  const bool row_vec = (ldd % 8) == 0;
  uint32_t r[32];
  tmem_ld32(taddr, r);
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += 32) {
    const int col0 = tile_col0 + c0;
    const bool full_cols = col0 + 32 <= N;
    // bias of these 32 columns first, so its latency overlaps the fetch (registers only: every index
    // below is a compile-time constant after unrolling)
    float bv[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) bv[j] = 0.f;
    if (slot == nullptr && bias != nullptr && col0 < N) {
      if (bias_vec && full_cols) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const Vec16<T> b = ld16(bias + col0 + v * 8);
#pragma unroll
          for (int j = 0; j < 8; ++j) bv[v * 8 + j] = Cvt<T>::to_f(b.v[j]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < N) bv[j] = Cvt<T>::to_f(bias[col0 + j]);
      }
    }
    tmem_wait_ld32(r);
    if (slot != nullptr) {
#pragma unroll
      for (int v = 0; v < 8; ++v)
        __stcg(sk_slot_ptr(slot, c0, v, part_row0 + lane), make_float4(__uint_as_float(r[v * 4]), __uint_as_float(r[v * 4 + 1]),
                                                                       __uint_as_float(r[v * 4 + 2]), __uint_as_float(r[v * 4 + 3])));
      if (c0 + 32 < BN) tmem_ld32(taddr + (uint32_t)(c0 + 32), r);
      continue;
    }
    float f[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      float x = __uint_as_float(r[j]) + bv[j];
      if (act == kActRelu) x = fmaxf(x, 0.f);
      else if (act == kActGelu) x = gelu_erf(x);
      f[j] = x;
    }
    // the next 32 columns travel from TMEM while these are converted and stored
    if (c0 + 32 < BN) tmem_ld32(taddr + (uint32_t)(c0 + 32), r);
    if (use_tma_store) {
      // rows as four 16-byte pieces in the swizzled layout of the store's tensor map; one bulk store per 32 x 32
      // block (rows and columns outside the matrix are clipped by the copy engine)
      // two staging tiles alternate (every tile width is an even number of 32-column blocks): the store issued two blocks
      // ago has released the tile reused now, the previous one may still be reading its own
      uint8_t* sb = stg + ((c0 >> 5) & 1) * 2048;
      if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      __syncwarp();
      if (col0 < N && row0 < M) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          Vec16<T> o;
#pragma unroll
          for (int j = 0; j < 8; ++j) o.v[j] = Cvt<T>::from_f(f[v * 8 + j]);
          st16(reinterpret_cast<T*>(sb + lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4)), o);
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_3d(map_d, sb, col0, row0, zb);
          tma_store_commit();
        }
      } else if (lane == 0) {
        tma_store_commit();            // an empty group keeps the count of groups per block, which the wait above relies on
      }
    } else if (row < M && col0 < N) {
      T* drow = D + (size_t)row * ldd + col0;
      if (full_cols && row_vec) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          Vec16<T> o;
#pragma unroll
          for (int j = 0; j < 8; ++j) o.v[j] = Cvt<T>::from_f(f[v * 8 + j]);
          st16(drow + v * 8, o);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < N) drow[j] = Cvt<T>::from_f(f[j]);
      }
    }
  }
}

// The work of one CTA of the persistent grid: first whole tiles (tile = blockIdx.x, + gridDim.x, ... below `full_tiles`),
// then its share of the stream-K region: the `sk_tiles` tiles after `full_tiles` are a sequence of sk_tiles * num_k
// k-steps that is cut into `sk_ctas` contiguous, equally long ranges, so a CTA computes the end of one tile, possibly
// whole tiles, and the beginning of another.  A piece that is not a whole tile is `partial`: its fp32 result goes to
// slot 0 of the CTA if the tile is the first one the CTA touches, else to slot 1 (a CTA has at most two partial pieces:
// the end of its first tile and the beginning of its last).  The three roles walk the same sequence.
struct UnitIter {
  int tile, k0, k1, sk_tile, slot;
  bool partial;
  int next_full, full_tiles, num_k, first_t;
  uint32_t a, b;
  __device__ __forceinline__ void init(int full_tiles_, int sk_tiles, int sk_ctas, int num_k_) {
    next_full = blockIdx.x;
    full_tiles = full_tiles_;
    num_k = num_k_;
    a = b = 0;
    if (sk_tiles > 0 && (int)blockIdx.x < sk_ctas) {
      const uint64_t total = (uint64_t)sk_tiles * (uint64_t)num_k;
      a = (uint32_t)((uint64_t)blockIdx.x * total / (uint64_t)sk_ctas);
      b = (uint32_t)((uint64_t)(blockIdx.x + 1) * total / (uint64_t)sk_ctas);
    }
    first_t = (int)(a / (uint32_t)num_k);
  }
  __device__ __forceinline__ bool next() {
    if (next_full < full_tiles) {
      tile = next_full;
      next_full += gridDim.x;
      k0 = 0; k1 = num_k; partial = false; sk_tile = -1; slot = 0;
      return true;
    }
    if (a < b) {
      const int t = (int)(a / (uint32_t)num_k);
      k0 = (int)(a - (uint32_t)t * (uint32_t)num_k);
      int len = (int)(b - a);
      if (len > num_k - k0) len = num_k - k0;
      k1 = k0 + len;
      tile = full_tiles + t;
      sk_tile = t;
      partial = len != num_k;
      slot = t == first_t ? 0 : 1;
      a += (uint32_t)len;
      return true;
    }
    return false;
  }
};

template <typename T, int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_d, int use_tma_store, T* __restrict__ D, const T* __restrict__ bias, int M,
               int N, int K, int ldd, int act, int bf16, int a_mn, int b_mn, const FastDiv fd_tiles_m,
               int full_tiles, int sk_tiles, int sk_ctas, float* __restrict__ sk_ws, int a3d, int b3d,
               const FastDiv fd_tiles_batch, long long stride_d, int* __restrict__ error_flag) {
  using Cfg = TileCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr uint32_t B_BYTES = Cfg::B_BYTES;
  extern __shared__ uint8_t smem_raw[];
  // tiles need 1024-byte alignment for the 128-byte swizzle pattern
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  uint8_t* sStg = smem + STAGES * (A_BYTES + B_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * (A_BYTES + B_BYTES) + Cfg::STG_BYTES);
  uint64_t* full = bars;                        // [STAGES] producer -> MMA
  uint64_t* empty = bars + kMaxStages;          // [STAGES] MMA -> producer
  uint64_t* acc_full = bars + 2 * kMaxStages;   // [2] accumulator ready for the epilogue
  uint64_t* acc_empty = acc_full + 2;           // [2] accumulator drained by the epilogue
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* issued_it = abort_flag + 1;     // k-steps whose TMA loads were issued
  volatile int* consumed_it = abort_flag + 2;   // k-steps whose loads were observed complete by the MMA warp

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_k = (K + BK - 1) / BK;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  constexpr uint32_t kTmemCols = Cfg::TMEM_COLS;     // two accumulators; a power of two >= 32

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
    *abort_flag = 0;
    *issued_it = 0;
    *consumed_it = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // TMEM allocation is a warp-wide operation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  // Tile order: consecutive CTAs take consecutive row tiles of the same column tile, so the B (weight) tile is
  // shared through L2 by the CTAs that run at the same time and A is streamed once.
  // The two single-thread roles keep their per-k-step instruction count minimal (ring position and parity as running
  // counters, descriptors advanced by additions, progress counters written to shared memory only when a loop ends):
  // their issue time is what bounds narrow tiles.
  if (warp == 0) {
    if (lane == 0) {
      int it = 0, st = 0;
      uint32_t ph = 0;
      bool ok = true;
      UnitIter u;
      u.init(full_tiles, sk_tiles, sk_ctas, num_k);
      while (ok && !*abort_flag && u.next()) {
        uint32_t zb_u, in_batch, tile_n_u, tile_m_u;
        fd_divmod((uint32_t)u.tile, fd_tiles_batch, &zb_u, &in_batch);      // the outermost coordinate of every map: the matrix of a batch
        fd_divmod(in_batch, fd_tiles_m, &tile_n_u, &tile_m_u);
        const int tile_m = (int)tile_m_u, tile_n = (int)tile_n_u, zb = (int)zb_u;
        const int k0 = u.k0, k1 = u.k1;
        for (int kt = k0; kt < k1; ++kt) {
          if (!mbar_wait(&empty[st], ph ^ 1u)) { *abort_flag = 1; ok = false; break; }
          mbar_expect_tx(&full[st], A_BYTES + B_BYTES);
          if (!a_mn) {
            tma_load_3d(sA + st * A_BYTES, &map_a, kt * BK, tile_m * BM, zb, &full[st]);
          } else if (a3d) {
            // all 64-column chunks of the tile in one box {64 columns, 64 k-rows, BM/64 chunks}
            tma_load_4d(sA + st * A_BYTES, &map_a, 0, kt * BK, tile_m * (BM / 64), zb, &full[st]);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_3d(sA + st * A_BYTES + c * kMnChunkBytes, &map_a, tile_m * BM + c * 64, kt * BK, zb, &full[st]);
          }
          if (!b_mn) {
            tma_load_3d(sB + st * B_BYTES, &map_b, kt * BK, tile_n * BN, zb, &full[st]);
          } else if (b3d) {
            tma_load_4d(sB + st * B_BYTES, &map_b, 0, kt * BK, tile_n * (BN / 64), zb, &full[st]);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_3d(sB + st * B_BYTES + c * kMnChunkBytes, &map_b, tile_n * BN + c * 64, kt * BK, zb, &full[st]);
          }
          ++it;
          if (++st == STAGES) { st = 0; ph ^= 1u; }
        }
      }
      *issued_it = it;
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(bf16, BN, a_mn, b_mn);
      // one UMMA_K step (16 elements of K): 32 bytes inside the swizzle atom for a K-major operand, 16 k-rows of
      // 128 bytes for an MN-major operand; in units of the descriptor's 16-byte address field
      const uint64_t a_step = a_mn ? (16 * 128) >> 4 : 2, b_step = b_mn ? (16 * 128) >> 4 : 2;
      // descriptors of stage 0; the start-address field (16-byte units, 14 bits) takes plain additions
      const uint64_t adesc0 = a_mn ? make_desc_mn(smem_u32(sA)) : make_desc(smem_u32(sA));
      const uint64_t bdesc0 = b_mn ? make_desc_mn(smem_u32(sB)) : make_desc(smem_u32(sB));
      int it = 0, st = 0, t = 0;
      uint32_t ph = 0;
      bool ok = true;
      UnitIter u;
      u.init(full_tiles, sk_tiles, sk_ctas, num_k);
      for (; ok && !*abort_flag && u.next(); ++t) {
        const int k0 = u.k0, k1 = u.k1;
        const int buf = t & 1;
        // wait until the epilogue has drained this accumulator (its first use passes immediately)
        if (!mbar_wait(&acc_empty[buf], (((uint32_t)t >> 1) & 1u) ^ 1u)) { *abort_flag = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * Cfg::ACC_STRIDE);
        for (int kt = k0; kt < k1; ++kt) {
          if (!mbar_wait(&full[st], ph)) { *abort_flag = 1; ok = false; break; }
          const uint64_t adesc = adesc0 + (uint64_t)(st * (int)(A_BYTES >> 4));
          const uint64_t bdesc = bdesc0 + (uint64_t)(st * (int)(B_BYTES >> 4));
          umma(tmem_d, adesc, bdesc, idesc, kt > k0 ? 1u : 0u);
#pragma unroll
          for (int k = 1; k < BK / UMMA_K; ++k)
            umma(tmem_d, adesc + a_step * (uint64_t)k, bdesc + b_step * (uint64_t)k, idesc, 1u);
          umma_commit(&empty[st]);        // the stage is free once these MMAs have read it
          ++it;
          if (++st == STAGES) { st = 0; ph ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&acc_full[buf]);     // arrives when every MMA of this tile has completed
      }
      *consumed_it = it;
    }
  } else {
    // epilogue warps 2..5: TMEM lane quarter = warp index modulo 4
    const int q = warp & 3;
    uint8_t* stg = sStg + q * 4096;       // this warp's two staging tiles: 32 rows x 64 bytes each, 64-byte swizzle
    int t = 0;
    UnitIter u;
    u.init(full_tiles, sk_tiles, sk_ctas, num_k);
    for (; u.next(); ++t) {
      uint32_t zb_u, in_batch, tile_n_u, tile_m_u;
      fd_divmod((uint32_t)u.tile, fd_tiles_batch, &zb_u, &in_batch);
      fd_divmod(in_batch, fd_tiles_m, &tile_n_u, &tile_m_u);
      const int tile_m = (int)tile_m_u, tile_n = (int)tile_n_u, zb = (int)zb_u;
      T* Db = D + (long long)zb * stride_d;
      const int buf = t & 1;
      const bool ready = mbar_wait(&acc_full[buf], ((uint32_t)t >> 1) & 1u);
      if (!ready) *abort_flag = 1;
      if (!ready || *abort_flag) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * Cfg::ACC_STRIDE);
      const int row0 = tile_m * BM + q * 32, col0 = tile_n * BN;
      if (!u.partial) {
        drain_quarter<T, BN>(taddr, stg, &map_d, use_tma_store, Db, bias, M, N, ldd, act, row0, col0, lane, zb);
      } else {
        // A piece of a stream-K tile: store this warp's 32 rows of fp32 partial products into this CTA's slot; the
        // finishing kernel that follows on the stream adds the pieces of each tile in a fixed order.
        drain_quarter<T, BN>(taddr, stg, &map_d, use_tma_store, Db, bias, M, N, ldd, act, row0, col0, lane, zb,
                             sk_ws + ((size_t)blockIdx.x * 2 + (size_t)u.slot) * ((size_t)BM * BN), q * 32);
      }
      // this warp has finished reading the accumulator: let the MMA warp reuse it
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    if (lane == 0) tma_store_wait_all();    // the staging tile must outlive the last store
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) {
    // gave up somewhere: before the shared memory is released, wait (bounded) for bulk copies that were
    // issued but never consumed, so none is still in flight when the CTA exits
    for (int it = *consumed_it; it < *issued_it; ++it) mbar_wait(&full[it % STAGES], (uint32_t)(it / STAGES) & 1u);
    if (error_flag) atomicExch(error_flag, 1);
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// Second half of a stream-K product: adds up the pieces of every tile of the stream-K region (in CTA order, so the result
// does not depend on timing), applies bias and activation and writes D.  One CTA per tile and 32-column chunk, one thread
// per (float4 of the chunk, row): it reads the slots in the layout the GEMM epilogue wrote (consecutive rows contiguous),
// all pieces with independent loads so that their latencies overlap.
constexpr int kSkMaxPieces = 8;      // the plan cuts a tile into at most this many pieces
template <typename T>
__global__ void __launch_bounds__(1024)
gemm_sk_finish_kernel(const float* __restrict__ sk_ws, const T* __restrict__ bias, T* __restrict__ D, int M, int N, int ldd, int act,
                      int bn, int tiles_m, int full_tiles, int sk_tiles, int sk_ctas, int num_k, int tiles_per_batch,
                      long long stride_d) {
  __shared__ const float* piece[kSkMaxPieces];
  __shared__ int n_pieces;
  const int chunks = bn >> 5;
  const int t = blockIdx.x / chunks, chunk = blockIdx.x - t * chunks;
  if (threadIdx.x == 0) {
    const uint64_t total = (uint64_t)sk_tiles * (uint64_t)num_k, lo = (uint64_t)t * (uint64_t)num_k;
    const int c_lo = (int)(((lo + 1) * (uint64_t)sk_ctas - 1) / total);
    const int c_hi = (int)(((lo + (uint64_t)num_k) * (uint64_t)sk_ctas - 1) / total);
    int n = 0;
    if (c_hi > c_lo) {                              // otherwise one CTA computed the whole tile and wrote it itself
      for (int c = c_lo; c <= c_hi && n < kSkMaxPieces; ++c) {
        const int first_c = (int)(((uint64_t)c * total / (uint64_t)sk_ctas) / (uint64_t)num_k);
        piece[n++] = sk_ws + ((size_t)c * 2 + (t == first_c ? 0 : 1)) * ((size_t)BM * bn);
      }
    }
    n_pieces = n;
  }
  __syncthreads();
  const int n = n_pieces;
  if (n == 0) return;
  const int tile = full_tiles + t;
  const int zb = tile / tiles_per_batch, in_batch = tile - zb * tiles_per_batch;
  const int tile_m = in_batch % tiles_m, tile_n = in_batch / tiles_m;
  D += (long long)zb * stride_d;
  const int v = threadIdx.x >> 7, r = threadIdx.x & (BM - 1);
  const size_t off = (size_t)(chunk * 8 + v) * BM + r;
  float4 p[kSkMaxPieces];
#pragma unroll
  for (int c = 0; c < kSkMaxPieces; ++c)
    p[c] = c < n ? __ldcg(reinterpret_cast<const float4*>(piece[c]) + off) : make_float4(0.f, 0.f, 0.f, 0.f);
  float4 acc = p[0];
#pragma unroll
  for (int c = 1; c < kSkMaxPieces; ++c) { acc.x += p[c].x; acc.y += p[c].y; acc.z += p[c].z; acc.w += p[c].w; }
  const int row = tile_m * BM + r, col = tile_n * bn + chunk * 32 + v * 4;
  if (row >= M || col >= N) return;
  const float x[4] = {acc.x, acc.y, acc.z, acc.w};
  T out[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float y = x[j] + ((bias && col + j < N) ? Cvt<T>::to_f(bias[col + j]) : 0.f);
    if (act == kActRelu) y = fmaxf(y, 0.f);
    else if (act == kActGelu) y = gelu_erf(y);
    out[j] = Cvt<T>::from_f(y);
  }
  T* drow = D + (size_t)row * ldd + col;
  if (col + 4 <= N && (ldd & 3) == 0) {
    *reinterpret_cast<uint2*>(drow) = *reinterpret_cast<const uint2*>(out);      // col is a multiple of 4: 8-byte aligned
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (col + j < N) drow[j] = out[j];
  }
}

// ---- CTA-pair variant -------------------------------------------------------------------------------------------------
// Two CTAs on neighbouring SMs (a cluster of 2) compute one 256 x BN output tile with tcgen05.mma.cta_group::2.  Each CTA
// stages ITS 128 rows of A and ITS BN/2 rows of B per k-step (plain per-CTA tiled loads whose transaction bytes are
// counted on the leader's mbarrier), so a CTA moves (128 + BN/2) x 64 operands for a 128 x BN share of the output: a third
// fewer L2-to-SM bytes per FLOP than the single-CTA kernel at BN = 256, and half the MMA instructions per FLOP.  The
// leader's MMA thread issues for both; its commits arrive on the ring / accumulator barriers of both CTAs.  Each CTA's
// epilogue drains the 128 accumulator rows that live in its own tensor memory.
// Roles per CTA as in the kernel above.  The ring's `empty` barriers and the `acc_full` barriers exist in both CTAs
// (signalled by the leader's commits); `full` and `acc_empty` are the leader's (the partner's loads and epilogue warps
// signal them through shared::cluster addresses).
template <int BN> struct PairCfg {
  static constexpr int BNH = BN / 2;                 // rows of B staged by each CTA
  static constexpr uint32_t B_BYTES = BNH * BK * 2;
  static constexpr int STAGES = BN == 256 ? 6 : (BN == 192 ? 6 : 8);
  static constexpr int ACC_STRIDE = BN == 192 ? 256 : BN;
  static constexpr uint32_t TMEM_COLS = 2 * ACC_STRIDE;
  static constexpr uint32_t STG_BYTES = 4 * 4096;
  static constexpr uint32_t SMEM_BYTES = STAGES * (A_BYTES + B_BYTES) + STG_BYTES + 1024 + 512;
};
constexpr int BM2 = 256;     // rows of a pair's tile

template <typename T, int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_d, int use_tma_store, T* __restrict__ D, const T* __restrict__ bias, int M,
                 int N, int K, int ldd, int act, int bf16, int a_mn, int b_mn, const FastDiv fd_tiles_m, int a3d,
                 int b3d, int* __restrict__ error_flag) {
  using Cfg = PairCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int BNH = Cfg::BNH;
  constexpr uint32_t B_BYTES = Cfg::B_BYTES;
  extern __shared__ uint8_t smem_raw[];
  // the dynamic shared memory starts at the same offset in both CTAs, so the rounded-up tile addresses agree too
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  uint8_t* sStg = smem + STAGES * (A_BYTES + B_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * (A_BYTES + B_BYTES) + Cfg::STG_BYTES);
  uint64_t* full = bars;                        // [STAGES] leader only: both CTAs' loads of a stage have landed
  uint64_t* empty = bars + kMaxStages;          // [STAGES] each CTA: the pair's MMAs have read this stage
  uint64_t* acc_full = bars + 2 * kMaxStages;   // [2] each CTA: accumulator complete
  uint64_t* acc_empty = acc_full + 2;           // [2] leader only: drained by the 8 epilogue warps of the pair
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* issued_it = abort_flag + 1;
  volatile int* consumed_it = abort_flag + 2;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();      // 0 = leader
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_k = (K + BK - 1) / BK;
  const int tiles_m = (M + BM2 - 1) / BM2, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_units = num_tiles;      // whole tiles only: this kernel is chosen for outputs with many rounds of tiles
  constexpr uint32_t kTmemCols = Cfg::TMEM_COLS;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
    *abort_flag = 0;
    *issued_it = 0;
    *consumed_it = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // the same warp of both CTAs allocates the pair's tensor memory
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();      // the partner's barriers exist before anything signals them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      const uint32_t full_leader = mapa_u32(smem_u32(&full[0]), 0);
      int it = 0, st = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int unit = pair; unit < num_units && ok && !*abort_flag; unit += num_pairs) {
        uint32_t tile_n_u, tile_m_u;
        fd_divmod((uint32_t)unit, fd_tiles_m, &tile_n_u, &tile_m_u);
        const int row_a = (int)tile_m_u * BM2 + (int)rank * BM;      // this CTA's rows of A (= rows of D)
        const int row_b = (int)tile_n_u * BN + (int)rank * BNH;      // this CTA's rows of B (= columns of D)
        const int k0 = 0, k1 = num_k;
        for (int kt = k0; kt < k1; ++kt) {
          if (!mbar_wait(&empty[st], ph ^ 1u)) { *abort_flag = 1; ok = false; break; }
          const uint32_t fb = full_leader + (uint32_t)st * 8u;
          if (rank == 0) mbar_expect_tx(&full[st], 2u * (A_BYTES + B_BYTES));
          if (!a_mn) {
            tma_pair_load_3d(sA + st * A_BYTES, &map_a, kt * BK, row_a, 0, fb);
          } else if (a3d) {
            tma_pair_load_4d(sA + st * A_BYTES, &map_a, 0, kt * BK, row_a / 64, 0, fb);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_pair_load_3d(sA + st * A_BYTES + c * kMnChunkBytes, &map_a, row_a + c * 64, kt * BK, 0, fb);
          }
          if (!b_mn) {
            tma_pair_load_3d(sB + st * B_BYTES, &map_b, kt * BK, row_b, 0, fb);
          } else if (b3d) {
            tma_pair_load_4d(sB + st * B_BYTES, &map_b, 0, kt * BK, row_b / 64, 0, fb);
          } else {
#pragma unroll
            for (int c = 0; c < BNH / 64; ++c)
              tma_pair_load_3d(sB + st * B_BYTES + c * kMnChunkBytes, &map_b, row_b + c * 64, kt * BK, 0, fb);
          }
          ++it;
          if (++st == STAGES) { st = 0; ph ^= 1u; }
        }
      }
      *issued_it = it;
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = make_idesc(bf16, BN, a_mn, b_mn, BM2);
      const uint64_t a_step = a_mn ? (16 * 128) >> 4 : 2, b_step = b_mn ? (16 * 128) >> 4 : 2;
      const uint64_t adesc0 = a_mn ? make_desc_mn(smem_u32(sA)) : make_desc(smem_u32(sA));
      const uint64_t bdesc0 = b_mn ? make_desc_mn(smem_u32(sB)) : make_desc(smem_u32(sB));
      int it = 0, st = 0, t = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int unit = pair; unit < num_units && ok && !*abort_flag; unit += num_pairs, ++t) {
        const int k0 = 0, k1 = num_k;
        const int buf = t & 1;
        if (!mbar_wait(&acc_empty[buf], (((uint32_t)t >> 1) & 1u) ^ 1u)) { *abort_flag = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * Cfg::ACC_STRIDE);
        for (int kt = k0; kt < k1; ++kt) {
          if (!mbar_wait(&full[st], ph)) { *abort_flag = 1; ok = false; break; }
          const uint64_t adesc = adesc0 + (uint64_t)(st * (int)(A_BYTES >> 4));
          const uint64_t bdesc = bdesc0 + (uint64_t)(st * (int)(B_BYTES >> 4));
          umma_pair(tmem_d, adesc, bdesc, idesc, kt > k0 ? 1u : 0u);
#pragma unroll
          for (int k = 1; k < BK / UMMA_K; ++k)
            umma_pair(tmem_d, adesc + a_step * (uint64_t)k, bdesc + b_step * (uint64_t)k, idesc, 1u);
          umma_pair_commit(&empty[st], 3);      // the stage is free in both CTAs once these MMAs have read it
          ++it;
          if (++st == STAGES) { st = 0; ph ^= 1u; }
        }
        if (!ok) break;
        umma_pair_commit(&acc_full[buf], 3);    // both CTAs' epilogues: every MMA of this tile has completed
      }
      *consumed_it = it;
    }
  } else {
    const int q = warp & 3;
    uint8_t* stg = sStg + q * 4096;
    const uint32_t acc_empty_leader = mapa_u32(smem_u32(&acc_empty[0]), 0);
    int t = 0;
    for (int unit = pair; unit < num_units; unit += num_pairs, ++t) {
      uint32_t tile_n_u, tile_m_u;
      fd_divmod((uint32_t)unit, fd_tiles_m, &tile_n_u, &tile_m_u);
      const int buf = t & 1;
      const bool ready = mbar_wait(&acc_full[buf], ((uint32_t)t >> 1) & 1u);
      if (!ready) *abort_flag = 1;
      if (!ready || *abort_flag) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * Cfg::ACC_STRIDE);
      drain_quarter<T, BN>(taddr, stg, &map_d, use_tma_store, D, bias, M, N, ldd, act,
                           (int)tile_m_u * BM2 + (int)rank * BM + q * 32, (int)tile_n_u * BN, lane, 0);
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader + (uint32_t)buf * 8u);
    }
    if (lane == 0) tma_store_wait_all();
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  // Both CTAs have left their loops: nothing new is issued.  Neither may release its shared or tensor memory while the
  // other could still signal or read it, hence the cluster-wide barriers around the clean-up.
  cluster_sync_all();
  if (threadIdx.x == 0 && *abort_flag && error_flag) atomicExch(error_flag, 1);
  if (threadIdx.x == 0 && rank == 0) {
    // If either CTA gave up, wait (bounded) for the loads that were issued but never consumed: every stage completes
    // on the leader's `full` barrier only when both halves have landed.
    const int peer_abort = (int)ld_cluster_u32(mapa_u32(smem_u32((const void*)abort_flag), 1));
    if (*abort_flag || peer_abort) {
      int issued = *issued_it;
      const int peer_issued = (int)ld_cluster_u32(mapa_u32(smem_u32((const void*)issued_it), 1));
      if (peer_issued < issued) issued = peer_issued;      // a stage completes only if both CTAs loaded it
      for (int it = *consumed_it; it < issued; ++it)
        if (!mbar_wait(&full[it % STAGES], (uint32_t)(it / STAGES) & 1u)) break;
    }
  }
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// Every tensor map carries the batch as its outermost dimension (extent 1 for a plain product), `bstride` elements
// apart, so that one kernel serves single and batched products and a tile never reads across matrices.
//
// Row-major [rows, cols] half matrices, row pitch `ld` elements; box = box_rows x 64 columns, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, int bf16, int64_t rows, int64_t cols, int64_t ld, int box_rows,
                    int64_t batch, int64_t bstride) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)(batch > 1 ? bstride : rows * ld) * 2};
  cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult rc = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base),
                   dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? 0 : -11;
}

// MN-major operand: global tensor [K rows, MN columns] with row pitch `ld`; box = 64 k-rows x 64 columns.
static int make_map_mn(CUtensorMap* map, const void* base, int bf16, int64_t krows, int64_t mn, int64_t ld, int64_t batch,
                       int64_t bstride) {
  return make_map(map, base, bf16, krows, mn, ld, BK, batch, bstride);
}

// The same operand when MN is a multiple of 64: a view {64 columns, K rows, MN/64 chunks, batch} (chunk stride 128
// bytes) whose box {64, 64, chunks, 1} brings every chunk of a tile with one copy, chunk after chunk in shared memory.
static int make_map_mn3(CUtensorMap* map, const void* base, int bf16, int64_t krows, int64_t mn, int64_t ld, int chunks,
                        int64_t batch, int64_t bstride) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  cuuint64_t dims[4] = {64, (cuuint64_t)krows, (cuuint64_t)(mn / 64), (cuuint64_t)batch};
  cuuint64_t strides[3] = {(cuuint64_t)ld * 2, 128, (cuuint64_t)(batch > 1 ? bstride : krows * ld) * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)BK, (cuuint32_t)chunks, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult rc = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base),
                   dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? 0 : -11;
}

// Output matrices [batch][M, N] with row pitch ldd for the epilogue's stores: box = 32 rows x 32 columns, 64-byte swizzle.
static int make_map_store(CUtensorMap* map, const void* base, int bf16, int64_t rows, int64_t cols, int64_t ld, int64_t batch,
                          int64_t bstride) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)(batch > 1 ? bstride : rows * ld) * 2};
  cuuint32_t box[3] = {32, 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult rc = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base),
                   dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? 0 : -11;
}

// Stream-K plan for `tiles` output tiles of `num_k` k-steps on a grid of G CTAs: whole rounds of tiles are computed
// tile by tile; the tiles of a last, partial round (or all tiles, when there are fewer than CTAs) become the stream-K
// region when cutting their k-steps evenly over the CTAs is shorter than one more round.  A piece is at least 6 k-steps
// long and at least a sixth of a tile.
struct SkPlan {
  int full_tiles, sk_tiles, sk_ctas;
};
constexpr int kSkCombineCost = 16;      // writing, the second launch and the summation, in k-steps of a CTA
static SkPlan plan_streamk(int tiles, int num_k, int G, bool allowed) {
  SkPlan p = {tiles, 0, 0};
  const int rem = tiles % G;
  if (!allowed || num_k < 8 || rem == 0) return p;
  // Measured: with whole rounds before it, the stream-K remainder (fp32 pieces + the finishing launch, about 15 us on
  // 8192-row outputs) costs more than the idle SMs of a partial last round; it pays when there are fewer tiles than CTAs
  // (a weight gradient with a long contraction: 45.7 -> 37.6 us for 2304 x 768 x 8192).
  if (tiles >= G) return p;
  const long total = (long)rem * num_k;
  int min_per = (num_k + 5) / 6;
  if (min_per < 6) min_per = 6;
  long ctas = total / min_per;
  if (ctas > G) ctas = G;
  if (ctas < 2) return p;
  const long per = (total + ctas - 1) / ctas;
  if (per + kSkCombineCost >= num_k) return p;     // no shorter than one more round of whole tiles
  p.full_tiles = tiles - rem;
  p.sk_tiles = rem;
  p.sk_ctas = (int)ctas;
  return p;
}

// Workspace of the stream-K pieces: two slots of 128 x 256 floats per CTA of the grid (no initial contents required).
static size_t sk_workspace_bytes() { return (size_t)sm_count() * 2 * BM * 256 * sizeof(float); }

template <typename T, int BN>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& md, int use_tma_store, void* D,
                       const void* bias, int M, int N, int K, int ldd, int act, int bf16, int a_mn, int b_mn, float* ws, int a3d,
                       int b3d, int* error_flag, cudaStream_t st, int batch = 1, long long stride_d = 0) {
  using Cfg = TileCfg<BN>;
  static unsigned long long attr_seen = 0;
  if (first_on_device(&attr_seen)) {
    cudaError_t rc = cudaFuncSetAttribute(gemm_tn_kernel<T, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (rc != cudaSuccess) return (int)rc;
  }
  const int tiles_m = (M + BM - 1) / BM;
  const int tiles_batch = tiles_m * ((N + BN - 1) / BN);
  if ((long)tiles_batch * batch > 0x3fffffffL) return -2;
  const int tiles = tiles_batch * batch;
  const int num_k = (K + BK - 1) / BK;
  const int sms = sm_count();
  const SkPlan plan = plan_streamk(tiles, num_k, sms, g_gemm_streamk && ws != nullptr && sms <= 1024);
  int grid = tiles < sms ? tiles : sms;
  if (plan.sk_tiles > 0 && plan.full_tiles == 0) grid = plan.sk_ctas > tiles ? plan.sk_ctas : tiles;
  if (plan.sk_tiles > 0 && plan.full_tiles > 0) grid = sms;
  if (grid > sms) grid = sms;
  gemm_tn_kernel<T, BN><<<grid, kGemmThreads, Cfg::SMEM_BYTES, st>>>(ma, mb, md, use_tma_store, (T*)D, (const T*)bias, M, N, K, ldd,
                                                                     act, bf16, a_mn, b_mn, make_fastdiv((uint32_t)tiles_m),
                                                                     plan.full_tiles, plan.sk_tiles, plan.sk_ctas, ws, a3d, b3d,
                                                                     make_fastdiv((uint32_t)tiles_batch), stride_d, error_flag);
  if (plan.sk_tiles > 0)
    gemm_sk_finish_kernel<T><<<plan.sk_tiles * (BN / 32), 1024, 0, st>>>(ws, (const T*)bias, (T*)D, M, N, ldd, act, BN, tiles_m,
                                                                        plan.full_tiles, plan.sk_tiles, plan.sk_ctas, num_k,
                                                                        tiles_batch, stride_d);
  return (int)cudaGetLastError();
}

// Tile width of the single-CTA kernel: narrow outputs take the narrow tile; otherwise the width with the lowest
// rounds x (width + tile height), where a round is one tile on every CTA of the persistent grid: this avoids a
// mostly empty last column tile (N = 384 -> 2 x 192) and a mostly empty last round (M = 8192, N = 768: 256 tiles of 192
// columns take two rounds of 320 instead of two rounds of 384).  Outputs with fewer tiles than CTAs are cut by k-steps
// (stream-K plan), so their rounds are fractional.
static int pick_bn(int M, int N, int K, int batch = 1) {
  if (N <= 64) return 64;
  if (N <= 128) return 128;
  const long G = sm_count(), tm = (long)((M + BM - 1) / BM) * batch;
  // Few tiles and a short contraction (no stream-K): the product is one round whatever the width, and the round lasts as
  // long as one tile, so the narrowest width that still fits one round wins (64 x 768 x 768: 12 tiles of 64 columns
  // instead of 3 of 256).
  if (K <= 32 * BK && tm * ((N + 255) / 256) < G / 2) {
    for (int bn = 64; bn <= 192; bn += 64)
      if (tm * ((N + bn - 1) / bn) <= G) return bn;
  }
  int best = 256;
  double best_cost = 0;
  for (int bn = 256; bn >= 128; bn -= 64) {
    const long tiles = tm * ((N + bn - 1) / bn);
    // short products (under 24 k-steps) are bound by the epilogue, whose cost per output element does not depend on the
    // tile width: they only avoid the empty last column tile
    const double rounds = K < 24 * BK ? (double)tiles : tiles < G ? (double)tiles / (double)G : (double)((tiles + G - 1) / G);
    const double cost = rounds * (bn + BM);              // a tile's time follows the operand bytes it loads per k-step
    if (bn == 256 || cost < 0.9 * best_cost) { best = bn; best_cost = cost; }      // narrower only for a clear gain
  }
  return best;
}

// How many CTA pairs of the pair kernel can be resident at once (asked from the runtime once per tile width; the
// persistent grid is never larger).
template <typename T, int BN>
static int pair_capacity() {
  static int caps[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  int& cap = caps[dev & 63];           // the function attribute below is per device, so is the answer
  if (cap) return cap;
  using Cfg = PairCfg<BN>;
  if (cudaFuncSetAttribute(gemm_pair_kernel<T, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess) {
    cudaGetLastError();
    return cap = -1;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * sm_count());
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<T, BN>, &cfg) != cudaSuccess || n < 1) {
    cudaGetLastError();
    return cap = -1;
  }
  const int half = sm_count() / 2;
  return cap = n < half ? n : half;
}

template <typename T, int BN>
static int launch_gemm_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& md, int use_tma_store, void* D,
                            const void* bias, int M, int N, int K, int ldd, int act, int bf16, int a_mn, int b_mn, float* ws,
                            int a3d, int b3d, int* error_flag, cudaStream_t st) {
  using Cfg = PairCfg<BN>;
  const int pairs = pair_capacity<T, BN>();
  if (pairs < 1) return -20;
  const int tiles_m = (M + BM2 - 1) / BM2;
  const int tiles = tiles_m * ((N + BN - 1) / BN);
  const int grid = 2 * (tiles < pairs ? tiles : pairs);
  gemm_pair_kernel<T, BN><<<grid, kGemmThreads, Cfg::SMEM_BYTES, st>>>(ma, mb, md, use_tma_store, (T*)D, (const T*)bias, M, N, K, ldd,
                                                                       act, bf16, a_mn, b_mn, make_fastdiv((uint32_t)tiles_m), a3d,
                                                                       b3d, error_flag);
  return (int)cudaGetLastError();
}


// Tile width of the pair kernel for an M x N x K product, or 0 for the single-CTA kernel.  Measured: the pair kernel
// wins where the operands do not stay in L2 and the grid runs many rounds of tiles (8192^3: 1.25x the single-CTA kernel,
// 1.36x the library); on products that fit in L2 its longer load-to-MMA path (the partner's loads and the commits cross
// to the other SM) makes it slower, so those stay on the single-CTA kernel.  Width: among 256, 192 (K-major B only: each
// CTA would hold one and a half 64-column chunks of an MN-major B) and 128 the lowest rounds x (width + fixed cost).
static int pick_pair_bn(int M, int N, int K, int b_mn) {
  if (g_gemm_variant == 1 || M <= BM || N <= 64) return 0;
  const long pairs = sm_count() / 2, tm = (M + BM2 - 1) / BM2;
  if (g_gemm_variant != 2) {
    const double operand_bytes = ((double)M + (double)N) * (double)K * 2.0;
    if (operand_bytes < 96e6 || tm * ((N + 255) / 256) < 6 * pairs) return 0;
  }
  if (N <= 128) return 128;
  int best = 0;
  long best_cost = 0;
  for (int bn = 256; bn >= 128; bn -= 64) {
    if (bn == 192 && b_mn) continue;
    const long units = tm * ((N + bn - 1) / bn);
    const long cost = ((units + pairs - 1) / pairs) * (bn + 32);
    if (!best || cost < best_cost) { best = bn; best_cost = cost; }
  }
  return best;
}
}  // namespace mxb

using namespace mxb;

// D[M,N] = act(op(A) * op(B) + bias).  a_mn = 0: A is [M, K] with row pitch lda; a_mn = 1: A is [K, M] with row pitch
// lda.  b_mn = 0: B is [N, K]; b_mn = 1: B is [K, N]; row pitch ldb.  ldd: row pitch of D.  All pitches in elements.
// Requirements: base pointers 16-byte aligned, lda and ldb multiples of 8 elements.  `error_flag` is a device int set
// to 1 when a CTA gave up waiting (the output is then incomplete).
static int gemm_run(int dtype, const void* A, const void* B, void* D, const void* bias, int M, int N, int K, int lda, int ldb,
                    int ldd, int a_mn, int b_mn, int act, float* ws, int* error_flag, void* stream, int batch = 1,
                    long long sa = 0, long long sb = 0, long long sd = 0) {
  if (dtype != kF16 && dtype != kBF16) return -1;
  if (M < 1 || N < 1 || K < 1) return -2;
  if ((lda % 8) || (ldb % 8) || ((uintptr_t)A % 16) || ((uintptr_t)B % 16) || ((uintptr_t)D % 16)) return -3;
  if (lda < (a_mn ? M : K) || ldb < (b_mn ? N : K) || ldd < N) return -3;
  if (batch < 1) return -2;
  if (batch > 1 && ((sa % 8) || (sb % 8) || (sd % 8) || sd < (long long)(M - 1) * ldd + N)) return -3;      // 16-byte aligned matrices
  const int bf16 = dtype == kBF16;
  const int pbn = batch > 1 ? 0 : pick_pair_bn(M, N, K, b_mn);
  const int bn = pbn ? pbn : pick_bn(M, N, K, batch);
  const int b_rows = pbn ? pbn / 2 : bn;          // rows of B one CTA stages per k-step
  CUtensorMap ma, mb;
  const int a3d = a_mn && (M % 64) == 0, b3d = b_mn && (N % 64) == 0;
  int rc = a3d ? make_map_mn3(&ma, A, bf16, K, M, lda, BM / 64, batch, sa)
               : (a_mn ? make_map_mn(&ma, A, bf16, K, M, lda, batch, sa) : make_map(&ma, A, bf16, M, K, lda, BM, batch, sa));
  if (rc) return rc;
  rc = b3d ? make_map_mn3(&mb, B, bf16, K, N, ldb, b_rows / 64, batch, sb)
           : (b_mn ? make_map_mn(&mb, B, bf16, K, N, ldb, batch, sb) : make_map(&mb, B, bf16, N, K, ldb, b_rows, batch, sb));
  if (rc) return rc;
  // the epilogue stores through the copy engine when D meets a tensor map's rules (16-byte row pitch); otherwise with
  // per-thread stores
  CUtensorMap md = ma;
  const int use_tma_store = (ldd % 8) == 0 ? 1 : 0;
  if (use_tma_store) {
    rc = make_map_store(&md, D, bf16, M, N, ldd, batch, sd);
    if (rc) return rc;
  }
  cudaStream_t st = (cudaStream_t)stream;
#define MXB_GEMM_ARGS ma, mb, md, use_tma_store, D, bias, M, N, K, ldd, act, bf16, a_mn, b_mn, ws, a3d, b3d, error_flag, st
  if (pbn) {
#define MXB_GEMM_PAIR(T) \
  (pbn == 256 ? launch_gemm_pair<T, 256>(MXB_GEMM_ARGS) : pbn == 192 ? launch_gemm_pair<T, 192>(MXB_GEMM_ARGS) : launch_gemm_pair<T, 128>(MXB_GEMM_ARGS))
    return bf16 ? MXB_GEMM_PAIR(__nv_bfloat16) : MXB_GEMM_PAIR(__half);
#undef MXB_GEMM_PAIR
  }
#define MXB_GEMM(T)                                                                                                 \
  (bn == 256 ? launch_gemm<T, 256>(MXB_GEMM_ARGS, batch, sd) : bn == 192 ? launch_gemm<T, 192>(MXB_GEMM_ARGS, batch, sd)    \
   : bn == 128 ? launch_gemm<T, 128>(MXB_GEMM_ARGS, batch, sd) : launch_gemm<T, 64>(MXB_GEMM_ARGS, batch, sd))
  return bf16 ? MXB_GEMM(__nv_bfloat16) : MXB_GEMM(__half);
#undef MXB_GEMM
#undef MXB_GEMM_ARGS
}

// Kernel selection for later calls: 0 = per shape (the default), 1 = single-CTA kernel only, 2 = the CTA-pair kernel
// wherever it applies.  For benchmarks and tests that compare the two.
MXB_EXPORT void mxb_gemm_set_variant(int v) { g_gemm_variant = v; }
MXB_EXPORT void mxb_gemm_set_streamk(int on) { g_gemm_streamk = on; }

MXB_EXPORT int mxb_gemm(int dtype, const void* A, const void* B, void* D, const void* bias, int M, int N, int K, int lda,
                        int ldb, int ldd, int a_mn, int b_mn, int act, int* error_flag, void* stream) {
  return gemm_run(dtype, A, B, D, bias, M, N, K, lda, ldb, ldd, a_mn, b_mn, act, nullptr, error_flag, stream);
}

// Bytes of the stream-K workspace that mxb_gemm_ws takes: allocate once per device and stream, fill with zeros once.
MXB_EXPORT uint64_t mxb_gemm_workspace_bytes() { return (uint64_t)sk_workspace_bytes(); }

// The same product with the stream-K workspace: a last round of tiles that would leave SMs idle (or an output with
// fewer tiles than SMs, such as a weight gradient with a long contraction) is cut evenly over the CTAs by k-steps; the
// pieces of a tile are combined by the CTA whose piece finishes last.  Launches that use one workspace must not overlap.
MXB_EXPORT int mxb_gemm_ws(int dtype, const void* A, const void* B, void* D, const void* bias, int M, int N, int K, int lda,
                           int ldb, int ldd, int a_mn, int b_mn, int act, float* workspace, int* error_flag, void* stream) {
  if (workspace && ((uintptr_t)workspace % 16)) return -3;
  return gemm_run(dtype, A, B, D, bias, M, N, K, lda, ldb, ldd, a_mn, b_mn, act, workspace, error_flag, stream);
}

// `batch` products of identical shape: matrix i of A, B, D starts `stride_a`, `stride_b`, `stride_d` elements (multiples of 8)
// after matrix i-1; the bias (one value per column) is shared.  Tiles of all matrices form one persistent grid; the
// stream-K workspace is used as for a single product.  This is the contraction behind batch_dot and the per-head
// products of attention (the reference calls cublasGemmStridedBatchedEx, src/operator/linalg_impl.h:538-544).
MXB_EXPORT int mxb_gemm_batched(int dtype, const void* A, const void* B, void* D, const void* bias, int batch, int M, int N, int K,
                                int lda, int ldb, int ldd, long long stride_a, long long stride_b, long long stride_d, int a_mn,
                                int b_mn, int act, float* workspace, int* error_flag, void* stream) {
  if (workspace && ((uintptr_t)workspace % 16)) return -3;
  return gemm_run(dtype, A, B, D, bias, M, N, K, lda, ldb, ldd, a_mn, b_mn, act, workspace, error_flag, stream, batch, stride_a,
                  stride_b, stride_d);
}

// Whether mxb_gemm_ws would cut this product by k-steps (for reports; callers may always pass the workspace).
MXB_EXPORT int mxb_gemm_wants_workspace(int M, int N, int K) {
  if (pick_pair_bn(M, N, K, 0)) return 0;
  const int bn = pick_bn(M, N, K);
  const int tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn);
  return plan_streamk(tiles, (K + BK - 1) / BK, sm_count(), true).sk_tiles > 0 ? 1 : 0;
}

// D[M,N] = act(A[M,K] * B[N,K]^T + bias): both operands K-major.
MXB_EXPORT int mxb_gemm_tn(int dtype, const void* A, const void* B, void* D, const void* bias, int M, int N, int K,
                           int lda, int ldb, int ldd, int act, int* error_flag, void* stream) {
  return mxb_gemm(dtype, A, B, D, bias, M, N, K, lda, ldb, ldd, 0, 0, act, error_flag, stream);
}

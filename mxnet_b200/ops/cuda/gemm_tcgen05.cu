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
  static constexpr uint32_t STG_BYTES = 4 * 2048;   // per epilogue warp: 32 rows x 64 bytes staged for the TMA store
  static constexpr uint32_t SMEM_BYTES = STAGES * (A_BYTES + B_BYTES) + STG_BYTES + 1024 /*alignment slack*/ + 512 /*barriers*/;
};

enum Act { kActNone = 0, kActRelu = 1, kActGelu = 2 };

__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.f + erf_fast(x * 0.70710678118654752f)); }

template <typename T, int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_d, int use_tma_store, T* __restrict__ D, const T* __restrict__ bias, int M,
               int N, int K, int ldd, int act, int bf16, int a_mn, int b_mn, const FastDiv fd_tiles_m,
               int ksplit, int ksteps_per, int full_tiles, const FastDiv fd_rem_tiles, float* __restrict__ ws, int a3d, int b3d,
               int* __restrict__ error_flag) {
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
  // Work units: the first `full_tiles` tiles are computed whole; each of the remaining tiles (the last, partial round of
  // the persistent grid, or all tiles of a small output) is split into `ksplit` k-ranges whose partial products are
  // added into the fp32 workspace.  Units of one k-range are adjacent.
  const int rem_tiles = num_tiles - full_tiles;
  const int num_units = full_tiles + rem_tiles * ksplit;
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
      for (int unit = blockIdx.x; unit < num_units && ok && !*abort_flag; unit += gridDim.x) {
        uint32_t ks_u = 0, tile_u = (uint32_t)unit, tile_n_u, tile_m_u;
        if (unit >= full_tiles) {
          fd_divmod((uint32_t)(unit - full_tiles), fd_rem_tiles, &ks_u, &tile_u);
          tile_u += (uint32_t)full_tiles;
        }
        fd_divmod(tile_u, fd_tiles_m, &tile_n_u, &tile_m_u);
        const int tile_m = (int)tile_m_u, tile_n = (int)tile_n_u;
        const int k0 = unit >= full_tiles ? (int)ks_u * ksteps_per : 0;
        const int k1 = unit >= full_tiles ? min(num_k, k0 + ksteps_per) : num_k;
        for (int kt = k0; kt < k1; ++kt) {
          if (!mbar_wait(&empty[st], ph ^ 1u)) { *abort_flag = 1; ok = false; break; }
          mbar_expect_tx(&full[st], A_BYTES + B_BYTES);
          if (!a_mn) {
            tma_load_2d(sA + st * A_BYTES, &map_a, kt * BK, tile_m * BM, &full[st]);
          } else if (a3d) {
            // all 64-column chunks of the tile in one box {64 columns, 64 k-rows, BM/64 chunks}
            tma_load_3d(sA + st * A_BYTES, &map_a, 0, kt * BK, tile_m * (BM / 64), &full[st]);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(sA + st * A_BYTES + c * kMnChunkBytes, &map_a, tile_m * BM + c * 64, kt * BK, &full[st]);
          }
          if (!b_mn) {
            tma_load_2d(sB + st * B_BYTES, &map_b, kt * BK, tile_n * BN, &full[st]);
          } else if (b3d) {
            tma_load_3d(sB + st * B_BYTES, &map_b, 0, kt * BK, tile_n * (BN / 64), &full[st]);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sB + st * B_BYTES + c * kMnChunkBytes, &map_b, tile_n * BN + c * 64, kt * BK, &full[st]);
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
      for (int unit = blockIdx.x; unit < num_units && ok && !*abort_flag; unit += gridDim.x, ++t) {
        const int ks = unit >= full_tiles ? (int)fd_div((uint32_t)(unit - full_tiles), fd_rem_tiles) : 0;
        const int k0 = unit >= full_tiles ? ks * ksteps_per : 0;
        const int k1 = unit >= full_tiles ? min(num_k, k0 + ksteps_per) : num_k;
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
    uint8_t* stg = sStg + q * 2048;       // this warp's staging tile: 32 rows x 64 bytes, 64-byte swizzle
    int t = 0;
    for (int unit = blockIdx.x; unit < num_units; unit += gridDim.x, ++t) {
      uint32_t ks_u = 0, tile_u = (uint32_t)unit, tile_n_u, tile_m_u;
      if (unit >= full_tiles) {
        fd_divmod((uint32_t)(unit - full_tiles), fd_rem_tiles, &ks_u, &tile_u);
        tile_u += (uint32_t)full_tiles;
      }
      fd_divmod(tile_u, fd_tiles_m, &tile_n_u, &tile_m_u);
      const int tile_m = (int)tile_m_u, tile_n = (int)tile_n_u;
      const bool to_ws = ws != nullptr && unit >= full_tiles;
      const int buf = t & 1;
      const bool ready = mbar_wait(&acc_full[buf], ((uint32_t)t >> 1) & 1u);
      if (!ready) *abort_flag = 1;
      if (!ready || *abort_flag) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row = tile_m * BM + q * 32 + lane;
      const bool bias_vec = bias != nullptr && ((reinterpret_cast<uintptr_t>(bias) & 15) == 0);
      const bool row_vec = (ldd % 8) == 0;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * Cfg::ACC_STRIDE);
      uint32_t r[32];
      tmem_ld32(taddr, r);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        const int col0 = tile_n * BN + c0;
        const bool full_cols = col0 + 32 <= N;
        // bias of these 32 columns first, so its latency overlaps the TMEM load (registers only: every index
        // below is a compile-time constant after unrolling)
        float bv[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) bv[j] = 0.f;
        if (bias != nullptr && col0 < N) {
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
        if (to_ws) {
          // split-K: add this k-range's partial tile to the fp32 workspace (bias and activation are applied by the
          // finishing kernel once every k-range has been added)
          if (row < M && col0 < N) {
            float* wrow = ws + (size_t)row * N + col0;
            if (full_cols && (N % 4) == 0) {
#pragma unroll
              for (int v = 0; v < 8; ++v)
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(wrow + v * 4), "f"(__uint_as_float(r[v * 4])),
                             "f"(__uint_as_float(r[v * 4 + 1])), "f"(__uint_as_float(r[v * 4 + 2])),
                             "f"(__uint_as_float(r[v * 4 + 3])) : "memory");
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < N) atomicAdd(wrow + j, __uint_as_float(r[j]));
            }
          }
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
          if (lane == 0) tma_store_wait_read();
          __syncwarp();
          if (col0 < N) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              Vec16<T> o;
#pragma unroll
              for (int j = 0; j < 8; ++j) o.v[j] = Cvt<T>::from_f(f[v * 8 + j]);
              st16(reinterpret_cast<T*>(stg + lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4)), o);
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&map_d, stg, col0, tile_m * BM + q * 32);
              tma_store_commit();
            }
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

// Split-K helpers over the tiles [first_tile, first_tile + gridDim.x) of a 128 x BN tiling (tile = tile_n * tiles_m +
// tile_m): `zero` clears their region of the fp32 workspace before the GEMM, `finish` computes D = act(ws + bias) there
// afterwards.  One CTA per tile, one thread per 8 columns of a row.
template <typename T, bool kFinish>
__global__ void __launch_bounds__(256)
gemm_splitk_tiles_kernel(float* __restrict__ ws, const T* __restrict__ bias, T* __restrict__ D, int M, int N, int ldd, int act,
                         int bn, int tiles_m, int first_tile) {
  const int tile = first_tile + blockIdx.x;
  const int tile_m = tile % tiles_m, tile_n = tile / tiles_m;
  const int vec_per_row = bn / 8;
  for (int i = threadIdx.x; i < BM * vec_per_row; i += blockDim.x) {
    const int row = tile_m * BM + i / vec_per_row, c = tile_n * bn + (i % vec_per_row) * 8;
    if (row >= M || c >= N) continue;
    float* w = ws + (size_t)row * N + c;
    if (!kFinish) {
      *reinterpret_cast<float4*>(w) = make_float4(0.f, 0.f, 0.f, 0.f);
      *reinterpret_cast<float4*>(w + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
      continue;
    }
    const float4 a = *reinterpret_cast<const float4*>(w);
    const float4 b = *reinterpret_cast<const float4*>(w + 4);
    float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    Vec16<T> o;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float x = v[j] + (bias ? Cvt<T>::to_f(bias[c + j]) : 0.f);
      if (act == kActRelu) x = fmaxf(x, 0.f);
      else if (act == kActGelu) x = gelu_erf(x);
      o.v[j] = Cvt<T>::from_f(x);
    }
    st16(D + (size_t)row * ldd + c, o);
  }
}

// 2-D row-major [rows, cols] half tensor, row pitch `ld` elements; box = box_rows x 64 columns, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, int bf16, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult rc = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base),
                   dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? 0 : -11;
}

// MN-major operand: global tensor [K rows, MN columns] with row pitch `ld`; box = 64 k-rows x 64 columns.
static int make_map_mn(CUtensorMap* map, const void* base, int bf16, int64_t krows, int64_t mn, int64_t ld) {
  return make_map(map, base, bf16, krows, mn, ld, BK);
}

// The same operand when MN is a multiple of 64: a 3-D view {64 columns, K rows, MN/64 chunks} (chunk stride 128 bytes)
// whose box {64, 64, chunks} brings every chunk of a tile with one copy, chunk after chunk in shared memory.
static int make_map_mn3(CUtensorMap* map, const void* base, int bf16, int64_t krows, int64_t mn, int64_t ld, int chunks) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  cuuint64_t dims[3] = {64, (cuuint64_t)krows, (cuuint64_t)(mn / 64)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, 128};
  cuuint32_t box[3] = {64, (cuuint32_t)BK, (cuuint32_t)chunks};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult rc = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base),
                   dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? 0 : -11;
}

// Output matrix [M, N] with row pitch ldd for the epilogue's stores: box = 32 rows x 32 columns, 64-byte swizzle.
static int make_map_store(CUtensorMap* map, const void* base, int bf16, int64_t rows, int64_t cols, int64_t ld) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult rc = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base),
                   dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? 0 : -11;
}

template <typename T, int BN>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& md, int use_tma_store, void* D,
                       const void* bias, int M, int N, int K, int ldd, int act, int bf16, int a_mn, int b_mn, float* ws, int a3d,
                       int b3d, int* error_flag, cudaStream_t st) {
  using Cfg = TileCfg<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t rc = cudaFuncSetAttribute(gemm_tn_kernel<T, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (rc != cudaSuccess) return (int)rc;
    attr_set = true;
  }
  const int tiles_m = (M + BM - 1) / BM;
  const int tiles = tiles_m * ((N + BN - 1) / BN);
  const int num_k = (K + BK - 1) / BK;
  // Split-K (needs the workspace) when the output has too few tiles to occupy the SMs.  The kernel can also split only
  // the tiles of a last, partial round (full_tiles > 0); measured on N = 768 outputs of 8192 rows that was slower than
  // leaving the round partial (the fp32 reductions and the two helper launches cost more than the idle SMs), so the
  // host does not select it.
  int full_tiles = tiles, ksplit = 1;
  const int sms = sm_count();
  if (ws != nullptr && (N % 8) == 0 && (ldd % 8) == 0 && num_k >= 8) {
    if (tiles * 10 < sms * 7) full_tiles = 0;
    if (full_tiles < tiles) {
      ksplit = sms / (tiles - full_tiles);
      if (ksplit > num_k / 4) ksplit = num_k / 4;
      if (ksplit < 2) { ksplit = 1; full_tiles = tiles; }
    }
  }
  int ksteps_per = (num_k + ksplit - 1) / ksplit;
  ksplit = (num_k + ksteps_per - 1) / ksteps_per;
  if (ksplit < 2) { ksplit = 1; full_tiles = tiles; ksteps_per = num_k; }
  const int rem_tiles = tiles - full_tiles;
  float* kws = rem_tiles > 0 ? ws : nullptr;
  if (kws) gemm_splitk_tiles_kernel<T, false><<<rem_tiles, 256, 0, st>>>(kws, nullptr, nullptr, M, N, ldd, act, BN, tiles_m, full_tiles);
  const long units = (long)full_tiles + (long)rem_tiles * ksplit;
  const int grid = units < sms ? (int)units : sms;
  gemm_tn_kernel<T, BN><<<grid, kGemmThreads, Cfg::SMEM_BYTES, st>>>(ma, mb, md, use_tma_store, (T*)D, (const T*)bias, M, N, K, ldd,
                                                                     act, bf16, a_mn, b_mn, make_fastdiv((uint32_t)tiles_m), ksplit,
                                                                     ksteps_per, full_tiles,
                                                                     make_fastdiv((uint32_t)(rem_tiles > 0 ? rem_tiles : 1)), kws, a3d,
                                                                     b3d, error_flag);
  if (kws) gemm_splitk_tiles_kernel<T, true><<<rem_tiles, 256, 0, st>>>(kws, (const T*)bias, (T*)D, M, N, ldd, act, BN, tiles_m, full_tiles);
  return (int)cudaGetLastError();
}

// Tile width: the widest tile that still gives every SM work, or the widest tile with split-K when the output has too
// few tiles for the SMs anyway; narrow outputs take the narrow tile.  (A 192-wide tile is compiled but not selected: it
// measured no faster than 128 or 256 on the shapes where it divides N.)
static int pick_bn(int M, int N) {
  const long tm = (M + BM - 1) / BM;
  if (N <= 64) return 64;
  if (N <= 128) return 128;
  const long tiles256 = tm * ((N + 255) / 256);
  if (tiles256 >= sm_count()) return 256;
  if (tiles256 * 10 < (long)sm_count() * 7) return 256;      // split-K fills the machine
  return 128;
}

}  // namespace mxb

using namespace mxb;

// D[M,N] = act(op(A) * op(B) + bias).  a_mn = 0: A is [M, K] with row pitch lda; a_mn = 1: A is [K, M] with row pitch
// lda.  b_mn = 0: B is [N, K]; b_mn = 1: B is [K, N]; row pitch ldb.  ldd: row pitch of D.  All pitches in elements.
// Requirements: base pointers 16-byte aligned, lda and ldb multiples of 8 elements.  `error_flag` is a device int set
// to 1 when a CTA gave up waiting (the output is then incomplete).
static int gemm_run(int dtype, const void* A, const void* B, void* D, const void* bias, int M, int N, int K, int lda, int ldb,
                    int ldd, int a_mn, int b_mn, int act, float* ws, int* error_flag, void* stream) {
  if (dtype != kF16 && dtype != kBF16) return -1;
  if (M < 1 || N < 1 || K < 1) return -2;
  if ((lda % 8) || (ldb % 8) || ((uintptr_t)A % 16) || ((uintptr_t)B % 16) || ((uintptr_t)D % 16)) return -3;
  if (lda < (a_mn ? M : K) || ldb < (b_mn ? N : K) || ldd < N) return -3;
  const int bf16 = dtype == kBF16;
  const int bn = pick_bn(M, N);
  CUtensorMap ma, mb;
  const int a3d = a_mn && (M % 64) == 0, b3d = b_mn && (N % 64) == 0;
  int rc = a3d ? make_map_mn3(&ma, A, bf16, K, M, lda, BM / 64)
               : (a_mn ? make_map_mn(&ma, A, bf16, K, M, lda) : make_map(&ma, A, bf16, M, K, lda, BM));
  if (rc) return rc;
  rc = b3d ? make_map_mn3(&mb, B, bf16, K, N, ldb, bn / 64)
           : (b_mn ? make_map_mn(&mb, B, bf16, K, N, ldb) : make_map(&mb, B, bf16, N, K, ldb, bn));
  if (rc) return rc;
  // the epilogue stores through the copy engine when D meets a tensor map's rules (16-byte row pitch); otherwise with
  // per-thread stores
  CUtensorMap md = ma;
  const int use_tma_store = (ldd % 8) == 0 ? 1 : 0;
  if (use_tma_store) {
    rc = make_map_store(&md, D, bf16, M, N, ldd);
    if (rc) return rc;
  }
  cudaStream_t st = (cudaStream_t)stream;
#define MXB_GEMM(T)                                                                                                        \
  (bn == 256 ? launch_gemm<T, 256>(ma, mb, md, use_tma_store, D, bias, M, N, K, ldd, act, bf16, a_mn, b_mn, ws, a3d, b3d, error_flag, st)  \
   : bn == 192 ? launch_gemm<T, 192>(ma, mb, md, use_tma_store, D, bias, M, N, K, ldd, act, bf16, a_mn, b_mn, ws, a3d, b3d, error_flag, st) \
   : bn == 128 ? launch_gemm<T, 128>(ma, mb, md, use_tma_store, D, bias, M, N, K, ldd, act, bf16, a_mn, b_mn, ws, a3d, b3d, error_flag, st) \
               : launch_gemm<T, 64>(ma, mb, md, use_tma_store, D, bias, M, N, K, ldd, act, bf16, a_mn, b_mn, ws, a3d, b3d, error_flag, st))
  return bf16 ? MXB_GEMM(__nv_bfloat16) : MXB_GEMM(__half);
#undef MXB_GEMM
}

MXB_EXPORT int mxb_gemm(int dtype, const void* A, const void* B, void* D, const void* bias, int M, int N, int K, int lda,
                        int ldb, int ldd, int a_mn, int b_mn, int act, int* error_flag, void* stream) {
  return gemm_run(dtype, A, B, D, bias, M, N, K, lda, ldb, ldd, a_mn, b_mn, act, nullptr, error_flag, stream);
}

// The same product with an fp32 workspace of M*N floats: outputs with too few tiles for the SMs (a weight gradient with
// a long contraction) are then computed as split-K partial products added into the workspace.
MXB_EXPORT int mxb_gemm_ws(int dtype, const void* A, const void* B, void* D, const void* bias, int M, int N, int K, int lda,
                           int ldb, int ldd, int a_mn, int b_mn, int act, float* workspace, int* error_flag, void* stream) {
  if (workspace && ((uintptr_t)workspace % 16)) return -3;
  return gemm_run(dtype, A, B, D, bias, M, N, K, lda, ldb, ldd, a_mn, b_mn, act, workspace, error_flag, stream);
}

// Whether mxb_gemm_ws would split the contraction of this shape (so that callers allocate the workspace only then).
MXB_EXPORT int mxb_gemm_wants_workspace(int M, int N, int K) {
  const int bn = pick_bn(M, N);
  const int tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn);
  const int num_k = (K + BK - 1) / BK;
  if ((N % 8) != 0 || num_k < 8) return 0;
  return tiles * 10 < sm_count() * 7 ? 1 : 0;
}

// D[M,N] = act(A[M,K] * B[N,K]^T + bias): both operands K-major.
MXB_EXPORT int mxb_gemm_tn(int dtype, const void* A, const void* B, void* D, const void* bias, int M, int N, int K,
                           int lda, int ldb, int ldd, int act, int* error_flag, void* stream) {
  return mxb_gemm(dtype, A, B, D, bias, M, N, K, lda, ldb, ldd, 0, 0, act, error_flag, stream);
}

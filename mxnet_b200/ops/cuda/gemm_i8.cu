// INT8 GEMM on the 5th-generation tensor cores: D[M, N] (int32) = A[M, K] (int8) . B[N, K]^T (int8), with an optional
// per-column int32 bias added to the accumulators.  This is the contraction of the quantised FullyConnected operator and
// of quantised 1x1 convolutions; the reference reaches it through cuBLAS / cuDNN int8 paths
// (src/operator/quantization/quantized_fully_connected.cu: cublasGemmEx with CUDA_R_8I operands and CUDA_R_32I
// accumulation).  Same structure as the half-precision kernel (gemm_tcgen05.cu): persistent CTAs walk 128 x BN output
// tiles; warp 0 lane 0 feeds a ring of TMA loads (128 rows x 128 bytes of K per operand and k-step, 128-byte swizzle),
// warp 1 lane 0 issues four tcgen05.mma.kind::i8 (M128 x N(BN) x K32) per k-step into one of two TMEM accumulators,
// warps 2..5 drain the other accumulator with tcgen05.ld and write 32 x 32 int32 tiles through swizzled staging and TMA stores.  Every mbarrier wait is bounded; a CTA that
// gives up raises the error flag, waits (bounded) for its copies in flight, frees its TMEM and exits.
#include "tcgen05.cuh"

namespace mxb {

constexpr int IBM = 128, IBK = 128, IUMMA_K = 32;      // IBK int8 elements = 128 bytes = one swizzle row
constexpr int kI8Threads = 192;
constexpr uint32_t IA_BYTES = IBM * IBK;

template <int BN> struct I8Cfg {
  static constexpr uint32_t B_BYTES = BN * IBK;
  static constexpr int STAGES = BN == 256 ? 4 : 6;
  static constexpr uint32_t TMEM_COLS = 2 * BN;
  static constexpr uint32_t STG_BYTES = 4 * 2 * 4096;     // per epilogue warp: two 32 x 32 int32 staging tiles
  static constexpr uint32_t SMEM_BYTES = STAGES * (IA_BYTES + B_BYTES) + STG_BYTES + 1024 + 512;
};

// Instruction descriptor for kind::i8: D = s32 (code 2 at bit 4), A and B signed 8-bit (code 1 at bits 7 and 10),
// both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc_i8(int bn, int bm = 128) {
  return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(bm >> 4) << 24);
}

__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

template <int BN>
__global__ void __launch_bounds__(kI8Threads, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_d, int use_tma_store, int32_t* __restrict__ D,
               const int32_t* __restrict__ bias, int M, int N, int K, int ldd, const FastDiv fd_tiles_m,
               int* __restrict__ error_flag) {
  using Cfg = I8Cfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr uint32_t B_BYTES = Cfg::B_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * IA_BYTES;
  uint8_t* sStage = smem + STAGES * (IA_BYTES + B_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStage + Cfg::STG_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + 8;
  uint64_t* acc_full = bars + 16;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* issued_it = abort_flag + 1;
  volatile int* consumed_it = abort_flag + 2;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_k = (K + IBK - 1) / IBK;
  const int tiles_m = (M + IBM - 1) / IBM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  constexpr uint32_t kTmemCols = Cfg::TMEM_COLS;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
    *abort_flag = 0;
    *issued_it = 0;
    *consumed_it = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0, st = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok && !*abort_flag; tile += gridDim.x) {
        uint32_t tn, tm;
        fd_divmod((uint32_t)tile, fd_tiles_m, &tn, &tm);
        for (int kt = 0; kt < num_k; ++kt) {
          if (!mbar_wait(&empty[st], ph ^ 1u)) { *abort_flag = 1; ok = false; break; }
          mbar_expect_tx(&full[st], IA_BYTES + B_BYTES);
          tma_load_2d(sA + st * IA_BYTES, &map_a, kt * IBK, (int)tm * IBM, &full[st]);
          tma_load_2d(sB + st * B_BYTES, &map_b, kt * IBK, (int)tn * BN, &full[st]);
          ++it;
          if (++st == STAGES) { st = 0; ph ^= 1u; }
        }
      }
      *issued_it = it;
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_i8(BN);
      const uint64_t adesc0 = make_desc(smem_u32(sA)), bdesc0 = make_desc(smem_u32(sB));
      int it = 0, st = 0, t = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok && !*abort_flag; tile += gridDim.x, ++t) {
        const int buf = t & 1;
        if (!mbar_wait(&acc_empty[buf], (((uint32_t)t >> 1) & 1u) ^ 1u)) { *abort_flag = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        for (int kt = 0; kt < num_k; ++kt) {
          if (!mbar_wait(&full[st], ph)) { *abort_flag = 1; ok = false; break; }
          const uint64_t adesc = adesc0 + (uint64_t)(st * (int)(IA_BYTES >> 4));
          const uint64_t bdesc = bdesc0 + (uint64_t)(st * (int)(B_BYTES >> 4));
          umma_i8(tmem_d, adesc, bdesc, idesc, kt > 0 ? 1u : 0u);
#pragma unroll
          for (int k = 1; k < IBK / IUMMA_K; ++k)      // 32 elements of K = 32 bytes inside the swizzle row
            umma_i8(tmem_d, adesc + 2 * (uint64_t)k, bdesc + 2 * (uint64_t)k, idesc, 1u);
          umma_commit(&empty[st]);
          ++it;
          if (++st == STAGES) { st = 0; ph ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&acc_full[buf]);
      }
      *consumed_it = it;
    }
  } else {
    const int q = warp & 3;
    int t = 0, nstore = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++t) {
      uint32_t tn, tm;
      fd_divmod((uint32_t)tile, fd_tiles_m, &tn, &tm);
      const int buf = t & 1;
      const bool ready = mbar_wait(&acc_full[buf], ((uint32_t)t >> 1) & 1u);
      if (!ready) *abort_flag = 1;
      if (!ready || *abort_flag) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row = (int)tm * IBM + q * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
      const bool row_vec = (ldd % 4) == 0;
      uint32_t r[32];
      tmem_ld32(taddr, r);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        const int col0 = (int)tn * BN + c0;
        tmem_wait_ld32(r);
        int32_t v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (int32_t)r[j];
        if (c0 + 32 < BN) tmem_ld32(taddr + (uint32_t)(c0 + 32), r);
        if (bias != nullptr && col0 < N) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < N) v[j] += bias[col0 + j];
        }
        if (use_tma_store) {
          // 32 x 32 int32 tile through a swizzled staging buffer and one TMA store (which clips at the matrix edge):
          // lane r writes row r; its 16-byte piece j goes to slot j ^ (r & 7), so a quarter warp hits eight different
          // bank groups.  Two buffers per warp: the store issued two chunks ago has released the one reused now.
          uint8_t* stg = sStage + (size_t)q * 8192 + (size_t)(nstore & 1) * 4096;
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          __syncwarp();
          if (col0 < N && (int)tm * IBM + q * 32 < M) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<int4*>(stg + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                  make_int4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&map_d, stg, col0, (int)tm * IBM + q * 32);
              tma_store_commit();
            }
            ++nstore;
          }
        } else if (row < M && col0 < N) {
          int32_t* drow = D + (size_t)row * ldd + col0;
          if (col0 + 32 <= N && row_vec) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) *reinterpret_cast<int4*>(drow + j) = make_int4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < N) drow[j] = v[j];
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    if (use_tma_store && lane == 0) tma_store_wait_all();
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) {
    for (int it = *consumed_it; it < *issued_it; ++it) mbar_wait(&full[it % STAGES], (uint32_t)(it / STAGES) & 1u);
    if (error_flag) atomicExch(error_flag, 1);
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// int8 row-major [rows, K] matrix, row pitch `ld` bytes (a multiple of 16); box = box_rows x 128 bytes, 128-byte swizzle.
static int make_map_i8(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld};
  cuuint32_t box[2] = {(cuuint32_t)IBK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? 0 : -11;
}

// int32 row-major [rows, cols] output, row pitch `ld` elements (a multiple of 4); box = 32 x 32 elements, 128-byte swizzle.
static int make_map_i32_store(CUtensorMap* map, void* base, int64_t rows, int64_t cols, int64_t ld) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -10;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? 0 : -11;
}

template <int BN>
static int launch_i8(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& md, int use_tma_store, int32_t* D, const int32_t* bias, int M, int N, int K, int ldd,
                     int* error_flag, cudaStream_t st) {
  using Cfg = I8Cfg<BN>;
  static unsigned long long attr_seen = 0;
  if (first_on_device(&attr_seen)) {
    cudaError_t rc = cudaFuncSetAttribute(gemm_i8_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (rc != cudaSuccess) return (int)rc;
  }
  const int tiles_m = (M + IBM - 1) / IBM;
  const long tiles = (long)tiles_m * ((N + BN - 1) / BN);
  if (tiles > 0x3fffffffL) return -2;
  const int grid = tiles < sm_count() ? (int)tiles : sm_count();
  gemm_i8_kernel<BN><<<grid, kI8Threads, Cfg::SMEM_BYTES, st>>>(ma, mb, md, use_tma_store, D, bias, M, N, K, ldd, make_fastdiv((uint32_t)tiles_m),
                                                               error_flag);
  return (int)cudaGetLastError();
}

}  // namespace mxb

using namespace mxb;

// D[M, N] (int32, row pitch ldd elements) = A[M, K] . B[N, K]^T + bias[N]; A, B signed 8-bit with row pitches lda, ldb
// bytes.  Requirements: K, lda, ldb multiples of 16; base pointers 16-byte aligned.  `error_flag`: device int set to 1
// when a CTA gave up waiting (the output is then incomplete).
MXB_EXPORT int mxb_gemm_i8(const void* A, const void* B, void* D, const void* bias, int M, int N, int K, int lda, int ldb, int ldd,
                           int* error_flag, void* stream) {
  if (M < 1 || N < 1 || K < 1) return -2;
  if ((K % 16) || (lda % 16) || (ldb % 16) || ((uintptr_t)A % 16) || ((uintptr_t)B % 16) || ((uintptr_t)D % 16)) return -3;
  if (lda < K || ldb < K || ldd < N) return -3;
  const int bn = N <= 128 ? 128 : 256;
  CUtensorMap ma, mb;
  int rc = make_map_i8(&ma, A, M, K, lda, IBM);
  if (rc) return rc;
  rc = make_map_i8(&mb, B, N, K, ldb, bn);
  if (rc) return rc;
  CUtensorMap md;
  const int use_tma_store = (ldd % 4) == 0 ? 1 : 0;     // a TMA row pitch is a multiple of 16 bytes
  if (use_tma_store) {
    rc = make_map_i32_store(&md, D, M, N, ldd);
    if (rc) return rc;
  } else {
    md = ma;
  }
  cudaStream_t st = (cudaStream_t)stream;
  return bn == 256 ? launch_i8<256>(ma, mb, md, use_tma_store, (int32_t*)D, (const int32_t*)bias, M, N, K, ldd, error_flag, st)
                   : launch_i8<128>(ma, mb, md, use_tma_store, (int32_t*)D, (const int32_t*)bias, M, N, K, ldd, error_flag, st);
}

// Dense GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) fed by TMA, for sm_100a.
//
//   D[M, N] = act( A[M, K] · B[N, K]^T + bias[N] )        A, B, D: fp16 or bf16, accumulation in fp32
//
// This is the contraction behind FullyConnected / dot / batch_dot and 1x1 NHWC convolutions; the
// reference sends all of them to cuBLAS (src/operator/linalg_impl.h: cublasGemmEx, pseudo-fp16 with fp32
// accumulation) followed by a separate add_bias_kernel (src/operator/nn/fully_connected-inl.h:165-367).
//
// Structure of one CTA (192 threads, one 128 x BN output tile, BN = 128):
//   warp 0     : TMA producer.  One elected lane issues cp.async.bulk.tensor.2d loads of a 128x64 A tile and
//                a BNx64 B tile per k-step into a 4-stage shared-memory ring (128-byte swizzle), completion
//                is signalled on an mbarrier with the transaction byte count.
//   warp 1     : MMA issuer.  One elected lane issues four tcgen05.mma (M128 x N128 x K16, kind::f16) per
//                k-step from shared-memory matrix descriptors into a TMEM accumulator (128 lanes x BN fp32
//                columns) and commits each stage back to the producer with tcgen05.commit.
//   warps 2..5 : epilogue.  After the last commit arrives, each warp reads its 32-lane quarter of TMEM with
//                tcgen05.ld (32 columns at a time), adds the bias, applies ReLU/GELU, converts and stores.
// No cluster features and no multicast loads are used, so the same binary runs in multi-GPU jobs.
// Every mbarrier wait is bounded; on expiry the CTA raises an error flag for the host, skips its remaining
// work, frees its TMEM columns and exits.
#include <cuda.h>

#include "common.cuh"

namespace mxb {

constexpr int BM = 128, BN = 128, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int kGemmThreads = 192;
constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
constexpr uint32_t SMEM_BYTES = STAGES * (A_BYTES + B_BYTES) + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr uint32_t kSpinLimit = 1u << 24;

enum Act { kActNone = 0, kActRelu = 1, kActGelu = 2 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: false when the barrier did not flip within the spin budget.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 4096) __nanosleep(64);
  }
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 64 elements (128 bytes),
// 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);          // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                            // leading byte offset (unused for swizzled K-major), bits [16,30)
  d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset between 8-row groups, bits [32,46)
  d |= (uint64_t)1 << 46;                            // descriptor version for sm_100
  d |= (uint64_t)2 << 61;                            // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16: D fp32, A/B fp16 or bf16, both K-major, N and M tile sizes.
__host__ __device__ constexpr uint32_t make_idesc(int bf16) {
  return (1u << 4) | ((uint32_t)bf16 << 7) | ((uint32_t)bf16 << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}

__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }

template <typename T>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, T* __restrict__ D,
               const T* __restrict__ bias, int M, int N, int K, int ldd, int act, int bf16, int* __restrict__ error_flag) {
  extern __shared__ uint8_t smem_raw[];
  // tiles need 1024-byte alignment for the 128-byte swizzle pattern
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * (A_BYTES + B_BYTES));
  uint64_t* full = bars;                  // [STAGES] producer -> MMA
  uint64_t* empty = bars + STAGES;        // [STAGES] MMA -> producer
  uint64_t* acc_full = bars + 2 * STAGES; // accumulator ready for the epilogue
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* issued_kt = abort_flag + 1;      // k-steps whose TMA loads were issued
  volatile int* consumed_kt = abort_flag + 2;    // k-steps whose loads were observed complete by the MMA warp

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_m = blockIdx.y, tile_n = blockIdx.x;
  const int num_k = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    *issued_kt = 0;
    *consumed_kt = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // TMEM allocation is a warp-wide operation; BN fp32 columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int kt = 0; kt < num_k; ++kt) {
        const int s = kt % STAGES;
        const uint32_t phase = (uint32_t)(kt / STAGES) & 1u;
        if (!mbar_wait(&empty[s], phase ^ 1u)) { *abort_flag = 1; break; }
        mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
        tma_load_2d(sA + s * A_BYTES, &map_a, kt * BK, tile_m * BM, &full[s]);
        tma_load_2d(sB + s * B_BYTES, &map_b, kt * BK, tile_n * BN, &full[s]);
        *issued_kt = kt + 1;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(bf16);
      bool ok = true;
      for (int kt = 0; kt < num_k && ok; ++kt) {
        const int s = kt % STAGES;
        const uint32_t phase = (uint32_t)(kt / STAGES) & 1u;
        if (!mbar_wait(&full[s], phase)) { *abort_flag = 1; ok = false; break; }
        *consumed_kt = kt + 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t adesc = make_desc(smem_u32(sA + s * A_BYTES));
        const uint64_t bdesc = make_desc(smem_u32(sB + s * B_BYTES));
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          // advancing K by 16 elements = 32 bytes inside the swizzle atom: +2 in the 16-byte address field
          umma(tmem_base, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, (kt > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty[s]);        // stage is free once these MMAs have read it
      }
      umma_commit(acc_full);           // arrives when every MMA issued above has completed
    }
  } else {
    // epilogue warps 2..5: TMEM lane quarter = warp index modulo 4
    const int q = warp & 3;
    const bool ready = mbar_wait(acc_full, 0);
    if (!ready) *abort_flag = 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int row = tile_m * BM + q * 32 + lane;
    if (ready && !*abort_flag) {
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int col0 = tile_n * BN + c0;
        if (row < M && col0 < N) {
          T* drow = D + (size_t)row * ldd + col0;
          if (col0 + 32 <= N && (ldd % 8 == 0)) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              Vec16<T> o;
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float f = __uint_as_float(r[v * 8 + j]);
                if (bias) f += Cvt<T>::to_f(bias[col0 + v * 8 + j]);
                if (act == kActRelu) f = fmaxf(f, 0.f);
                else if (act == kActGelu) f = gelu_erf(f);
                o.v[j] = Cvt<T>::from_f(f);
              }
              st16(drow + v * 8, o);
            }
          } else {
            for (int j = 0; j < 32 && col0 + j < N; ++j) {
              float f = __uint_as_float(r[j]);
              if (bias) f += Cvt<T>::to_f(bias[col0 + j]);
              if (act == kActRelu) f = fmaxf(f, 0.f);
              else if (act == kActGelu) f = gelu_erf(f);
              drow[j] = Cvt<T>::from_f(f);
            }
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) {
    // gave up somewhere: before the shared memory is released, wait (bounded) for bulk copies that were
    // issued but never consumed, so none is still in flight when the CTA exits
    for (int kt = *consumed_kt; kt < *issued_kt; ++kt) mbar_wait(&full[kt % STAGES], (uint32_t)(kt / STAGES) & 1u);
    if (error_flag) atomicExch(error_flag, 1);
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess) fn = (EncodeTiledFn)p;
  }
  return fn;
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

}  // namespace mxb

using namespace mxb;

// D[M,N] = act(A[M,K] * B[N,K]^T + bias).  lda/ldb/ldd are row pitches in elements.  Requirements: base
// pointers 16-byte aligned, lda and ldb multiples of 8 elements, K >= 1.  `error_flag` is a device int set to
// 1 when a CTA gave up waiting (the output is then incomplete).
MXB_EXPORT int mxb_gemm_tn(int dtype, const void* A, const void* B, void* D, const void* bias, int M, int N, int K,
                           int lda, int ldb, int ldd, int act, int* error_flag, void* stream) {
  if (dtype != kF16 && dtype != kBF16) return -1;
  if ((lda % 8) || (ldb % 8) || ((uintptr_t)A % 16) || ((uintptr_t)B % 16) || ((uintptr_t)D % 16)) return -3;
  const int bf16 = dtype == kBF16;
  CUtensorMap ma, mb;
  int rc = make_map(&ma, A, bf16, M, K, lda, BM);
  if (rc) return rc;
  rc = make_map(&mb, B, bf16, N, K, ldb, BN);
  if (rc) return rc;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  cudaStream_t st = (cudaStream_t)stream;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(gemm_tn_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    cudaFuncSetAttribute(gemm_tn_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    attr_set = true;
  }
  if (bf16)
    gemm_tn_kernel<__nv_bfloat16><<<grid, kGemmThreads, SMEM_BYTES, st>>>(ma, mb, (__nv_bfloat16*)D, (const __nv_bfloat16*)bias,
                                                                         M, N, K, ldd, act, 1, error_flag);
  else
    gemm_tn_kernel<__half><<<grid, kGemmThreads, SMEM_BYTES, st>>>(ma, mb, (__half*)D, (const __half*)bias, M, N, K, ldd, act,
                                                                  0, error_flag);
  return (int)cudaGetLastError();
}

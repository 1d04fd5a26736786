// Products of a CSR matrix with a dense matrix from the compressed components (sm_100a).
//
// Reference behaviour: DotCsrDnsDns / DotCsrDnsRsp / the transposed forms of src/operator/tensor/dot-inl.cuh (warp and
// thread kernels over the rows of the CSR operand, atomic adds for the transposed product).
// Both kernels are bound by the gather of dense rows, so the work is laid out for coalesced 128-byte reads:
//   out = A B    : one warp per (row of A, tile of 32 * V columns); the warp walks the non-zeros of its row (value and
//                  column index are the same for all lanes: one broadcast load each) and every lane accumulates V
//                  adjacent columns of B[col, :] in fp32 registers; one coalesced store at the end.  No atomics: the
//                  result does not depend on the schedule.
//   out = A^T B  : the same walk, but the products of row r go to out[col, :]; rows of A that share a column collide, so
//                  the accumulation is an fp32 atomic add into a zeroed fp32 buffer (converted by the caller for half
//                  types).  The sum order depends on the schedule, as in the reference kernel.
#include "common.cuh"

namespace mxb {

template <typename T, int V>
__global__ void __launch_bounds__(128)
csr_dot_dense_kernel(const T* __restrict__ vals, const int64_t* __restrict__ idx, const int64_t* __restrict__ ptr,
                     const T* __restrict__ B, T* __restrict__ out, int64_t M, int N) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= M) return;
  const int col0 = (blockIdx.y * 32 + lane) * V;
  float acc[V];
#pragma unroll
  for (int v = 0; v < V; ++v) acc[v] = 0.f;
  const int64_t begin = ptr[row], end = ptr[row + 1];
  for (int64_t j = begin; j < end; ++j) {
    const float a = Cvt<T>::to_f(vals[j]);
    const T* brow = B + idx[j] * (int64_t)N;
#pragma unroll
    for (int v = 0; v < V; ++v)
      if (col0 + v < N) acc[v] += a * Cvt<T>::to_f(brow[col0 + v]);
  }
#pragma unroll
  for (int v = 0; v < V; ++v)
    if (col0 + v < N) out[row * (int64_t)N + col0 + v] = Cvt<T>::from_f(acc[v]);
}

template <typename T, int V>
__global__ void __launch_bounds__(128)
csr_t_dot_dense_kernel(const T* __restrict__ vals, const int64_t* __restrict__ idx, const int64_t* __restrict__ ptr,
                       const T* __restrict__ B, float* __restrict__ out, int64_t M, int N) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= M) return;
  const int col0 = (blockIdx.y * 32 + lane) * V;
  float b[V];
#pragma unroll
  for (int v = 0; v < V; ++v) b[v] = col0 + v < N ? Cvt<T>::to_f(B[row * (int64_t)N + col0 + v]) : 0.f;
  const int64_t begin = ptr[row], end = ptr[row + 1];
  for (int64_t j = begin; j < end; ++j) {
    const float a = Cvt<T>::to_f(vals[j]);
    float* orow = out + idx[j] * (int64_t)N;
#pragma unroll
    for (int v = 0; v < V; ++v)
      if (col0 + v < N) atomicAdd(orow + col0 + v, a * b[v]);
  }
}

template <typename T>
static int csr_launch(bool transposed, const void* vals, const int64_t* idx, const int64_t* ptr, const void* B, void* out, int64_t M,
                      int N, cudaStream_t st) {
  if (M == 0 || N == 0) return 0;
  const int64_t gx = (M + 3) / 4;                  // four rows (warps) per block
  const int V = N > 64 ? 4 : N > 32 ? 2 : 1;      // all 32 lanes of a warp get columns: 64 columns = 32 lanes x 2
  const int64_t gy = ((int64_t)N + 32 * V - 1) / (32 * V);
  if (gx > 0x7fffffffLL || gy > 65535) return -2;
  const dim3 grid((unsigned)gx, (unsigned)gy);
  const T* v = static_cast<const T*>(vals);
  const T* b = static_cast<const T*>(B);
  if (V == 4) {
    if (transposed) csr_t_dot_dense_kernel<T, 4><<<grid, 128, 0, st>>>(v, idx, ptr, b, static_cast<float*>(out), M, N);
    else csr_dot_dense_kernel<T, 4><<<grid, 128, 0, st>>>(v, idx, ptr, b, static_cast<T*>(out), M, N);
  } else if (V == 2) {
    if (transposed) csr_t_dot_dense_kernel<T, 2><<<grid, 128, 0, st>>>(v, idx, ptr, b, static_cast<float*>(out), M, N);
    else csr_dot_dense_kernel<T, 2><<<grid, 128, 0, st>>>(v, idx, ptr, b, static_cast<T*>(out), M, N);
  } else {
    if (transposed) csr_t_dot_dense_kernel<T, 1><<<grid, 128, 0, st>>>(v, idx, ptr, b, static_cast<float*>(out), M, N);
    else csr_dot_dense_kernel<T, 1><<<grid, 128, 0, st>>>(v, idx, ptr, b, static_cast<T*>(out), M, N);
  }
  return (int)cudaGetLastError();
}

}  // namespace mxb

using namespace mxb;

// out[M, N] = csr[M, K] . B[K, N] (transposed = 0), or out32[K, N] += csr[M, K]^T . B[M, N] (transposed = 1; out32 is a zeroed
// fp32 buffer whatever the value type).  Column indices and row pointers are int64; B and out are dense, row-major.
MXB_EXPORT int mxb_csr_dot_dense(int dtype, int transposed, const void* vals, const int64_t* idx, const int64_t* ptr, const void* B,
                                 void* out, long long M, int N, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == kF32) return csr_launch<float>(transposed != 0, vals, idx, ptr, B, out, M, N, st);
  if (dtype == kF16) return csr_launch<__half>(transposed != 0, vals, idx, ptr, B, out, M, N, st);
  if (dtype == kBF16) return csr_launch<__nv_bfloat16>(transposed != 0, vals, idx, ptr, B, out, M, N, st);
  return -1;
}

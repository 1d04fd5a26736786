// 1-bit and 2-bit gradient compression with residual accumulation (sm_100a).
//
// Reference behaviour: quantize_2bit / dequantize_2bit / quantize_1bit / dequantize_1bit functors of
// src/kvstore/gradient_compression-inl.h:45-215 (one generic-kernel thread per packed 32-bit word).
// 2-bit: residual += grad; a value >= threshold sends code 3 and subtracts the threshold from the residual, a value
// <= -threshold sends code 2 and adds it, anything else sends 0.  1-bit: code 1 (and residual -= 1) when the residual
// exceeds the threshold, else code 0 (and residual += 1).  Code j of a word sits at bit j*bits.
// One thread produces one packed word: 16 (or 32) consecutive gradient values are read as 16-byte vectors, the
// residual is updated in place in the same pass, so a gradient is read once and its residual read and written once.
#include "common.cuh"

namespace mxb {

template <int BITS>
__global__ void __launch_bounds__(256)
quantize_kernel(const float* __restrict__ grad, float* __restrict__ residual, uint32_t* __restrict__ packed, int64_t n,
                float threshold) {
  constexpr int PER = 32 / BITS;
  const int64_t words = (n + PER - 1) / PER;
  for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < words; w += (int64_t)gridDim.x * blockDim.x) {
    const int64_t base = w * PER;
    uint32_t word = 0;
    if (base + PER <= n) {
#pragma unroll
      for (int v = 0; v < PER / 4; ++v) {
        const float4 g = *reinterpret_cast<const float4*>(grad + base + v * 4);
        float4 r = *reinterpret_cast<float4*>(residual + base + v * 4);
        float rr[4] = {r.x + g.x, r.y + g.y, r.z + g.z, r.w + g.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t code;
          if (BITS == 2) {
            if (rr[j] >= threshold) { code = 3u; rr[j] -= threshold; }
            else if (rr[j] <= -threshold) { code = 2u; rr[j] += threshold; }
            else code = 0u;
          } else {
            if (rr[j] > threshold) { code = 1u; rr[j] -= 1.f; }
            else { code = 0u; rr[j] += 1.f; }
          }
          word |= code << ((v * 4 + j) * BITS);
        }
        *reinterpret_cast<float4*>(residual + base + v * 4) = make_float4(rr[0], rr[1], rr[2], rr[3]);
      }
    } else {
      for (int j = 0; j < PER && base + j < n; ++j) {
        float r = residual[base + j] + grad[base + j];
        uint32_t code;
        if (BITS == 2) {
          if (r >= threshold) { code = 3u; r -= threshold; }
          else if (r <= -threshold) { code = 2u; r += threshold; }
          else code = 0u;
        } else {
          if (r > threshold) { code = 1u; r -= 1.f; }
          else { code = 0u; r += 1.f; }
        }
        residual[base + j] = r;
        word |= code << (j * BITS);
      }
    }
    packed[w] = word;
  }
}

// out (+)= decoded values; `accumulate` sums the contributions of several senders into one buffer.
template <int BITS>
__global__ void __launch_bounds__(256)
dequantize_kernel(const uint32_t* __restrict__ packed, float* __restrict__ out, int64_t n, float threshold, int accumulate) {
  constexpr int PER = 32 / BITS;
  const int64_t words = (n + PER - 1) / PER;
  for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < words; w += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t word = packed[w];
    const int64_t base = w * PER;
    for (int j = 0; j < PER && base + j < n; ++j) {
      const uint32_t code = (word >> (j * BITS)) & ((1u << BITS) - 1u);
      float v;
      if (BITS == 2) v = code == 3u ? threshold : (code == 2u ? -threshold : 0.f);
      else v = code == 1u ? 1.f : -1.f;
      out[base + j] = accumulate ? out[base + j] + v : v;
    }
  }
}

inline int compress_grid(int64_t words) {
  int64_t blocks = (words + 255) / 256;
  int64_t cap = (int64_t)sm_count() * 8;
  if (blocks < 1) blocks = 1;
  return (int)(blocks < cap ? blocks : cap);
}

}  // namespace mxb

using namespace mxb;

// grad, residual: n floats (16-byte aligned); packed: ceil(n / (32 / bits)) words.  bits: 1 or 2.
MXB_EXPORT int mxb_gc_quantize(int bits, const float* grad, float* residual, uint32_t* packed, int64_t n, float threshold,
                               void* stream) {
  if (n < 1) return -2;
  if (((uintptr_t)grad % 16) || ((uintptr_t)residual % 16)) return -3;
  cudaStream_t st = (cudaStream_t)stream;
  if (bits == 2) quantize_kernel<2><<<compress_grid((n + 15) / 16), 256, 0, st>>>(grad, residual, packed, n, threshold);
  else if (bits == 1) quantize_kernel<1><<<compress_grid((n + 31) / 32), 256, 0, st>>>(grad, residual, packed, n, threshold);
  else return -1;
  return (int)cudaGetLastError();
}

MXB_EXPORT int mxb_gc_dequantize(int bits, const uint32_t* packed, float* out, int64_t n, float threshold, int accumulate,
                                 void* stream) {
  if (n < 1) return -2;
  cudaStream_t st = (cudaStream_t)stream;
  if (bits == 2) dequantize_kernel<2><<<compress_grid((n + 15) / 16), 256, 0, st>>>(packed, out, n, threshold, accumulate);
  else if (bits == 1) dequantize_kernel<1><<<compress_grid((n + 31) / 32), 256, 0, st>>>(packed, out, n, threshold, accumulate);
  else return -1;
  return (int)cudaGetLastError();
}

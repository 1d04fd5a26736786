// Detection operators for sm_100a: ROIAlign forward / backward and the suppression core of box_nms / Proposal.
//
// Reference behaviour: src/operator/contrib/roi_align.cu (RoIAlignForwardKernel / RoIAlignBackwardKernel with the
// bilinear_interpolate boundary rules, sampling_ratio, position_sensitive, aligned) and
// src/operator/contrib/bounding_box-inl.cuh (nms: boxes sorted by score, triangular overlap test, sequential keep scan).
// These are cold-path kernels (one thread per output element, atomics in the ROIAlign backward); what they replace is a
// per-ROI host loop, so the gain is in launches and host synchronisation, not in bandwidth.
#include "common.cuh"

namespace mxb {

constexpr int kDetThreads = 256;

// The sampling point's four neighbours and weights.  Points more than one pixel outside the map contribute nothing;
// points in the one-pixel border are clamped onto the edge (roi_align.cu: bilinear_interpolate).
struct Bilinear {
  int y0, x0, y1, x1;
  float w00, w01, w10, w11;
  bool inside;
};

__device__ __forceinline__ Bilinear bilinear_setup(float y, float x, int H, int W) {
  Bilinear b;
  b.inside = !(y < -1.f || y > (float)H || x < -1.f || x > (float)W);
  if (!b.inside) {
    b.y0 = b.x0 = b.y1 = b.x1 = 0;
    b.w00 = b.w01 = b.w10 = b.w11 = 0.f;
    return b;
  }
  y = fmaxf(y, 0.f);
  x = fmaxf(x, 0.f);
  b.y0 = (int)y;
  b.x0 = (int)x;
  if (b.y0 >= H - 1) { b.y1 = b.y0 = H - 1; y = (float)b.y0; } else { b.y1 = b.y0 + 1; }
  if (b.x0 >= W - 1) { b.x1 = b.x0 = W - 1; x = (float)b.x0; } else { b.x1 = b.x0 + 1; }
  const float ly = y - b.y0, lx = x - b.x0, hy = 1.f - ly, hx = 1.f - lx;
  b.w00 = hy * hx; b.w01 = hy * lx; b.w10 = ly * hx; b.w11 = ly * lx;
  return b;
}

struct RoiGeom {
  int R, C, H, W, PH, PW;       // C: output channels (input channels / (PH*PW) when position sensitive)
  int CI;                       // input channels
  float scale, offset;
  int sample_ratio, position_sensitive, aligned;
};

struct RoiBin {
  int batch;
  float y_start, x_start, bin_h, bin_w;
  int gh, gw;
};

template <typename T>
__device__ __forceinline__ RoiBin roi_bin(const T* __restrict__ rois, int r, const RoiGeom& g) {
  const T* roi = rois + (int64_t)r * 5;
  RoiBin b;
  b.batch = (int)Cvt<T>::to_f(roi[0]);
  const float x1 = Cvt<T>::to_f(roi[1]) * g.scale - g.offset, y1 = Cvt<T>::to_f(roi[2]) * g.scale - g.offset;
  const float x2 = Cvt<T>::to_f(roi[3]) * g.scale - g.offset, y2 = Cvt<T>::to_f(roi[4]) * g.scale - g.offset;
  float rw = x2 - x1, rh = y2 - y1;
  if (!g.aligned) { rw = fmaxf(rw, 1.f); rh = fmaxf(rh, 1.f); }
  b.y_start = y1; b.x_start = x1;
  b.bin_h = rh / g.PH; b.bin_w = rw / g.PW;
  b.gh = g.sample_ratio > 0 ? g.sample_ratio : max((int)ceilf(rh / g.PH), 1);
  b.gw = g.sample_ratio > 0 ? g.sample_ratio : max((int)ceilf(rw / g.PW), 1);
  return b;
}

// one thread per output element (r, c, ph, pw)
template <typename T>
__global__ void __launch_bounds__(kDetThreads)
roi_align_fwd_kernel(const T* __restrict__ data, const T* __restrict__ rois, T* __restrict__ out, RoiGeom g, int64_t total) {
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int pw = idx % g.PW, ph = (idx / g.PW) % g.PH, c = (idx / ((int64_t)g.PW * g.PH)) % g.C, r = idx / ((int64_t)g.PW * g.PH * g.C);
    const RoiBin b = roi_bin(rois, r, g);
    if (b.batch < 0) { out[idx] = Cvt<T>::from_f(0.f); continue; }
    const int ci = g.position_sensitive ? (c * g.PH + ph) * g.PW + pw : c;
    const T* plane = data + ((int64_t)b.batch * g.CI + ci) * g.H * g.W;
    float acc = 0.f;
    for (int iy = 0; iy < b.gh; ++iy) {
      const float y = b.y_start + ph * b.bin_h + (iy + 0.5f) * b.bin_h / b.gh;
      for (int ix = 0; ix < b.gw; ++ix) {
        const float x = b.x_start + pw * b.bin_w + (ix + 0.5f) * b.bin_w / b.gw;
        const Bilinear s = bilinear_setup(y, x, g.H, g.W);
        if (!s.inside) continue;
        acc += s.w00 * Cvt<T>::to_f(plane[s.y0 * g.W + s.x0]) + s.w01 * Cvt<T>::to_f(plane[s.y0 * g.W + s.x1]) +
               s.w10 * Cvt<T>::to_f(plane[s.y1 * g.W + s.x0]) + s.w11 * Cvt<T>::to_f(plane[s.y1 * g.W + s.x1]);
      }
    }
    out[idx] = Cvt<T>::from_f(acc / (float)(b.gh * b.gw));
  }
}

// one thread per output-gradient element; scatters into an fp32 gradient of the input
template <typename T>
__global__ void __launch_bounds__(kDetThreads)
roi_align_bwd_kernel(const T* __restrict__ dout, const T* __restrict__ rois, float* __restrict__ ddata, RoiGeom g, int64_t total) {
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int pw = idx % g.PW, ph = (idx / g.PW) % g.PH, c = (idx / ((int64_t)g.PW * g.PH)) % g.C, r = idx / ((int64_t)g.PW * g.PH * g.C);
    const RoiBin b = roi_bin(rois, r, g);
    if (b.batch < 0) continue;
    const int ci = g.position_sensitive ? (c * g.PH + ph) * g.PW + pw : c;
    float* plane = ddata + ((int64_t)b.batch * g.CI + ci) * g.H * g.W;
    const float go = Cvt<T>::to_f(dout[idx]) / (float)(b.gh * b.gw);
    for (int iy = 0; iy < b.gh; ++iy) {
      const float y = b.y_start + ph * b.bin_h + (iy + 0.5f) * b.bin_h / b.gh;
      for (int ix = 0; ix < b.gw; ++ix) {
        const float x = b.x_start + pw * b.bin_w + (ix + 0.5f) * b.bin_w / b.gw;
        const Bilinear s = bilinear_setup(y, x, g.H, g.W);
        if (!s.inside) continue;
        atomicAdd(plane + s.y0 * g.W + s.x0, go * s.w00);
        atomicAdd(plane + s.y0 * g.W + s.x1, go * s.w01);
        atomicAdd(plane + s.y1 * g.W + s.x0, go * s.w10);
        atomicAdd(plane + s.y1 * g.W + s.x1, go * s.w11);
      }
    }
  }
}

// ---- non-maximum suppression ----------------------------------------------------------------------------------------
// boxes [n][4] corner format, sorted by descending score; ids [n] class of each box or null.  mask [n][words]: bit j of
// row i set when box j (j > i) overlaps box i by more than `thresh` (and has the same id unless ids is null).
// `e`: 0 for continuous coordinates (box_nms), 1 for the inclusive-pixel convention of the region-proposal operators.
__device__ __forceinline__ float iou_corner(const float4 a, const float4 b, float e) {
  const float w = fmaxf(fminf(a.z, b.z) - fmaxf(a.x, b.x) + e, 0.f), h = fmaxf(fminf(a.w, b.w) - fmaxf(a.y, b.y) + e, 0.f);
  const float inter = w * h;
  const float uni = (a.z - a.x + e) * (a.w - a.y + e) + (b.z - b.x + e) * (b.w - b.y + e) - inter;
  return inter / fmaxf(uni, 1e-12f);
}

__global__ void __launch_bounds__(64)
nms_mask_kernel(const float* __restrict__ boxes, const float* __restrict__ ids, unsigned long long* __restrict__ mask, int n,
                int words, float thresh, float extent) {
  const int row_blk = blockIdx.y, col_blk = blockIdx.x;
  if (col_blk < row_blk) return;                         // only j > i matters
  __shared__ float4 cb[64];
  __shared__ float cid[64];
  const int cj = col_blk * 64 + threadIdx.x;
  if (cj < n) {
    cb[threadIdx.x] = reinterpret_cast<const float4*>(boxes)[cj];
    cid[threadIdx.x] = ids ? ids[cj] : 0.f;
  }
  __syncthreads();
  const int i = row_blk * 64 + threadIdx.x;
  if (i >= n) return;
  const float4 a = reinterpret_cast<const float4*>(boxes)[i];
  const float aid = ids ? ids[i] : 0.f;
  unsigned long long bits = 0ull;
  const int cols = min(64, n - col_blk * 64);
  for (int k = 0; k < cols; ++k) {
    const int j = col_blk * 64 + k;
    if (j <= i) continue;
    if (ids && cid[k] != aid) continue;
    if (iou_corner(a, cb[k], extent) > thresh) bits |= 1ull << k;
  }
  mask[(int64_t)i * words + col_blk] = bits;
}

// Sequential scan in score order by one CTA: box i is kept when no kept box before it suppressed it.
// keep [n] bytes (1 = kept); at most `max_keep` boxes are kept (<= 0: no limit).
__global__ void __launch_bounds__(kDetThreads)
nms_scan_kernel(const unsigned long long* __restrict__ mask, unsigned char* __restrict__ keep, int n, int words, int max_keep) {
  extern __shared__ unsigned long long removed[];        // [words]
  for (int w = threadIdx.x; w < words; w += blockDim.x) removed[w] = 0ull;
  __shared__ int kept_count;
  if (threadIdx.x == 0) kept_count = 0;
  __syncthreads();
  for (int i = 0; i < n; ++i) {
    const bool gone = (removed[i >> 6] >> (i & 63)) & 1ull;
    const bool full = max_keep > 0 && kept_count >= max_keep;
    __syncthreads();                                     // every thread has read the state of box i
    if (gone || full) {
      if (threadIdx.x == 0) keep[i] = 0;
      continue;
    }
    if (threadIdx.x == 0) { keep[i] = 1; kept_count += 1; }
    for (int w = (i >> 6) + threadIdx.x; w < words; w += blockDim.x) removed[w] |= mask[(int64_t)i * words + w];
    __syncthreads();
  }
}

template <typename T>
static int roi_align_launch(bool backward, const void* a, const void* rois, void* out, const RoiGeom& g, cudaStream_t st) {
  const int64_t total = (int64_t)g.R * g.C * g.PH * g.PW;
  if (total == 0) return 0;
  const int blocks = (int)((total + kDetThreads - 1) / kDetThreads < 148 * 16 ? (total + kDetThreads - 1) / kDetThreads : 148 * 16);
  if (backward)
    roi_align_bwd_kernel<T><<<blocks, kDetThreads, 0, st>>>(static_cast<const T*>(a), static_cast<const T*>(rois),
                                                            static_cast<float*>(out), g, total);
  else
    roi_align_fwd_kernel<T><<<blocks, kDetThreads, 0, st>>>(static_cast<const T*>(a), static_cast<const T*>(rois),
                                                            static_cast<T*>(out), g, total);
  return (int)cudaGetLastError();
}

}  // namespace mxb

using namespace mxb;

static RoiGeom make_geom(int R, int CI, int H, int W, int PH, int PW, float scale, int sample_ratio, int position_sensitive,
                         int aligned) {
  RoiGeom g;
  g.R = R; g.CI = CI; g.H = H; g.W = W; g.PH = PH; g.PW = PW;
  g.C = position_sensitive ? CI / (PH * PW) : CI;
  g.scale = scale; g.offset = aligned ? 0.5f : 0.f;
  g.sample_ratio = sample_ratio; g.position_sensitive = position_sensitive; g.aligned = aligned;
  return g;
}

// data [N, CI, H, W], rois [R, 5] (batch index, x1, y1, x2, y2) in the data type, out [R, C, PH, PW].
MXB_EXPORT int mxb_roi_align_forward(int dtype, const void* data, const void* rois, void* out, int R, int CI, int H, int W,
                                     int PH, int PW, float scale, int sample_ratio, int position_sensitive, int aligned,
                                     void* stream) {
  if (PH < 1 || PW < 1 || H < 1 || W < 1 || (position_sensitive && CI % (PH * PW))) return -2;
  const RoiGeom g = make_geom(R, CI, H, W, PH, PW, scale, sample_ratio, position_sensitive, aligned);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == kF32) return roi_align_launch<float>(false, data, rois, out, g, st);
  if (dtype == kF16) return roi_align_launch<__half>(false, data, rois, out, g, st);
  if (dtype == kBF16) return roi_align_launch<__nv_bfloat16>(false, data, rois, out, g, st);
  return -1;
}

// dout [R, C, PH, PW] in the data type; ddata [N, CI, H, W] fp32, zero-initialised by the caller (accumulated into).
MXB_EXPORT int mxb_roi_align_backward(int dtype, const void* dout, const void* rois, float* ddata, int R, int CI, int H, int W,
                                      int PH, int PW, float scale, int sample_ratio, int position_sensitive, int aligned,
                                      void* stream) {
  if (PH < 1 || PW < 1 || H < 1 || W < 1 || (position_sensitive && CI % (PH * PW))) return -2;
  const RoiGeom g = make_geom(R, CI, H, W, PH, PW, scale, sample_ratio, position_sensitive, aligned);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == kF32) return roi_align_launch<float>(true, dout, rois, ddata, g, st);
  if (dtype == kF16) return roi_align_launch<__half>(true, dout, rois, ddata, g, st);
  if (dtype == kBF16) return roi_align_launch<__nv_bfloat16>(true, dout, rois, ddata, g, st);
  return -1;
}

// Number of 64-bit words per row of the suppression mask for n boxes.
MXB_EXPORT int mxb_nms_words(int n) { return (n + 63) / 64; }

// boxes [n, 4] fp32 corner format sorted by descending score (16-byte aligned), ids [n] fp32 or null, mask scratch of
// n * mxb_nms_words(n) 64-bit words, keep [n] bytes.  `extent`: 0, or 1 for inclusive pixel coordinates.
MXB_EXPORT int mxb_nms(const float* boxes, const float* ids, unsigned long long* mask, unsigned char* keep, int n, float thresh,
                       float extent, int max_keep, void* stream) {
  if (n <= 0) return 0;
  const int words = (n + 63) / 64;
  if ((size_t)words * 8 > 48 * 1024) return -4;           // 393,216 boxes: beyond that the scan's state leaves shared memory
  cudaStream_t st = (cudaStream_t)stream;
  cudaMemsetAsync(mask, 0, (size_t)n * words * 8, st);
  nms_mask_kernel<<<dim3(words, words), 64, 0, st>>>(boxes, ids, mask, n, words, thresh, extent);
  nms_scan_kernel<<<1, kDetThreads, (size_t)words * 8, st>>>(mask, keep, n, words, max_keep);
  return (int)cudaGetLastError();
}

// Image input pipeline on the GPU: JPEG decode (nvJPEG, loaded at run time) and one augmentation kernel that turns the
// decoded images into the training batch.
//
// Reference: src/io/iter_image_recordio_2.cc (ImageRecordIOParser2: OpenCV decode on `preprocess_threads` host threads),
// src/io/image_aug_default.cc (resize, random / centre crop, mirror), src/io/iter_normalize.h (mean / std / scale), then a
// host-to-device copy of the float batch.  Here only the COMPRESSED bytes cross to the device: the images are decoded
// there into one packed uint8 buffer, and a single kernel reads each crop rectangle with bilinear resampling, mirrors,
// normalises, casts to the training dtype and writes NHWC or NCHW, so the float batch is written once and never copied.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nvjpeg.h>

#include <atomic>
#include <mutex>
#include <thread>
#include <vector>

#include "common.cuh"

namespace mxb {

// ---- nvJPEG through dlopen: the kernel library must load on machines without it ------------------------------------------
struct NvJpegApi {
  void* lib = nullptr;
  nvjpegStatus_t (*CreateSimple)(nvjpegHandle_t*) = nullptr;
  nvjpegStatus_t (*Destroy)(nvjpegHandle_t) = nullptr;
  nvjpegStatus_t (*JpegStateCreate)(nvjpegHandle_t, nvjpegJpegState_t*) = nullptr;
  nvjpegStatus_t (*JpegStateDestroy)(nvjpegJpegState_t) = nullptr;
  nvjpegStatus_t (*GetImageInfo)(nvjpegHandle_t, const unsigned char*, size_t, int*, nvjpegChromaSubsampling_t*, int*, int*) = nullptr;
  nvjpegStatus_t (*Decode)(nvjpegHandle_t, nvjpegJpegState_t, const unsigned char*, size_t, nvjpegOutputFormat_t, nvjpegImage_t*,
                           cudaStream_t) = nullptr;
  bool ok = false;
};

static NvJpegApi& nvjpeg_api() {
  static NvJpegApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    for (const char* name : {"libnvjpeg.so.12", "libnvjpeg.so"}) {
      api.lib = dlopen(name, RTLD_NOW | RTLD_LOCAL);
      if (api.lib) break;
    }
    if (!api.lib) return;
    auto sym = [&](const char* n) { return dlsym(api.lib, n); };
    api.CreateSimple = (decltype(api.CreateSimple))sym("nvjpegCreateSimple");
    api.Destroy = (decltype(api.Destroy))sym("nvjpegDestroy");
    api.JpegStateCreate = (decltype(api.JpegStateCreate))sym("nvjpegJpegStateCreate");
    api.JpegStateDestroy = (decltype(api.JpegStateDestroy))sym("nvjpegJpegStateDestroy");
    api.GetImageInfo = (decltype(api.GetImageInfo))sym("nvjpegGetImageInfo");
    api.Decode = (decltype(api.Decode))sym("nvjpegDecode");
    api.ok = api.CreateSimple && api.Destroy && api.JpegStateCreate && api.JpegStateDestroy && api.GetImageInfo && api.Decode;
  });
  return api;
}

// One nvJPEG handle, and per worker thread a decoder state and a stream: the entropy decoding of the default back end runs
// on the host inside nvjpegDecode, so a batch is spread over several host threads, each feeding its own stream.
struct JpegDecoder {
  nvjpegHandle_t handle = nullptr;
  std::vector<nvjpegJpegState_t> states;
  std::vector<cudaStream_t> streams;
  std::vector<cudaEvent_t> events;
  int device = 0;
};

// ---- augmentation kernel ----------------------------------------------------------------------------------------------------
struct AugImage {
  long long offset;        // byte offset of the decoded image (uint8, HWC, 3 channels, rows packed) in the source buffer
  int width, height;       // decoded size
  float x0, y0, cw, ch;    // crop rectangle in source pixels (may be fractional)
  int mirror;              // 1: flip left-right
};

// One thread per output pixel (all channels).  Sample position: pixel centres, as OpenCV's INTER_LINEAR and PIL's bilinear
// use for up-sampling (src = (dst + 0.5) * scale - 0.5, clamped to the image).
template <typename T>
__global__ void __launch_bounds__(256)
image_augment_kernel(const unsigned char* __restrict__ src, const AugImage* __restrict__ imgs, T* __restrict__ out, int n, int H, int W,
                     int nhwc, float mean0, float mean1, float mean2, float istd0, float istd1, float istd2, float scale) {
  const int img = blockIdx.y;
  const int pix = blockIdx.x * blockDim.x + threadIdx.x;
  if (img >= n || pix >= H * W) return;
  const AugImage a = imgs[img];
  const int oy = pix / W, ox = pix - oy * W;
  const int sx_out = a.mirror ? (W - 1 - ox) : ox;
  float fx = a.x0 + (sx_out + 0.5f) * (a.cw / W) - 0.5f;
  float fy = a.y0 + (oy + 0.5f) * (a.ch / H) - 0.5f;
  fx = fminf(fmaxf(fx, 0.f), (float)(a.width - 1));
  fy = fminf(fmaxf(fy, 0.f), (float)(a.height - 1));
  const int x0 = (int)fx, y0 = (int)fy;
  const int x1 = min(x0 + 1, a.width - 1), y1 = min(y0 + 1, a.height - 1);
  const float wx = fx - x0, wy = fy - y0;
  const unsigned char* base = src + a.offset;
  const size_t pitch = (size_t)a.width * 3;
  const unsigned char* p00 = base + y0 * pitch + (size_t)x0 * 3;
  const unsigned char* p01 = base + y0 * pitch + (size_t)x1 * 3;
  const unsigned char* p10 = base + y1 * pitch + (size_t)x0 * 3;
  const unsigned char* p11 = base + y1 * pitch + (size_t)x1 * 3;
  const float mean[3] = {mean0, mean1, mean2};
  const float istd[3] = {istd0, istd1, istd2};
#pragma unroll
  for (int c = 0; c < 3; ++c) {
    const float top = p00[c] + wx * ((float)p01[c] - (float)p00[c]);
    const float bot = p10[c] + wx * ((float)p11[c] - (float)p10[c]);
    const float v = ((top + wy * (bot - top)) - mean[c]) * istd[c] * scale;
    const size_t o = nhwc ? (((size_t)img * H + oy) * W + ox) * 3 + c : (((size_t)img * 3 + c) * H + oy) * W + ox;
    out[o] = Cvt<T>::from_f(v);
  }
}

}  // namespace mxb

using namespace mxb;

// 1 when nvJPEG could be loaded.
MXB_EXPORT int mxb_jpeg_available() { return nvjpeg_api().ok ? 1 : 0; }

// A decoder bound to the current device with `threads` host workers (at least 1); null on failure.
MXB_EXPORT void* mxb_jpeg_decoder_create(int threads) {
  NvJpegApi& api = nvjpeg_api();
  if (!api.ok) return nullptr;
  JpegDecoder* d = new JpegDecoder();
  cudaGetDevice(&d->device);
  if (api.CreateSimple(&d->handle) != NVJPEG_STATUS_SUCCESS) { delete d; return nullptr; }
  if (threads < 1) threads = 1;
  if (threads > 32) threads = 32;
  for (int i = 0; i < threads; ++i) {
    nvjpegJpegState_t st = nullptr;
    cudaStream_t cs = nullptr;
    cudaEvent_t ev = nullptr;
    if (api.JpegStateCreate(d->handle, &st) != NVJPEG_STATUS_SUCCESS || cudaStreamCreateWithFlags(&cs, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) {
      if (st) api.JpegStateDestroy(st);
      if (cs) cudaStreamDestroy(cs);
      break;
    }
    d->states.push_back(st);
    d->streams.push_back(cs);
    d->events.push_back(ev);
  }
  if (d->states.empty()) { api.Destroy(d->handle); delete d; return nullptr; }
  return d;
}

MXB_EXPORT void mxb_jpeg_decoder_destroy(void* dec) {
  JpegDecoder* d = static_cast<JpegDecoder*>(dec);
  if (!d) return;
  NvJpegApi& api = nvjpeg_api();
  for (size_t i = 0; i < d->states.size(); ++i) {
    cudaStreamSynchronize(d->streams[i]);
    api.JpegStateDestroy(d->states[i]);
    cudaStreamDestroy(d->streams[i]);
    cudaEventDestroy(d->events[i]);
  }
  if (d->handle) api.Destroy(d->handle);
  delete d;
}

// Width, height and number of components of `n` JPEG streams (host pointers).  Returns 0, or 100 + the index of the first
// stream that is not a readable JPEG.
MXB_EXPORT int mxb_jpeg_info_batch(void* dec, int n, const unsigned char* const* bufs, const long long* lens, int* widths, int* heights,
                                   int* comps) {
  JpegDecoder* d = static_cast<JpegDecoder*>(dec);
  NvJpegApi& api = nvjpeg_api();
  if (!d || !api.ok) return -1;
  for (int i = 0; i < n; ++i) {
    int nc = 0, w[NVJPEG_MAX_COMPONENT] = {0}, h[NVJPEG_MAX_COMPONENT] = {0};
    nvjpegChromaSubsampling_t ss;
    if (api.GetImageInfo(d->handle, bufs[i], (size_t)lens[i], &nc, &ss, w, h) != NVJPEG_STATUS_SUCCESS) return 100 + i;
    widths[i] = w[0];
    heights[i] = h[0];
    comps[i] = nc;
  }
  return 0;
}

// Decode `n` JPEG streams into `out` (device memory) as interleaved RGB, image i at byte offset offsets[i] with rows of
// 3 * widths[i] bytes.  The images are spread over the decoder's worker threads and streams; those streams first wait for
// `stream` (the buffer may still be read by earlier work there) and `stream` then waits for all of them.  Returns 0, or
// 100 + the index of a stream that failed.
MXB_EXPORT int mxb_jpeg_decode_batch(void* dec, int n, const unsigned char* const* bufs, const long long* lens, unsigned char* out,
                                     const long long* offsets, const int* widths, void* stream) {
  JpegDecoder* d = static_cast<JpegDecoder*>(dec);
  NvJpegApi& api = nvjpeg_api();
  if (!d || !api.ok) return -1;
  cudaStream_t user = (cudaStream_t)stream;
  const int workers = (int)std::min<size_t>(d->states.size(), (size_t)n);
  cudaEvent_t start = d->events[0];
  cudaEventRecord(start, user);
  for (int w = 0; w < workers; ++w) cudaStreamWaitEvent(d->streams[w], start, 0);
  std::atomic<int> failed(-1);
  auto work = [&](int w) {
    cudaSetDevice(d->device);
    for (int i = w; i < n; i += workers) {
      nvjpegImage_t img = {};
      img.channel[0] = out + offsets[i];
      img.pitch[0] = (size_t)widths[i] * 3;
      if (api.Decode(d->handle, d->states[w], bufs[i], (size_t)lens[i], NVJPEG_OUTPUT_RGBI, &img, d->streams[w]) != NVJPEG_STATUS_SUCCESS) {
        int expect = -1;
        failed.compare_exchange_strong(expect, i);
        return;
      }
    }
  };
  std::vector<std::thread> pool;
  for (int w = 1; w < workers; ++w) pool.emplace_back(work, w);
  work(0);
  for (auto& t : pool) t.join();
  for (int w = 0; w < workers; ++w) {
    cudaEventRecord(d->events[w], d->streams[w]);
    cudaStreamWaitEvent(user, d->events[w], 0);
  }
  return failed.load() >= 0 ? 100 + failed.load() : 0;
}

// Crop + bilinear resize + mirror + normalise + cast + layout for a batch.  `imgs`: device array of n records
// {int64 offset, int32 width, height, float x0, y0, cw, ch, int32 mirror, int32 padding} (40 bytes each).  out: [n, H, W, 3] (nhwc = 1) or
// [n, 3, H, W] of `dtype`.  value = (pixel - mean[c]) / std[c] * scale.
MXB_EXPORT int mxb_image_augment_batch(int dtype, const void* src, const void* imgs, void* out, int n, int H, int W, int nhwc,
                                       const float* mean, const float* std, float scale, void* stream) {
  if (n < 1 || H < 1 || W < 1) return -2;
  static_assert(sizeof(AugImage) == 40, "record layout shared with the Python side");
  dim3 grid((H * W + 255) / 256, n);
  cudaStream_t st = (cudaStream_t)stream;
  const float i0 = 1.f / std[0], i1 = 1.f / std[1], i2 = 1.f / std[2];
  const AugImage* a = static_cast<const AugImage*>(imgs);
  const unsigned char* s = static_cast<const unsigned char*>(src);
  if (dtype == kF32)
    image_augment_kernel<float><<<grid, 256, 0, st>>>(s, a, (float*)out, n, H, W, nhwc, mean[0], mean[1], mean[2], i0, i1, i2, scale);
  else if (dtype == kF16)
    image_augment_kernel<__half><<<grid, 256, 0, st>>>(s, a, (__half*)out, n, H, W, nhwc, mean[0], mean[1], mean[2], i0, i1, i2, scale);
  else
    image_augment_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(s, a, (__nv_bfloat16*)out, n, H, W, nhwc, mean[0], mean[1], mean[2], i0, i1,
                                                             i2, scale);
  return (int)cudaGetLastError();
}

MXB_EXPORT int mxb_image_aug_record_bytes() { return (int)sizeof(mxb::AugImage); }

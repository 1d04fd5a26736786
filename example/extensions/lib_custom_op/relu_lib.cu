// An operator library with one operator that runs on the host and on the GPU:
//   my_relu(data)      max(x, 0) for float32, forward and backward; on a GPU the kernels are enqueued on the stream the
//                      framework passes in
// Build:   nvcc -O2 -shared -Xcompiler -fPIC -gencode arch=compute_100a,code=sm_100a -I<include dir> relu_lib.cu -o librelu_lib.so
// Load:    mx.library.load('/abs/path/librelu_lib.so');  mx.nd.my_relu(x)
#include <cuda_runtime.h>

#include <string>

#include "mxb_lib_api.h"

namespace {

std::string last_error;

int64_t count(const MXBTensor& t) {
  int64_t n = 1;
  for (int i = 0; i < t.ndim; ++i) n *= t.shape[i];
  return n;
}

__global__ void relu_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    y[i] = fmaxf(x[i], 0.f);
}

__global__ void relu_bwd_kernel(const float* __restrict__ dy, const float* __restrict__ x, float* __restrict__ dx, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    dx[i] = x[i] > 0.f ? dy[i] : 0.f;
}

int grid_for(int64_t n) {
  const int64_t blocks = (n + 255) / 256;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > 148 * 8 ? 148 * 8 : blocks));
}

int relu_infer_type(const MXBAttrs*, int32_t, const int32_t* in_types, int32_t, int32_t* out_types) {
  if (in_types[0] != kMXBFloat32) {
    last_error = "my_relu is float32 only";
    return 1;
  }
  out_types[0] = kMXBFloat32;
  return 0;
}

int relu_forward(const MXBAttrs*, int32_t, const MXBTensor* in, int32_t, MXBTensor* out, void* stream, MXBOpState) {
  const int64_t n = count(in[0]);
  const float* x = static_cast<const float*>(in[0].data);
  float* y = static_cast<float*>(out[0].data);
  if (in[0].dev_type == kMXBGPU) {
    if (n > 0) relu_fwd_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, y, n);
    return cudaGetLastError() == cudaSuccess ? 0 : 2;
  }
  for (int64_t i = 0; i < n; ++i) y[i] = x[i] > 0.f ? x[i] : 0.f;
  return 0;
}

int relu_backward(const MXBAttrs*, int32_t, const MXBTensor* ograds, int32_t, const MXBTensor* in, const MXBTensor*,
                  MXBTensor* igrads, void* stream, MXBOpState) {
  const int64_t n = count(in[0]);
  const float* dy = static_cast<const float*>(ograds[0].data);
  const float* x = static_cast<const float*>(in[0].data);
  float* dx = static_cast<float*>(igrads[0].data);
  if (in[0].dev_type == kMXBGPU) {
    if (n > 0) relu_bwd_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(dy, x, dx, n);
    return cudaGetLastError() == cudaSuccess ? 0 : 2;
  }
  for (int64_t i = 0; i < n; ++i) dx[i] = x[i] > 0.f ? dy[i] : 0.f;
  return 0;
}

// shape: same as the input (infer_shape left NULL)
const MXBOpDesc kOps[] = {
    {"my_relu", "max(x, 0) on the host or the GPU (example operator library)", 1, 1, nullptr, nullptr, relu_infer_type,
     relu_forward, relu_backward, nullptr, nullptr},
};

}  // namespace

extern "C" {
int mxb_lib_api_version(void) { return MXB_LIB_API_VERSION; }
int mxb_lib_num_ops(void) { return 1; }
const MXBOpDesc* mxb_lib_op(int index) { return &kOps[index]; }
const char* mxb_lib_last_error(void) { return last_error.c_str(); }
}

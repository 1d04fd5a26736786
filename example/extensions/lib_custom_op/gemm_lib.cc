// An operator library with two operators on the C ABI of mxb_lib_api.h:
//   my_gemm(A, B)          C = A x B for 2-D float32 matrices, with a backward pass
//   my_state_gemm(A, B)    the same product through a per-call state that counts its forward calls ("count" attribute
//                          gives the start value); shows create_state / destroy_state
// Build:   g++ -O2 -shared -fPIC -I<include dir> gemm_lib.cc -o libgemm_lib.so
// Load:    mx.library.load('/abs/path/libgemm_lib.so');  mx.nd.my_gemm(a, b)
#include <cstdlib>
#include <cstring>
#include <string>

#include "mxb_lib_api.h"

namespace {

std::string last_error;

int fail(const char* msg) {
  last_error = msg;
  return 1;
}

// C[n x m] = op(A) x op(B) with explicit leading extents; plain loops: this is an example, not a fast GEMM
void matmul(const float* a, const float* b, float* c, int64_t n, int64_t k, int64_t m, bool a_t, bool b_t) {
  for (int64_t i = 0; i < n; ++i)
    for (int64_t j = 0; j < m; ++j) {
      float acc = 0.f;
      for (int64_t x = 0; x < k; ++x) {
        const float av = a_t ? a[x * n + i] : a[i * k + x];
        const float bv = b_t ? b[j * k + x] : b[x * m + j];
        acc += av * bv;
      }
      c[i * m + j] = acc;
    }
}

int gemm_infer_shape(const MXBAttrs*, int32_t nin, const int64_t* const* in_shapes, const int32_t* in_ndims, int32_t nout,
                     int64_t* const* out_shapes, int32_t* out_ndims) {
  if (nin != 2 || nout != 1) return fail("my_gemm takes two inputs and gives one output");
  if (in_ndims[0] != 2 || in_ndims[1] != 2) return fail("my_gemm takes 2-D matrices");
  if (in_shapes[0][1] != in_shapes[1][0]) return fail("my_gemm: inner extents differ");
  out_shapes[0][0] = in_shapes[0][0];
  out_shapes[0][1] = in_shapes[1][1];
  out_ndims[0] = 2;
  return 0;
}

int gemm_infer_type(const MXBAttrs*, int32_t, const int32_t* in_types, int32_t, int32_t* out_types) {
  if (in_types[0] != kMXBFloat32 || in_types[1] != kMXBFloat32) return fail("my_gemm is float32 only");
  out_types[0] = kMXBFloat32;
  return 0;
}

int gemm_forward(const MXBAttrs*, int32_t, const MXBTensor* in, int32_t, MXBTensor* out, void*, MXBOpState) {
  if (in[0].dev_type != kMXBCPU) return fail("my_gemm runs on the host only");
  matmul(static_cast<const float*>(in[0].data), static_cast<const float*>(in[1].data), static_cast<float*>(out[0].data),
         in[0].shape[0], in[0].shape[1], in[1].shape[1], false, false);
  return 0;
}

// dA = dC x Bt, dB = At x dC
int gemm_backward(const MXBAttrs*, int32_t, const MXBTensor* ograds, int32_t, const MXBTensor* in, const MXBTensor*,
                  MXBTensor* igrads, void*, MXBOpState) {
  const int64_t n = in[0].shape[0], k = in[0].shape[1], m = in[1].shape[1];
  const float* dc = static_cast<const float*>(ograds[0].data);
  matmul(dc, static_cast<const float*>(in[1].data), static_cast<float*>(igrads[0].data), n, m, k, false, true);
  matmul(static_cast<const float*>(in[0].data), dc, static_cast<float*>(igrads[1].data), k, n, m, true, false);
  return 0;
}

struct CountState {
  long calls;
};

int state_create(const MXBAttrs* attrs, MXBOpState* state) {
  CountState* s = new CountState{0};
  for (int i = 0; i < attrs->num; ++i)
    if (std::strcmp(attrs->keys[i], "count") == 0) s->calls = std::atol(attrs->vals[i]);
  *state = s;
  return 0;
}

void state_destroy(MXBOpState state) { delete static_cast<CountState*>(state); }

int state_infer_shape(const MXBAttrs* attrs, int32_t nin, const int64_t* const* in_shapes, const int32_t* in_ndims,
                      int32_t, int64_t* const* out_shapes, int32_t* out_ndims) {
  int64_t* gemm_out[1] = {out_shapes[0]};
  if (int rc = gemm_infer_shape(attrs, nin, in_shapes, in_ndims, 1, gemm_out, out_ndims)) return rc;
  out_shapes[1][0] = 1;          // second output: the call counter
  out_ndims[1] = 1;
  return 0;
}

int state_infer_type(const MXBAttrs*, int32_t, const int32_t*, int32_t, int32_t* out_types) {
  out_types[0] = kMXBFloat32;
  out_types[1] = kMXBInt64;
  return 0;
}

int state_forward(const MXBAttrs* attrs, int32_t nin, const MXBTensor* in, int32_t, MXBTensor* out, void* stream,
                  MXBOpState state) {
  CountState* s = static_cast<CountState*>(state);
  if (s == nullptr) return fail("my_state_gemm called without its state");
  s->calls += 1;
  static_cast<int64_t*>(out[1].data)[0] = s->calls;
  return gemm_forward(attrs, nin, in, 1, out, stream, nullptr);
}

const char* const kGemmInputs[] = {"A", "B"};

const MXBOpDesc kOps[] = {
    {"my_gemm", "C = A x B for 2-D float32 matrices (example operator library)", 2, 1, kGemmInputs, gemm_infer_shape,
     gemm_infer_type, gemm_forward, gemm_backward, nullptr, nullptr},
    {"my_state_gemm", "A x B plus the number of calls seen by this call's state", 2, 2, kGemmInputs, state_infer_shape,
     state_infer_type, state_forward, nullptr, state_create, state_destroy},
};

}  // namespace

extern "C" {
int mxb_lib_api_version(void) { return MXB_LIB_API_VERSION; }
int mxb_lib_init(int framework_version) { return framework_version >= 0 ? 0 : 1; }
int mxb_lib_num_ops(void) { return static_cast<int>(sizeof(kOps) / sizeof(kOps[0])); }
const MXBOpDesc* mxb_lib_op(int index) { return &kOps[index]; }
const char* mxb_lib_last_error(void) { return last_error.c_str(); }
}

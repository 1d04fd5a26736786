/*
 * C ABI of operator libraries loaded at run time with mxnet_b200.library.load("/abs/path/libfoo.so").
 *
 * The role of include/mxnet/lib_api.h in the reference (MXLoadLib, src/c_api/c_api.cc): a shared object built
 * outside the framework adds operators that then appear as mx.nd.<name>, mx.sym.<name> and mx.npx.<name>, take part
 * in autograd, in symbolic shape/type inference and in hybridized blocks.  The ABI is plain C so that the library
 * may be written in C, C++ or CUDA and does not depend on the framework's headers, compiler or C++ runtime.
 *
 * A library exports
 *     int                mxb_lib_api_version(void);      must return MXB_LIB_API_VERSION
 *     int                mxb_lib_num_ops(void);
 *     const MXBOpDesc*   mxb_lib_op(int index);          descriptors live as long as the library
 * and optionally
 *     int                mxb_lib_init(int framework_version);     called once after loading; non-zero = refuse
 *     const char*        mxb_lib_last_error(void);                text for the last non-zero return
 *     int                mxb_lib_num_passes(void);                graph passes, usable as
 *     const MXBPassDesc* mxb_lib_pass(int index);                 Symbol.optimize_for("<pass name>", ...)
 *
 * Every callback returns 0 on success.  Tensors are dense, row-major and contiguous.  For tensors on a GPU the
 * callbacks receive the CUDA stream (a cudaStream_t) on which the framework ordered the inputs; the work must be
 * enqueued on that stream and must not synchronise the device.
 */
#ifndef MXB_LIB_API_H_
#define MXB_LIB_API_H_

#include <stdint.h>

#define MXB_LIB_API_VERSION 1
#define MXB_MAX_NDIM 8

#ifdef __cplusplus
extern "C" {
#endif

/* element types: the framework's on-disk type flags */
enum MXBDType {
  kMXBFloat32 = 0, kMXBFloat64 = 1, kMXBFloat16 = 2, kMXBUint8 = 3, kMXBInt32 = 4, kMXBInt8 = 5, kMXBInt64 = 6,
  kMXBBool = 7, kMXBInt16 = 8, kMXBBFloat16 = 12
};

enum MXBDevType { kMXBCPU = 1, kMXBGPU = 2 };

typedef struct MXBTensor {
  void* data;                 /* host or device pointer, by dev_type */
  int64_t shape[MXB_MAX_NDIM];
  int32_t ndim;
  int32_t dtype;              /* MXBDType */
  int32_t dev_type;           /* MXBDevType */
  int32_t dev_id;
} MXBTensor;

/* attributes of one call: parallel arrays of keys and values, all values as text ("3", "(2, 2)", "True") */
typedef struct MXBAttrs {
  int32_t num;
  const char* const* keys;
  const char* const* vals;
} MXBAttrs;

/* opaque per-call-site state of a stateful operator */
typedef void* MXBOpState;

typedef struct MXBOpDesc {
  const char* name;
  const char* doc;            /* may be NULL */
  int32_t num_inputs;
  int32_t num_outputs;
  /* names of the array inputs, num_inputs entries (NULL: data0, data1, ...) */
  const char* const* input_names;

  /* out_shapes[i] has room for MXB_MAX_NDIM extents.  NULL: every output has the shape of input 0. */
  int (*infer_shape)(const MXBAttrs* attrs, int32_t nin, const int64_t* const* in_shapes, const int32_t* in_ndims,
                     int32_t nout, int64_t* const* out_shapes, int32_t* out_ndims);
  /* NULL: every output has the type of input 0 */
  int (*infer_type)(const MXBAttrs* attrs, int32_t nin, const int32_t* in_types, int32_t nout, int32_t* out_types);

  /* outputs are allocated by the framework from the inferred shapes and types */
  int (*forward)(const MXBAttrs* attrs, int32_t nin, const MXBTensor* inputs, int32_t nout, MXBTensor* outputs,
                 void* stream, MXBOpState state);
  /* NULL: the operator is not differentiable.  in_grads[i] is the gradient of input i (same shape and type as the
   * input, allocated by the framework, to be overwritten).  The call sees the output gradients, the forward inputs
   * and the forward outputs. */
  int (*backward)(const MXBAttrs* attrs, int32_t nout, const MXBTensor* out_grads, int32_t nin, const MXBTensor* inputs,
                  const MXBTensor* outputs, MXBTensor* in_grads, void* stream, MXBOpState state);

  /* stateful operators (both NULL otherwise): a state is created per call and handed to forward and backward of
   * that call, then destroyed when its autograd record is released */
  int (*create_state)(const MXBAttrs* attrs, MXBOpState* state);
  void (*destroy_state)(MXBOpState state);
} MXBOpDesc;

/* A graph pass: rewrites a Symbol given in the framework's JSON form ("nodes", "arg_nodes", "heads").  On success
 * *out_json points to a NUL-terminated text owned by the library that stays valid until the next call into the library
 * from the same thread.  Options are the keyword arguments of optimize_for, as text. */
typedef struct MXBPassDesc {
  const char* name;
  int (*run)(const char* graph_json, const MXBAttrs* options, const char** out_json);
} MXBPassDesc;

#ifdef __cplusplus
}  /* extern "C" */
#endif
#endif  /* MXB_LIB_API_H_ */

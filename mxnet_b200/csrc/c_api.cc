// C interface of the native runtime (declared in include/mxnet_b200/c_api.h): arrays over the pooled storage manager,
// the legacy array file format, the dependency engine, a local key-value store and imperative invocation of operators
// that exist natively (plain C++ on the host, the sm_100a kernel library on a GPU).  Conventions of the reference's
// src/c_api/c_api.cc: 0 / -1 return codes, thread-local last error, thread-local return buffers.
#include <dlfcn.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "../include/mxnet_b200/c_api.h"

// ---- the rest of the runtime library (engine.cc, storage.cc, ndarray_io.cc) ------------------------------------------
extern "C" {
void* mxb_engine_create_ex(int kind, int nworkers, int nprio);
void* mxb_engine_new_var(void* e);
void mxb_engine_delete_var(void* e, void* v);
typedef int (*MxbTaskFn)(void* arg, char* err, int errlen);
void mxb_engine_push(void* e, MxbTaskFn fn, void* arg, void** reads, int nr, void** writes, int nw, int priority, const char* name);
int mxb_engine_wait_var(void* e, void* v, char* err, int errlen);
int mxb_engine_wait_all(void* e, char* err, int errlen);
void* mxb_pool_create(int dev_type, int dev_id, int strategy, uint64_t page, uint64_t large_round, int reserve, int cutoff);
void* mxb_pool_alloc(void* pool, uint64_t nbytes, int failsafe, uint64_t* rounded);
void mxb_pool_free(void* pool, void* ptr, uint64_t rounded);
void mxb_pool_release_all(void* pool);
void* mxb_ndlist_load_file(const char* path);
void mxb_ndlist_free(void* h);
const char* mxb_ndlist_error(void* h);
int64_t mxb_ndlist_count(void* h);
int64_t mxb_ndlist_num_names(void* h);
const char* mxb_ndlist_name(void* h, int64_t i, int64_t* len);
void mxb_ndlist_meta(void* h, int64_t i, int64_t* meta8);
void mxb_ndlist_shape(void* h, int64_t i, int64_t* out);
const void* mxb_ndlist_data(void* h, int64_t i, uint64_t* nbytes);
void* mxb_ndwriter_create();
void mxb_ndwriter_free(void* w);
void mxb_ndwriter_add_dense(void* wh, int np_shape, const int64_t* shape, int ndim, int dev_type, int dev_id, int type_flag,
                            const void* data, uint64_t nbytes, int is_none);
void mxb_ndwriter_add_name(void* wh, const char* name, uint64_t len);
int mxb_ndwriter_save(void* wh, const char* path);
}

namespace capi {

thread_local std::string last_error;

struct Error : std::runtime_error {
  explicit Error(const std::string& m) : std::runtime_error(m) {}
};
#define CAPI_CHECK(cond, msg) \
  do { if (!(cond)) throw capi::Error(msg); } while (0)
#define API_BEGIN() try {
#define API_END()                                                   \
  }                                                                 \
  catch (const std::exception& e) { capi::last_error = e.what(); return -1; } \
  return 0;

// ---- CUDA runtime and kernel library, looked up at run time so that the same binary serves hosts without a GPU ------------
struct Cuda {
  int (*Memcpy)(void*, const void*, size_t, int) = nullptr;
  int (*Memset)(void*, int, size_t) = nullptr;
  int (*DeviceSynchronize)() = nullptr;
  int (*GetDeviceCount)(int*) = nullptr;
  int (*MemGetInfo)(size_t*, size_t*) = nullptr;
  int (*SetDevice)(int) = nullptr;
  int (*GetDevice)(int*) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  bool ok = false;
  Cuda() {
    void* h = nullptr;
    for (const char* n : {"libcudart.so.12", "libcudart.so", "libcudart.so.13"}) { h = dlopen(n, RTLD_NOW | RTLD_GLOBAL); if (h) break; }
    if (!h) return;
#define CAPI_SYM(field, name) field = reinterpret_cast<decltype(field)>(dlsym(h, name))
    CAPI_SYM(Memcpy, "cudaMemcpy"); CAPI_SYM(Memset, "cudaMemset"); CAPI_SYM(DeviceSynchronize, "cudaDeviceSynchronize");
    CAPI_SYM(GetDeviceCount, "cudaGetDeviceCount"); CAPI_SYM(MemGetInfo, "cudaMemGetInfo"); CAPI_SYM(SetDevice, "cudaSetDevice");
    CAPI_SYM(GetDevice, "cudaGetDevice"); CAPI_SYM(GetErrorString, "cudaGetErrorString");
#undef CAPI_SYM
    ok = Memcpy && Memset && DeviceSynchronize && GetDeviceCount && MemGetInfo && SetDevice && GetDevice;
  }
  int Count() { int n = 0; if (!ok || GetDeviceCount(&n) != 0) return 0; return n; }
};
static Cuda& cuda() { static Cuda c; return c; }
static void cuda_check(int rc, const char* what) {
  if (rc != 0) throw Error(std::string(what) + ": " + (cuda().GetErrorString ? cuda().GetErrorString(rc) : "CUDA error") + " (" + std::to_string(rc) + ")");
}
struct DeviceScope {      // makes `dev` current for the calls inside the scope
  int prev = -1;
  explicit DeviceScope(int dev) { if (cuda().ok && dev >= 0) { cuda().GetDevice(&prev); if (prev != dev) cuda_check(cuda().SetDevice(dev), "cudaSetDevice"); else prev = -1; } }
  ~DeviceScope() { if (prev >= 0) cuda().SetDevice(prev); }
};

// entry points of libmxb200_kernels.so (ops/cuda/*.cu); dtype codes there: 0 fp32, 1 fp16, 2 bf16
struct Kernels {
  int (*softmax_forward)(int, const void*, void*, int64_t, int, int, void*) = nullptr;
  int (*add_n)(int, const void* const*, int, void*, int64_t, void*) = nullptr;
  int (*add_n_max)() = nullptr;
  int (*cast)(int, int, const void*, void*, int64_t, void*) = nullptr;
  int (*gelu_forward)(int, const void*, const void*, void*, int64_t, int, void*) = nullptr;
  int (*transpose)(int, const void*, void*, int, int, int, void*) = nullptr;
  int (*gemm)(int, const void*, const void*, void*, const void*, int, int, int, int, int, int, int, int, int, int*, void*) = nullptr;
  int (*ln_forward)(int, const void*, const float*, const float*, void*, float*, float*, int64_t, int, float, void*) = nullptr;
  std::string why;
  bool ok = false;
  Kernels() {
    std::string path;
    if (const char* env = std::getenv("MXNET_B200_KERNEL_LIBRARY")) path = env;
    else {
      Dl_info info;
      if (dladdr(reinterpret_cast<void*>(&cuda), &info) && info.dli_fname) {
        path = info.dli_fname;
        size_t cut = path.rfind('/');
        path = (cut == std::string::npos ? std::string(".") : path.substr(0, cut)) + "/../ops/cuda/libmxb200_kernels.so";
      }
    }
    void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!h) { why = std::string("cannot load the kernel library ") + path + ": " + dlerror(); return; }
#define CAPI_SYM(field, name) field = reinterpret_cast<decltype(field)>(dlsym(h, name))
    CAPI_SYM(softmax_forward, "mxb_softmax_forward"); CAPI_SYM(add_n, "mxb_add_n"); CAPI_SYM(add_n_max, "mxb_add_n_max");
    CAPI_SYM(cast, "mxb_cast"); CAPI_SYM(gelu_forward, "mxb_gelu_forward"); CAPI_SYM(transpose, "mxb_transpose");
    CAPI_SYM(gemm, "mxb_gemm"); CAPI_SYM(ln_forward, "mxb_ln_forward");
#undef CAPI_SYM
    ok = softmax_forward && add_n && add_n_max && cast && gelu_forward && transpose && gemm && ln_forward;
    if (!ok) why = "the kernel library lacks an expected entry point";
  }
};
static Kernels& kernels() {
  static Kernels k;
  if (!k.ok) throw Error(k.why);
  return k;
}

// ---- element types ------------------------------------------------------------------------------------------------------
static size_t elem_size(int dtype) {
  switch (dtype) {
    case kMXFloat32: case kMXInt32: return 4;
    case kMXFloat64: case kMXInt64: return 8;
    case kMXFloat16: case kMXBfloat16: return 2;
    case kMXUint8: case kMXInt8: case kMXBool: return 1;
    default: throw Error("unknown dtype " + std::to_string(dtype));
  }
}
static int kernel_dtype(int dtype) {      // code of the kernel library, or -1
  return dtype == kMXFloat32 ? 0 : dtype == kMXFloat16 ? 1 : dtype == kMXBfloat16 ? 2 : -1;
}

// ---- storage: one pool per (device type, device id) from the pooled storage manager ------------------------------------
static std::mutex pools_mu;
static std::map<std::pair<int, int>, void*> pools;
static void* pool_for(int dev_type, int dev_id) {
  std::lock_guard<std::mutex> lk(pools_mu);
  auto key = std::make_pair(dev_type, dev_id);
  auto it = pools.find(key);
  if (it != pools.end()) return it->second;
  void* p = mxb_pool_create(dev_type, dev_id, /*round*/ 1, 4096, 2u << 20, 5, 24);
  pools[key] = p;
  return p;
}

struct Chunk {      // one allocation; arrays that are views of each other share it
  void* ptr = nullptr;
  uint64_t rounded = 0;
  int dev_type = kMXCPU, dev_id = 0;
  ~Chunk() { if (ptr) mxb_pool_free(pool_for(dev_type, dev_id), ptr, rounded); }
};

static void* engine() {
  static void* e = mxb_engine_create_ex(2, 4, 2);
  return e;
}

struct Array {
  std::shared_ptr<Chunk> chunk;
  size_t offset = 0;                 // bytes into the chunk
  std::vector<int64_t> shape;
  int dtype = kMXFloat32, dev_type = kMXCPU, dev_id = 0;
  bool none = true;
  std::shared_ptr<void> var;         // engine variable, shared by views, created on first use
  std::vector<int> shape_i32;        // return buffers of the shape getters
  std::vector<uint32_t> shape_u32;

  int64_t size() const { int64_t n = 1; for (int64_t d : shape) n *= d; return n; }
  size_t nbytes() const { return static_cast<size_t>(size()) * elem_size(dtype); }
  char* data() const { return chunk ? static_cast<char*>(chunk->ptr) + offset : nullptr; }
  bool on_gpu() const { return dev_type == kMXGPU; }
  void* engine_var() {
    if (!var) {
      void* v = mxb_engine_new_var(engine());
      var = std::shared_ptr<void>(v, [](void* p) { mxb_engine_delete_var(engine(), p); });
    }
    return var.get();
  }
};

static Array* make_array(const std::vector<int64_t>& shape, int dtype, int dev_type, int dev_id) {
  CAPI_CHECK(dev_type == kMXCPU || dev_type == kMXGPU || dev_type == kMXCPUPinned, "unknown device type " + std::to_string(dev_type));
  if (dev_type != kMXCPU) {
    CAPI_CHECK(cuda().ok, "no CUDA runtime on this machine");
    if (dev_type == kMXGPU) CAPI_CHECK(dev_id >= 0 && dev_id < cuda().Count(), "no such GPU: " + std::to_string(dev_id));
  }
  for (int64_t d : shape) CAPI_CHECK(d >= 0, "negative dimension");
  auto a = std::unique_ptr<Array>(new Array());
  a->shape = shape; a->dtype = dtype; a->dev_type = dev_type; a->dev_id = dev_id; a->none = false;
  size_t bytes = std::max<size_t>(a->nbytes(), 1);
  auto c = std::make_shared<Chunk>();
  c->dev_type = dev_type; c->dev_id = dev_id;
  c->ptr = mxb_pool_alloc(pool_for(dev_type, dev_id), bytes, 0, &c->rounded);
  CAPI_CHECK(c->ptr != nullptr, "out of memory allocating " + std::to_string(bytes) + " bytes");
  a->chunk = c;
  return a.release();
}

static Array* as_array(NDArrayHandle h) {
  CAPI_CHECK(h != nullptr, "null NDArrayHandle");
  return static_cast<Array*>(h);
}

static void wait_engine(Array* a) {
  if (!a->var) return;
  char err[1024] = {0};
  if (mxb_engine_wait_var(engine(), a->var.get(), err, sizeof(err))) throw Error(err);
}
static void sync_device(const Array* a) {
  if (a->on_gpu()) { DeviceScope s(a->dev_id); cuda_check(cuda().DeviceSynchronize(), "cudaDeviceSynchronize"); }
}

// copies `bytes` between arrays on any devices (cudaMemcpyDefault = 4 resolves the direction from the pointers)
static void copy_bytes(void* dst, bool dst_gpu, const void* src, bool src_gpu, size_t bytes) {
  if (bytes == 0) return;
  if (!dst_gpu && !src_gpu) { std::memcpy(dst, src, bytes); return; }
  cuda_check(cuda().Memcpy(dst, src, bytes, 4), "cudaMemcpy");
}

}  // namespace capi

using capi::Array;
using capi::as_array;
using capi::Error;

// =====================================================================================================================
// library-wide calls
// =====================================================================================================================
const char* MXGetLastError(void) { return capi::last_error.c_str(); }

int MXGetVersion(int* out) {
  API_BEGIN();
  *out = 20000;      // the 2.0 interface
  API_END();
}

int MXGetGPUCount(int* out) {
  API_BEGIN();
  *out = capi::cuda().Count();
  API_END();
}

int MXGetGPUMemoryInformation64(int dev, uint64_t* free_mem, uint64_t* total_mem) {
  API_BEGIN();
  CAPI_CHECK(capi::cuda().ok && dev >= 0 && dev < capi::cuda().Count(), "no such GPU");
  capi::DeviceScope s(dev);
  size_t f = 0, t = 0;
  capi::cuda_check(capi::cuda().MemGetInfo(&f, &t), "cudaMemGetInfo");
  *free_mem = f;
  *total_mem = t;
  API_END();
}

static std::atomic<int> g_seed{0};
int MXRandomSeed(int seed) {
  API_BEGIN();
  g_seed = seed;
  API_END();
}

int MXNotifyShutdown(void) {
  API_BEGIN();
  char err[1024] = {0};
  mxb_engine_wait_all(capi::engine(), err, sizeof(err));
  API_END();
}

int MXStorageEmptyCache(int dev_type, int dev_id) {
  API_BEGIN();
  mxb_pool_release_all(capi::pool_for(dev_type, dev_id));
  API_END();
}

// =====================================================================================================================
// arrays
// =====================================================================================================================
int MXNDArrayCreateNone(NDArrayHandle* out) {
  API_BEGIN();
  *out = new Array();
  API_END();
}

int MXNDArrayCreateEx(const uint32_t* shape, uint32_t ndim, int dev_type, int dev_id, int delay_alloc, int dtype,
                      NDArrayHandle* out) {
  API_BEGIN();
  (void)delay_alloc;      // memory comes from a pool: allocating at once costs nothing worth delaying
  std::vector<int64_t> s(shape, shape + ndim);
  *out = capi::make_array(s, dtype, dev_type, dev_id);
  API_END();
}

int MXNDArrayCreate(const uint32_t* shape, uint32_t ndim, int dev_type, int dev_id, int delay_alloc, NDArrayHandle* out) {
  return MXNDArrayCreateEx(shape, ndim, dev_type, dev_id, delay_alloc, kMXFloat32, out);
}

int MXNDArrayFree(NDArrayHandle handle) {
  API_BEGIN();
  delete static_cast<Array*>(handle);
  API_END();
}

int MXNDArrayGetShapeEx(NDArrayHandle handle, int* out_dim, const int** out_pdata) {
  API_BEGIN();
  Array* a = as_array(handle);
  if (a->none) { *out_dim = -1; *out_pdata = nullptr; return 0; }
  a->shape_i32.assign(a->shape.begin(), a->shape.end());
  *out_dim = static_cast<int>(a->shape.size());
  *out_pdata = a->shape_i32.data();
  API_END();
}

int MXNDArrayGetShape(NDArrayHandle handle, uint32_t* out_dim, const uint32_t** out_pdata) {
  API_BEGIN();
  Array* a = as_array(handle);
  a->shape_u32.assign(a->shape.begin(), a->shape.end());
  *out_dim = static_cast<uint32_t>(a->shape.size());
  *out_pdata = a->shape_u32.data();
  API_END();
}

int MXNDArrayGetDType(NDArrayHandle handle, int* out_dtype) {
  API_BEGIN();
  Array* a = as_array(handle);
  *out_dtype = a->none ? -1 : a->dtype;
  API_END();
}

int MXNDArrayGetContext(NDArrayHandle handle, int* out_dev_type, int* out_dev_id) {
  API_BEGIN();
  Array* a = as_array(handle);
  *out_dev_type = a->none ? 0 : a->dev_type;
  *out_dev_id = a->none ? 0 : a->dev_id;
  API_END();
}

int MXNDArrayGetData(NDArrayHandle handle, void** out_pdata) {
  API_BEGIN();
  Array* a = as_array(handle);
  capi::wait_engine(a);
  *out_pdata = a->none ? nullptr : a->data();
  API_END();
}

int MXNDArraySyncCopyFromCPU(NDArrayHandle handle, const void* data, size_t size) {
  API_BEGIN();
  Array* a = as_array(handle);
  CAPI_CHECK(!a->none, "the array has no storage");
  CAPI_CHECK(static_cast<int64_t>(size) == a->size(), "size mismatch: the array holds " + std::to_string(a->size()) + " elements");
  capi::wait_engine(a);
  capi::DeviceScope s(a->on_gpu() ? a->dev_id : -1);
  capi::copy_bytes(a->data(), a->on_gpu(), data, false, a->nbytes());
  API_END();
}

int MXNDArraySyncCopyToCPU(NDArrayHandle handle, void* data, size_t size) {
  API_BEGIN();
  Array* a = as_array(handle);
  CAPI_CHECK(!a->none, "the array has no storage");
  CAPI_CHECK(static_cast<int64_t>(size) == a->size(), "size mismatch: the array holds " + std::to_string(a->size()) + " elements");
  capi::wait_engine(a);
  capi::DeviceScope s(a->on_gpu() ? a->dev_id : -1);
  capi::copy_bytes(data, false, a->data(), a->on_gpu(), a->nbytes());      // a blocking copy: ordered after the kernels
  API_END();
}

int MXNDArrayWaitToRead(NDArrayHandle handle) {
  API_BEGIN();
  Array* a = as_array(handle);
  capi::wait_engine(a);
  capi::sync_device(a);
  API_END();
}

int MXNDArrayWaitToWrite(NDArrayHandle handle) { return MXNDArrayWaitToRead(handle); }

int MXNDArrayWaitAll(void) {
  API_BEGIN();
  char err[1024] = {0};
  int failed = mxb_engine_wait_all(capi::engine(), err, sizeof(err));
  for (int d = 0; d < capi::cuda().Count(); ++d) {
    capi::DeviceScope s(d);
    capi::cuda_check(capi::cuda().DeviceSynchronize(), "cudaDeviceSynchronize");
  }
  if (failed) throw Error(err);
  API_END();
}

int MXNDArrayGetEngineVar(NDArrayHandle handle, EngineVarHandle* out) {
  API_BEGIN();
  *out = as_array(handle)->engine_var();
  API_END();
}

int MXNDArraySave(const char* fname, uint32_t num_args, NDArrayHandle* args, const char** keys) {
  API_BEGIN();
  void* w = mxb_ndwriter_create();
  std::vector<std::vector<char>> staged(num_args);      // host copies of device arrays
  try {
    for (uint32_t i = 0; i < num_args; ++i) {
      Array* a = as_array(args[i]);
      if (a->none) { mxb_ndwriter_add_dense(w, 0, nullptr, 0, kMXCPU, 0, 0, nullptr, 0, 1); continue; }
      capi::wait_engine(a);
      const void* host = a->data();
      if (a->on_gpu()) {
        staged[i].resize(a->nbytes());
        capi::DeviceScope s(a->dev_id);
        capi::copy_bytes(staged[i].data(), false, a->data(), true, a->nbytes());
        host = staged[i].data();
      }
      mxb_ndwriter_add_dense(w, 0, a->shape.data(), static_cast<int>(a->shape.size()), kMXCPU, 0, a->dtype, host, a->nbytes(), 0);
    }
    if (keys)
      for (uint32_t i = 0; i < num_args; ++i) mxb_ndwriter_add_name(w, keys[i], std::strlen(keys[i]));
    CAPI_CHECK(mxb_ndwriter_save(w, fname) == 0, std::string("cannot write ") + fname);
  } catch (...) {
    mxb_ndwriter_free(w);
    throw;
  }
  mxb_ndwriter_free(w);
  API_END();
}

int MXNDArrayLoad(const char* fname, uint32_t* out_size, NDArrayHandle** out_arr, uint32_t* out_name_size,
                  const char*** out_names) {
  thread_local std::vector<NDArrayHandle> handles;
  thread_local std::vector<std::string> names;
  thread_local std::vector<const char*> name_ptrs;
  API_BEGIN();
  void* l = mxb_ndlist_load_file(fname);
  std::vector<NDArrayHandle> loaded;
  try {
    if (const char* e = mxb_ndlist_error(l)) throw Error(e);
    const int64_t n = mxb_ndlist_count(l);
    for (int64_t i = 0; i < n; ++i) {
      int64_t meta[8];
      mxb_ndlist_meta(l, i, meta);
      if (meta[0]) { loaded.push_back(new Array()); continue; }
      CAPI_CHECK(meta[1] == 0, "sparse arrays are not available through this interface");
      std::vector<int64_t> shape(static_cast<size_t>(meta[2]));
      mxb_ndlist_shape(l, i, shape.data());
      Array* a = capi::make_array(shape, static_cast<int>(meta[5]), kMXCPU, 0);
      loaded.push_back(a);
      uint64_t nbytes = 0;
      const void* src = mxb_ndlist_data(l, i, &nbytes);
      CAPI_CHECK(nbytes == a->nbytes(), "corrupt file: payload size does not match the shape");
      std::memcpy(a->data(), src, nbytes);
    }
    names.clear();
    for (int64_t i = 0; i < mxb_ndlist_num_names(l); ++i) {
      int64_t len = 0;
      const char* p = mxb_ndlist_name(l, i, &len);
      names.emplace_back(p, static_cast<size_t>(len));
    }
  } catch (...) {
    for (NDArrayHandle h : loaded) delete static_cast<Array*>(h);
    mxb_ndlist_free(l);
    throw;
  }
  mxb_ndlist_free(l);
  handles = loaded;
  name_ptrs.clear();
  for (auto& s : names) name_ptrs.push_back(s.c_str());
  *out_size = static_cast<uint32_t>(handles.size());
  *out_arr = handles.data();
  *out_name_size = static_cast<uint32_t>(names.size());
  *out_names = name_ptrs.data();
  API_END();
}

static Array* view_of(Array* a, size_t offset_elems, const std::vector<int64_t>& shape) {
  auto v = std::unique_ptr<Array>(new Array(*a));      // shares the chunk and the engine variable
  v->offset = a->offset + offset_elems * capi::elem_size(a->dtype);
  v->shape = shape;
  return v.release();
}

int MXNDArraySlice(NDArrayHandle handle, uint32_t slice_begin, uint32_t slice_end, NDArrayHandle* out) {
  API_BEGIN();
  Array* a = as_array(handle);
  CAPI_CHECK(!a->none && !a->shape.empty(), "cannot slice a scalar or an empty handle");
  CAPI_CHECK(slice_begin <= slice_end && slice_end <= static_cast<uint64_t>(a->shape[0]), "slice out of range");
  a->engine_var();      // created before the copy so that the view shares it
  std::vector<int64_t> s = a->shape;
  const int64_t row = a->shape[0] ? a->size() / a->shape[0] : 0;
  s[0] = slice_end - slice_begin;
  *out = view_of(a, static_cast<size_t>(slice_begin) * row, s);
  API_END();
}

int MXNDArrayAt(NDArrayHandle handle, uint32_t idx, NDArrayHandle* out) {
  API_BEGIN();
  Array* a = as_array(handle);
  CAPI_CHECK(!a->none && !a->shape.empty() && idx < static_cast<uint64_t>(a->shape[0]), "index out of range");
  a->engine_var();
  const int64_t row = a->size() / a->shape[0];
  *out = view_of(a, static_cast<size_t>(idx) * row, std::vector<int64_t>(a->shape.begin() + 1, a->shape.end()));
  API_END();
}

int MXNDArrayReshape64(NDArrayHandle handle, int ndim, const int64_t* dims, int reverse, NDArrayHandle* out) {
  API_BEGIN();
  Array* a = as_array(handle);
  CAPI_CHECK(!a->none, "the array has no storage");
  (void)reverse;
  std::vector<int64_t> s(dims, dims + ndim);
  int64_t known = 1, infer = -1;
  for (int i = 0; i < ndim; ++i) {
    if (s[i] == 0 && i < static_cast<int>(a->shape.size())) s[i] = a->shape[i];      // 0 keeps the input dimension
    if (s[i] == -1) { CAPI_CHECK(infer < 0, "at most one dimension can be inferred"); infer = i; } else known *= s[i];
  }
  if (infer >= 0) { CAPI_CHECK(known > 0 && a->size() % known == 0, "cannot infer the missing dimension"); s[infer] = a->size() / known; known *= s[infer]; }
  CAPI_CHECK(known == a->size(), "reshape changes the number of elements");
  a->engine_var();
  *out = view_of(a, 0, s);
  API_END();
}

// =====================================================================================================================
// operators
// =====================================================================================================================
namespace capi {

struct Params {      // the string attributes of one invocation
  std::map<std::string, std::string> kv;
  std::string get(const std::string& k, const std::string& dflt) const { auto it = kv.find(k); return it == kv.end() ? dflt : it->second; }
  long integer(const std::string& k, long dflt) const { auto it = kv.find(k); return it == kv.end() ? dflt : std::stol(it->second); }
  double real(const std::string& k, double dflt) const { auto it = kv.find(k); return it == kv.end() ? dflt : std::stod(it->second); }
  bool flag(const std::string& k, bool dflt) const {
    auto it = kv.find(k);
    if (it == kv.end()) return dflt;
    return it->second == "1" || it->second == "True" || it->second == "true";
  }
};

struct Call {
  std::vector<Array*> in;
  std::vector<Array*> out;      // filled by `infer`, or the caller's arrays
  Params params;
};

struct OpDef {
  std::string name;
  int num_outputs = 1;
  // shapes and types of the outputs from the inputs: {shape, dtype} per output
  std::function<std::vector<std::pair<std::vector<int64_t>, int>>(const Call&)> infer;
  std::function<void(Call&)> cpu;
  std::function<void(Call&)> gpu;
};

static std::vector<OpDef>& registry() { static std::vector<OpDef> r; return r; }

static std::vector<std::pair<std::vector<int64_t>, int>> same_as_first(const Call& c) {
  return {{c.in.at(0)->shape, c.in.at(0)->dtype}};
}
static void need_inputs(const Call& c, size_t n, const char* op) {
  CAPI_CHECK(c.in.size() == n, std::string(op) + " takes " + std::to_string(n) + " inputs, got " + std::to_string(c.in.size()));
}
static void need_f32(const Call& c, const char* op) {
  for (Array* a : c.in) CAPI_CHECK(a->dtype == kMXFloat32, std::string(op) + " on the host is implemented for float32 arrays");
}
static int need_kernel_dtype(const Array* a, const char* op) {
  int k = kernel_dtype(a->dtype);
  CAPI_CHECK(k >= 0, std::string(op) + " on a GPU takes float32, float16 or bfloat16 arrays");
  return k;
}
static void kcheck(int rc, const char* what) {
  if (rc != 0) throw Error(std::string(what) + " failed with code " + std::to_string(rc));
}
template <typename T> static T* ptr(Array* a) { return reinterpret_cast<T*>(a->data()); }

// softmax / log_softmax over the last axis
static void softmax_cpu(Call& c, bool log) {
  need_f32(c, "softmax");
  Array* x = c.in[0];
  const int64_t C = x->shape.empty() ? 1 : x->shape.back(), rows = C ? x->size() / C : 0;
  const float* in = ptr<float>(x);
  float* out = ptr<float>(c.out[0]);
  for (int64_t r = 0; r < rows; ++r) {
    const float* xi = in + r * C;
    float m = xi[0], s = 0.f;
    for (int64_t j = 1; j < C; ++j) m = std::max(m, xi[j]);
    for (int64_t j = 0; j < C; ++j) s += std::exp(xi[j] - m);
    const float ls = std::log(s);
    for (int64_t j = 0; j < C; ++j) out[r * C + j] = log ? xi[j] - m - ls : std::exp(xi[j] - m) / s;
  }
}
static void softmax_gpu(Call& c, bool log) {
  Array* x = c.in[0];
  const int64_t C = x->shape.empty() ? 1 : x->shape.back(), rows = C ? x->size() / C : 0;
  kcheck(kernels().softmax_forward(need_kernel_dtype(x, "softmax"), x->data(), c.out[0]->data(), rows, static_cast<int>(C), log ? 1 : 0, nullptr),
         "softmax kernel");
}
static void check_last_axis(const Call& c, const char* op) {
  const long axis = c.params.integer("axis", -1);
  CAPI_CHECK(axis == -1 || axis == static_cast<long>(c.in[0]->shape.size()) - 1, std::string(op) + ": only the last axis is available natively");
}

static void add_cpu(Call& c) {
  need_f32(c, "elemwise_add");
  float* out = ptr<float>(c.out[0]);
  const int64_t n = c.out[0]->size();
  for (int64_t i = 0; i < n; ++i) {
    float s = 0.f;
    for (Array* a : c.in) s += ptr<float>(a)[i];
    out[i] = s;
  }
}
static void add_gpu(Call& c) {
  const int dt = need_kernel_dtype(c.in[0], "elemwise_add");
  const int64_t n = c.out[0]->size();
  const int group = kernels().add_n_max();
  // sums of more inputs than one launch takes: partial sums accumulate in the output
  std::vector<const void*> srcs;
  size_t done = 0;
  while (done < c.in.size()) {
    srcs.clear();
    if (done) srcs.push_back(c.out[0]->data());
    while (done < c.in.size() && static_cast<int>(srcs.size()) < group) srcs.push_back(c.in[done++]->data());
    kcheck(kernels().add_n(dt, srcs.data(), static_cast<int>(srcs.size()), c.out[0]->data(), n, nullptr), "add_n kernel");
  }
}
static std::vector<std::pair<std::vector<int64_t>, int>> infer_add(const Call& c) {
  CAPI_CHECK(!c.in.empty(), "a sum needs at least one input");
  for (Array* a : c.in) CAPI_CHECK(a->shape == c.in[0]->shape && a->dtype == c.in[0]->dtype, "the inputs of a sum differ in shape or type");
  return {{c.in[0]->shape, c.in[0]->dtype}};
}

// FullyConnected: data [M, K] (higher ranks flattened), weight [N, K], optional bias [N]
static std::vector<std::pair<std::vector<int64_t>, int>> infer_fc(const Call& c) {
  const bool no_bias = c.params.flag("no_bias", false);
  need_inputs(c, no_bias ? 2 : 3, "FullyConnected");
  Array *x = c.in[0], *w = c.in[1];
  CAPI_CHECK(w->shape.size() == 2 && !x->shape.empty(), "FullyConnected: weight must be 2-D");
  const int64_t M = x->shape[0], K = M ? x->size() / M : 0;
  CAPI_CHECK(K == w->shape[1], "FullyConnected: the input has " + std::to_string(K) + " features, the weight expects " + std::to_string(w->shape[1]));
  const long hidden = c.params.integer("num_hidden", w->shape[0]);
  CAPI_CHECK(hidden == w->shape[0], "FullyConnected: num_hidden does not match the weight");
  return {{{M, w->shape[0]}, x->dtype}};
}
static void fc_cpu(Call& c) {
  need_f32(c, "FullyConnected");
  Array *x = c.in[0], *w = c.in[1];
  const int64_t M = x->shape[0], N = w->shape[0], K = w->shape[1];
  const float *a = ptr<float>(x), *b = ptr<float>(w), *bias = c.in.size() > 2 ? ptr<float>(c.in[2]) : nullptr;
  float* y = ptr<float>(c.out[0]);
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) {
      double s = bias ? bias[j] : 0.0;
      for (int64_t k = 0; k < K; ++k) s += static_cast<double>(a[i * K + k]) * b[j * K + k];
      y[i * N + j] = static_cast<float>(s);
    }
}
static void fc_gpu(Call& c) {
  Array *x = c.in[0], *w = c.in[1];
  const int dt = kernel_dtype(x->dtype);
  CAPI_CHECK(dt == 1 || dt == 2, "FullyConnected on a GPU runs on the tensor-core kernel: float16 or bfloat16 arrays");
  const int64_t M = x->shape[0], N = w->shape[0], K = w->shape[1];
  CAPI_CHECK(K % 8 == 0, "FullyConnected on a GPU needs a feature count that is a multiple of 8");
  const void* bias = c.in.size() > 2 ? c.in[2]->data() : nullptr;
  kcheck(kernels().gemm(dt, x->data(), w->data(), c.out[0]->data(), bias, static_cast<int>(M), static_cast<int>(N), static_cast<int>(K),
                        static_cast<int>(K), static_cast<int>(K), static_cast<int>(N), 0, 0, 0, nullptr, nullptr),
         "tcgen05 GEMM");
}

// Cast
static std::vector<std::pair<std::vector<int64_t>, int>> infer_cast(const Call& c) {
  need_inputs(c, 1, "Cast");
  static const std::map<std::string, int> names = {{"float32", kMXFloat32}, {"float64", kMXFloat64}, {"float16", kMXFloat16},
                                                  {"bfloat16", kMXBfloat16}, {"int32", kMXInt32}, {"int64", kMXInt64},
                                                  {"uint8", kMXUint8}, {"int8", kMXInt8}};
  auto it = names.find(c.params.get("dtype", "float32"));
  CAPI_CHECK(it != names.end(), "Cast: unknown dtype " + c.params.get("dtype", ""));
  return {{c.in[0]->shape, it->second}};
}
template <typename S, typename D> static void cast_loop(const void* s, void* d, int64_t n) {
  for (int64_t i = 0; i < n; ++i) static_cast<D*>(d)[i] = static_cast<D>(static_cast<const S*>(s)[i]);
}
template <typename S> static void cast_from(const void* s, void* d, int to, int64_t n) {
  switch (to) {
    case kMXFloat32: cast_loop<S, float>(s, d, n); break;
    case kMXFloat64: cast_loop<S, double>(s, d, n); break;
    case kMXInt32: cast_loop<S, int32_t>(s, d, n); break;
    case kMXInt64: cast_loop<S, int64_t>(s, d, n); break;
    case kMXUint8: cast_loop<S, uint8_t>(s, d, n); break;
    case kMXInt8: cast_loop<S, int8_t>(s, d, n); break;
    default: throw Error("Cast on the host: half-precision targets need a GPU");
  }
}
static void cast_cpu(Call& c) {
  Array *x = c.in[0], *y = c.out[0];
  const int64_t n = x->size();
  switch (x->dtype) {
    case kMXFloat32: cast_from<float>(x->data(), y->data(), y->dtype, n); break;
    case kMXFloat64: cast_from<double>(x->data(), y->data(), y->dtype, n); break;
    case kMXInt32: cast_from<int32_t>(x->data(), y->data(), y->dtype, n); break;
    case kMXInt64: cast_from<int64_t>(x->data(), y->data(), y->dtype, n); break;
    case kMXUint8: cast_from<uint8_t>(x->data(), y->data(), y->dtype, n); break;
    case kMXInt8: cast_from<int8_t>(x->data(), y->data(), y->dtype, n); break;
    default: throw Error("Cast on the host: half-precision sources need a GPU");
  }
}
static void cast_gpu(Call& c) {
  const int s = need_kernel_dtype(c.in[0], "Cast"), d = need_kernel_dtype(c.out[0], "Cast");
  kcheck(kernels().cast(s, d, c.in[0]->data(), c.out[0]->data(), c.in[0]->size(), nullptr), "cast kernel");
}

// transpose of the last two axes (leading axes are a batch)
static std::vector<std::pair<std::vector<int64_t>, int>> infer_transpose(const Call& c) {
  need_inputs(c, 1, "transpose");
  std::vector<int64_t> s = c.in[0]->shape;
  CAPI_CHECK(s.size() >= 2, "transpose needs at least two axes");
  std::swap(s[s.size() - 1], s[s.size() - 2]);
  return {{s, c.in[0]->dtype}};
}
static void transpose_cpu(Call& c) {
  Array* x = c.in[0];
  const size_t es = elem_size(x->dtype);
  const int64_t C = x->shape.back(), R = x->shape[x->shape.size() - 2], B = x->size() / (R * C);
  const char* in = x->data();
  char* out = c.out[0]->data();
  for (int64_t b = 0; b < B; ++b)
    for (int64_t r = 0; r < R; ++r)
      for (int64_t k = 0; k < C; ++k) std::memcpy(out + ((b * C + k) * R + r) * es, in + ((b * R + r) * C + k) * es, es);
}
static void transpose_gpu(Call& c) {
  Array* x = c.in[0];
  const int64_t C = x->shape.back(), R = x->shape[x->shape.size() - 2], B = x->size() / (R * C);
  kcheck(kernels().transpose(static_cast<int>(elem_size(x->dtype)), x->data(), c.out[0]->data(), static_cast<int>(B), static_cast<int>(R),
                             static_cast<int>(C), nullptr), "transpose kernel");
}

// GELU (LeakyReLU with act_type=gelu) and ReLU
static void gelu_cpu(Call& c) {
  need_f32(c, "gelu");
  const float* x = ptr<float>(c.in[0]);
  float* y = ptr<float>(c.out[0]);
  for (int64_t i = 0; i < c.in[0]->size(); ++i) y[i] = 0.5f * x[i] * (1.f + std::erf(x[i] * 0.70710678f));
}
static void gelu_gpu(Call& c) {
  Array* x = c.in[0];
  kcheck(kernels().gelu_forward(need_kernel_dtype(x, "gelu"), x->data(), nullptr, c.out[0]->data(), x->size(), 1, nullptr), "GELU kernel");
}
static void relu_cpu(Call& c) {
  need_f32(c, "relu");
  const float* x = ptr<float>(c.in[0]);
  float* y = ptr<float>(c.out[0]);
  for (int64_t i = 0; i < c.in[0]->size(); ++i) y[i] = x[i] > 0.f ? x[i] : 0.f;
}

// LayerNorm over the last axis: data, gamma, beta (float32 parameters)
static std::vector<std::pair<std::vector<int64_t>, int>> infer_ln(const Call& c) {
  need_inputs(c, 3, "LayerNorm");
  const int64_t C = c.in[0]->shape.back();
  CAPI_CHECK(c.in[1]->size() == C && c.in[2]->size() == C, "LayerNorm: gamma and beta must have one value per channel");
  CAPI_CHECK(c.in[1]->dtype == kMXFloat32 && c.in[2]->dtype == kMXFloat32, "LayerNorm: gamma and beta are float32");
  return {{c.in[0]->shape, c.in[0]->dtype}};
}
static void ln_cpu(Call& c) {
  CAPI_CHECK(c.in[0]->dtype == kMXFloat32, "LayerNorm on the host is implemented for float32 arrays");
  const int64_t C = c.in[0]->shape.back(), rows = c.in[0]->size() / C;
  const float eps = static_cast<float>(c.params.real("eps", 1e-5));
  const float *x = ptr<float>(c.in[0]), *g = ptr<float>(c.in[1]), *b = ptr<float>(c.in[2]);
  float* y = ptr<float>(c.out[0]);
  for (int64_t r = 0; r < rows; ++r) {
    double m = 0, v = 0;
    for (int64_t j = 0; j < C; ++j) m += x[r * C + j];
    m /= C;
    for (int64_t j = 0; j < C; ++j) v += (x[r * C + j] - m) * (x[r * C + j] - m);
    const float rstd = 1.f / std::sqrt(static_cast<float>(v / C) + eps);
    for (int64_t j = 0; j < C; ++j) y[r * C + j] = (x[r * C + j] - static_cast<float>(m)) * rstd * g[j] + b[j];
  }
}
static void ln_gpu(Call& c) {
  Array* x = c.in[0];
  const int64_t C = x->shape.back(), rows = x->size() / C;
  std::unique_ptr<Array> mean(make_array({rows}, kMXFloat32, kMXGPU, x->dev_id)), rstd(make_array({rows}, kMXFloat32, kMXGPU, x->dev_id));
  kcheck(kernels().ln_forward(need_kernel_dtype(x, "LayerNorm"), x->data(), ptr<float>(c.in[1]), ptr<float>(c.in[2]), c.out[0]->data(),
                              ptr<float>(mean.get()), ptr<float>(rstd.get()), rows, static_cast<int>(C),
                              static_cast<float>(c.params.real("eps", 1e-5)), nullptr), "LayerNorm kernel");
  cuda_check(cuda().DeviceSynchronize(), "cudaDeviceSynchronize");      // the statistics buffers are released on return
}

// _copyto: the (single) output lives wherever the caller created it
static void copy_any(Call& c) {
  Array *x = c.in[0], *y = c.out[0];
  CAPI_CHECK(x->size() == y->size() && x->dtype == y->dtype, "_copyto: source and destination differ in size or type");
  DeviceScope s(y->on_gpu() ? y->dev_id : (x->on_gpu() ? x->dev_id : -1));
  copy_bytes(y->data(), y->on_gpu(), x->data(), x->on_gpu(), x->nbytes());
}

static void add_op(const char* name, decltype(OpDef::infer) infer, std::function<void(Call&)> cpu, std::function<void(Call&)> gpu) {
  OpDef d;
  d.name = name; d.infer = std::move(infer); d.cpu = std::move(cpu); d.gpu = std::move(gpu);
  registry().push_back(std::move(d));
}

static void build_registry() {
  static std::once_flag once;
  std::call_once(once, [] {
    auto unary = [](const Call& c) { need_inputs(c, 1, "this operator"); return same_as_first(c); };
    add_op("softmax", [unary](const Call& c) { check_last_axis(c, "softmax"); return unary(c); },
           [](Call& c) { softmax_cpu(c, false); }, [](Call& c) { softmax_gpu(c, false); });
    add_op("log_softmax", [unary](const Call& c) { check_last_axis(c, "log_softmax"); return unary(c); },
           [](Call& c) { softmax_cpu(c, true); }, [](Call& c) { softmax_gpu(c, true); });
    for (const char* n : {"elemwise_add", "_plus", "add_n", "ElementWiseSum"}) add_op(n, infer_add, add_cpu, add_gpu);
    add_op("FullyConnected", infer_fc, fc_cpu, fc_gpu);
    add_op("Cast", infer_cast, cast_cpu, cast_gpu);
    add_op("transpose", infer_transpose, transpose_cpu, transpose_gpu);
    add_op("relu", unary, relu_cpu, nullptr);
    add_op("LeakyReLU", [unary](const Call& c) {
             CAPI_CHECK(c.params.get("act_type", "leaky") == "gelu", "LeakyReLU: only act_type=gelu is available natively");
             return unary(c);
           }, gelu_cpu, gelu_gpu);
    add_op("LayerNorm", infer_ln, ln_cpu, ln_gpu);
    add_op("_copyto", [](const Call& c) { need_inputs(c, 1, "_copyto"); return same_as_first(c); }, copy_any, copy_any);
    add_op("_copy", [](const Call& c) { need_inputs(c, 1, "_copy"); return same_as_first(c); }, copy_any, copy_any);
  });
}

}  // namespace capi

int MXListAllOpNames(uint32_t* out_size, const char*** out_array) {
  thread_local std::vector<const char*> names;
  API_BEGIN();
  capi::build_registry();
  names.clear();
  for (auto& d : capi::registry()) names.push_back(d.name.c_str());
  *out_size = static_cast<uint32_t>(names.size());
  *out_array = names.data();
  API_END();
}

int NNGetOpHandle(const char* op_name, OpHandle* op_out) {
  API_BEGIN();
  capi::build_registry();
  for (auto& d : capi::registry())
    if (d.name == op_name) { *op_out = &d; return 0; }
  throw Error(std::string("operator ") + op_name + " is not available through the native interface");
  API_END();
}

int MXImperativeInvoke(AtomicSymbolCreator creator, int num_inputs, NDArrayHandle* inputs, int* num_outputs,
                       NDArrayHandle** outputs, int num_params, const char** param_keys, const char** param_vals) {
  thread_local std::vector<NDArrayHandle> returned;
  API_BEGIN();
  CAPI_CHECK(creator != nullptr, "null operator handle");
  auto* op = static_cast<capi::OpDef*>(creator);
  capi::Call call;
  for (int i = 0; i < num_inputs; ++i) {
    Array* a = as_array(inputs[i]);
    CAPI_CHECK(!a->none, op->name + ": input " + std::to_string(i) + " has no storage");
    capi::wait_engine(a);
    call.in.push_back(a);
  }
  for (int i = 0; i < num_params; ++i) call.params.kv[param_keys[i]] = param_vals[i];
  CAPI_CHECK(!call.in.empty(), op->name + " needs at least one input");
  const bool gpu = call.in[0]->on_gpu();
  for (Array* a : call.in)
    CAPI_CHECK((a->on_gpu() == gpu && (!gpu || a->dev_id == call.in[0]->dev_id)) || op->name == "_copyto",
               op->name + ": the inputs live on different devices");
  auto outs = op->infer(call);
  std::vector<std::unique_ptr<Array>> created;
  if (*outputs == nullptr) {
    for (auto& o : outs) {
      created.emplace_back(capi::make_array(o.first, o.second, call.in[0]->dev_type, call.in[0]->dev_id));
      call.out.push_back(created.back().get());
    }
  } else {
    CAPI_CHECK(*num_outputs == static_cast<int>(outs.size()), op->name + " has " + std::to_string(outs.size()) + " outputs");
    for (size_t i = 0; i < outs.size(); ++i) {
      Array* o = as_array((*outputs)[i]);
      if (o->none) {      // an empty handle receives the result
        std::unique_ptr<Array> fresh(capi::make_array(outs[i].first, outs[i].second, call.in[0]->dev_type, call.in[0]->dev_id));
        *o = *fresh;
      }
      CAPI_CHECK(o->size() == [&] { int64_t n = 1; for (int64_t d : outs[i].first) n *= d; return n; }() &&
                     (o->dtype == outs[i].second), op->name + ": output " + std::to_string(i) + " has the wrong size or type");
      capi::wait_engine(o);
      call.out.push_back(o);
    }
  }
  const bool run_gpu = gpu || (op->name.rfind("_copy", 0) == 0 && call.out[0]->on_gpu());
  if (run_gpu) {
    CAPI_CHECK(op->gpu != nullptr, op->name + " has no native GPU kernel");
    capi::DeviceScope s(call.out[0]->on_gpu() ? call.out[0]->dev_id : call.in[0]->dev_id);
    op->gpu(call);
  } else {
    op->cpu(call);
  }
  if (*outputs == nullptr) {
    returned.clear();
    for (auto& c : created) returned.push_back(c.release());
    *outputs = returned.data();
  }
  *num_outputs = static_cast<int>(call.out.size());
  API_END();
}

// =====================================================================================================================
// engine
// =====================================================================================================================
namespace capi {

struct PushedFn {
  EngineSyncFunc sync = nullptr;
  EngineAsyncFunc async = nullptr;
  void* param = nullptr;
  EngineFuncParamDeleter deleter = nullptr;
  // completion of an asynchronous function: the engine task returns only when the callee has signalled it
  std::mutex mu;
  std::condition_variable* cv = nullptr;
  bool done = false;
};

static int run_pushed(void* arg, char* err, int errlen) {
  std::unique_ptr<PushedFn> f(static_cast<PushedFn*>(arg));
  int rc = 0;
  try {
    if (f->sync) {
      f->sync(nullptr, f->param);
    } else {
      std::condition_variable cv;
      f->cv = &cv;
      f->async(nullptr, f.get(), f->param);
      std::unique_lock<std::mutex> lk(f->mu);
      cv.wait(lk, [&] { return f->done; });
    }
  } catch (const std::exception& e) {
    std::snprintf(err, errlen, "%s", e.what());
    rc = 1;
  }
  if (f->deleter) f->deleter(f->param);
  return rc;
}

static int push(PushedFn* f, EngineVarHandle const_vars, int nc, EngineVarHandle mutable_vars, int nm, int priority, const char* name,
                bool wait) {
  void** r = static_cast<void**>(const_vars);
  void** w = static_cast<void**>(mutable_vars);
  mxb_engine_push(engine(), run_pushed, f, r, nc, w, nm, priority, name ? name : "pushed");
  if (wait) {
    char err[1024] = {0};
    for (int i = 0; i < nm; ++i)
      if (mxb_engine_wait_var(engine(), w[i], err, sizeof(err))) throw Error(err);
  }
  return 0;
}

}  // namespace capi

int MXEnginePushSync(EngineSyncFunc sync_func, void* func_param, EngineFuncParamDeleter deleter, ContextHandle ctx_handle,
                     EngineVarHandle const_vars_handle, int num_const_vars, EngineVarHandle mutable_vars_handle,
                     int num_mutable_vars, EngineFnPropertyHandle prop_handle, int priority, const char* opr_name) {
  API_BEGIN();
  (void)ctx_handle; (void)prop_handle;
  CAPI_CHECK(sync_func != nullptr, "null function");
  auto* f = new capi::PushedFn();
  f->sync = sync_func; f->param = func_param; f->deleter = deleter;
  capi::push(f, const_vars_handle, num_const_vars, mutable_vars_handle, num_mutable_vars, priority, opr_name, false);
  API_END();
}

int MXEnginePushAsync(EngineAsyncFunc async_func, void* func_param, EngineFuncParamDeleter deleter, ContextHandle ctx_handle,
                      EngineVarHandle const_vars_handle, int num_const_vars, EngineVarHandle mutable_vars_handle,
                      int num_mutable_vars, EngineFnPropertyHandle prop_handle, int priority, const char* opr_name, int wait) {
  API_BEGIN();
  (void)ctx_handle; (void)prop_handle;
  CAPI_CHECK(async_func != nullptr, "null function");
  auto* f = new capi::PushedFn();
  f->async = async_func; f->param = func_param; f->deleter = deleter;
  capi::push(f, const_vars_handle, num_const_vars, mutable_vars_handle, num_mutable_vars, priority, opr_name, wait != 0);
  API_END();
}

int MXEngineAsyncComplete(void* on_complete) {
  API_BEGIN();
  auto* f = static_cast<capi::PushedFn*>(on_complete);
  CAPI_CHECK(f != nullptr && f->cv != nullptr, "not a completion handle of a running asynchronous function");
  {
    std::lock_guard<std::mutex> lk(f->mu);
    f->done = true;
    f->cv->notify_all();
  }
  API_END();
}

static std::atomic<int> g_bulk_size{15};
int MXEngineSetBulkSize(int bulk_size, int* prev_bulk_size) {
  API_BEGIN();
  *prev_bulk_size = g_bulk_size.exchange(bulk_size);
  API_END();
}

// =====================================================================================================================
// key-value store: one process, values of a key summed over its pushes (src/kvstore/kvstore_local.h)
// =====================================================================================================================
namespace capi {

struct KVStore {
  std::string type;
  std::mutex mu;
  std::map<std::string, std::unique_ptr<Array>> store;
};

static void sum_into(Array* dst, const std::vector<Array*>& vals) {
  // every value is brought to the store's device (a staging copy when it lives elsewhere), then summed by the
  // operator of that device
  std::vector<std::unique_ptr<Array>> staged;
  Call c;
  for (Array* v : vals) {
    CAPI_CHECK(v->size() == dst->size() && v->dtype == dst->dtype, "a pushed value differs in size or type from the stored one");
    wait_engine(v);
    if (v->dev_type == dst->dev_type && v->dev_id == dst->dev_id) { c.in.push_back(v); continue; }
    staged.emplace_back(make_array(dst->shape, dst->dtype, dst->dev_type, dst->dev_id));
    DeviceScope s(dst->on_gpu() ? dst->dev_id : (v->on_gpu() ? v->dev_id : -1));
    copy_bytes(staged.back()->data(), dst->on_gpu(), v->data(), v->on_gpu(), v->nbytes());
    c.in.push_back(staged.back().get());
  }
  c.out.push_back(dst);
  if (dst->on_gpu()) { DeviceScope s(dst->dev_id); add_gpu(c); cuda_check(cuda().DeviceSynchronize(), "cudaDeviceSynchronize"); }
  else add_cpu(c);
}

static void copy_out(Array* src, Array* dst) {
  CAPI_CHECK(src->size() == dst->size() && src->dtype == dst->dtype, "the output differs in size or type from the stored value");
  wait_engine(dst);
  DeviceScope s(dst->on_gpu() ? dst->dev_id : (src->on_gpu() ? src->dev_id : -1));
  copy_bytes(dst->data(), dst->on_gpu(), src->data(), src->on_gpu(), src->nbytes());
}

// groups the (key, value) pairs of one call by key, keeping first-seen order
static std::vector<std::pair<std::string, std::vector<Array*>>> group(uint32_t num, const char** keys, NDArrayHandle* vals) {
  std::vector<std::pair<std::string, std::vector<Array*>>> g;
  for (uint32_t i = 0; i < num; ++i) {
    auto it = std::find_if(g.begin(), g.end(), [&](auto& p) { return p.first == keys[i]; });
    if (it == g.end()) { g.emplace_back(keys[i], std::vector<Array*>()); it = g.end() - 1; }
    it->second.push_back(as_array(vals[i]));
  }
  return g;
}

}  // namespace capi

int MXKVStoreCreate(const char* type, KVStoreHandle* out) {
  API_BEGIN();
  const std::string t = type ? type : "local";
  CAPI_CHECK(t == "local" || t == "device", "the native key-value store serves one process: type 'local' or 'device'");
  auto* kv = new capi::KVStore();
  kv->type = t;
  *out = kv;
  API_END();
}

int MXKVStoreFree(KVStoreHandle handle) {
  API_BEGIN();
  delete static_cast<capi::KVStore*>(handle);
  API_END();
}

int MXKVStoreInitEx(KVStoreHandle handle, uint32_t num, const char** keys, NDArrayHandle* vals) {
  API_BEGIN();
  auto* kv = static_cast<capi::KVStore*>(handle);
  std::lock_guard<std::mutex> lk(kv->mu);
  for (uint32_t i = 0; i < num; ++i) {
    CAPI_CHECK(kv->store.find(keys[i]) == kv->store.end(), std::string("duplicate init of key ") + keys[i]);
    Array* v = as_array(vals[i]);
    std::unique_ptr<Array> s(capi::make_array(v->shape, v->dtype, v->dev_type, v->dev_id));
    capi::copy_out(v, s.get());
    kv->store[keys[i]] = std::move(s);
  }
  API_END();
}

int MXKVStorePushEx(KVStoreHandle handle, uint32_t num, const char** keys, NDArrayHandle* vals, int priority) {
  API_BEGIN();
  (void)priority;      // pushes complete before the call returns: there is nothing to order
  auto* kv = static_cast<capi::KVStore*>(handle);
  std::lock_guard<std::mutex> lk(kv->mu);
  for (auto& g : capi::group(num, keys, vals)) {
    auto it = kv->store.find(g.first);
    CAPI_CHECK(it != kv->store.end(), "key " + g.first + " has not been initialized");
    capi::sum_into(it->second.get(), g.second);      // without an updater the merged value replaces the stored one
  }
  API_END();
}

int MXKVStorePullEx(KVStoreHandle handle, uint32_t num, const char** keys, NDArrayHandle* vals, int priority) {
  API_BEGIN();
  (void)priority;
  auto* kv = static_cast<capi::KVStore*>(handle);
  std::lock_guard<std::mutex> lk(kv->mu);
  for (uint32_t i = 0; i < num; ++i) {
    auto it = kv->store.find(keys[i]);
    CAPI_CHECK(it != kv->store.end(), std::string("key ") + keys[i] + " has not been initialized");
    capi::copy_out(it->second.get(), as_array(vals[i]));
  }
  API_END();
}

int MXKVStorePushPullEx(KVStoreHandle handle, uint32_t vnum, const char** vkeys, uint32_t onum, const char** okeys,
                        NDArrayHandle* vals, NDArrayHandle* outs, int priority) {
  if (MXKVStorePushEx(handle, vnum, vkeys, vals, priority) != 0) return -1;
  return MXKVStorePullEx(handle, onum, okeys, outs, priority);
}

int MXKVStoreGetType(KVStoreHandle handle, const char** type) {
  API_BEGIN();
  *type = static_cast<capi::KVStore*>(handle)->type.c_str();
  API_END();
}
int MXKVStoreGetRank(KVStoreHandle handle, int* ret) { (void)handle; *ret = 0; return 0; }
int MXKVStoreGetGroupSize(KVStoreHandle handle, int* ret) { (void)handle; *ret = 1; return 0; }
int MXKVStoreBarrier(KVStoreHandle handle) { (void)handle; return 0; }

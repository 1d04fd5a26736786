/* Exercises the C interface (include/mxnet_b200/c_api.h) from plain C, without Python: arrays, the file format, operator
 * invocation, the engine and the key-value store.  `c_api_test cpu` runs on the host; `c_api_test gpu` runs the same
 * checks on GPU 0 with half-precision arrays on the native kernels.  Exit code 0 = every check passed. */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "mxnet_b200/c_api.h"

static int failures = 0;
#define CHECK(cond, ...)                                           \
  do {                                                             \
    if (!(cond)) {                                                 \
      ++failures;                                                  \
      fprintf(stderr, "FAILED %s:%d: ", __FILE__, __LINE__);       \
      fprintf(stderr, __VA_ARGS__);                                \
      fprintf(stderr, " (last error: %s)\n", MXGetLastError());    \
    }                                                              \
  } while (0)
#define OK(call) CHECK((call) == 0, #call)

static NDArrayHandle make(const uint32_t* shape, uint32_t ndim, int dev, int dtype, const void* host, size_t n) {
  NDArrayHandle h = NULL;
  OK(MXNDArrayCreateEx(shape, ndim, dev, 0, 0, dtype, &h));
  if (host) OK(MXNDArraySyncCopyFromCPU(h, host, n));
  return h;
}

static NDArrayHandle invoke1(const char* op, int nin, NDArrayHandle* in, int nparam, const char** keys, const char** vals) {
  OpHandle handle = NULL;
  OK(NNGetOpHandle(op, &handle));
  int nout = 0;
  NDArrayHandle* outs = NULL;
  if (MXImperativeInvoke(handle, nin, in, &nout, &outs, nparam, keys, vals) != 0) {
    CHECK(0, "invoke %s", op);
    return NULL;
  }
  CHECK(nout == 1, "%s returned %d outputs", op, nout);
  return outs[0];
}

/* float <-> half conversions for the GPU run (round to nearest even is not needed for these small integers) */
static uint16_t f2h(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u, mant = x & 0x7fffffu;
  int exp = (int)((x >> 23) & 0xff) - 127 + 15;
  if (exp <= 0) return (uint16_t)sign;
  if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
  return (uint16_t)(sign | ((uint32_t)exp << 10) | (mant >> 13));
}
static float h2f(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16, exp = (h >> 10) & 0x1f, mant = h & 0x3ffu, x;
  if (exp == 0) x = sign;
  else x = sign | ((exp - 15 + 127) << 23) | (mant << 13);
  float f;
  memcpy(&f, &x, 4);
  return f;
}

struct fill_param { float* dst; int n; float value; };
static void fill_fn(void* rctx, void* param) {
  (void)rctx;
  struct fill_param* p = (struct fill_param*)param;
  for (int i = 0; i < p->n; ++i) p->dst[i] = p->value;
}
static int deleted = 0;
static void count_delete(void* p) { (void)p; ++deleted; }

int main(int argc, char** argv) {
  const int gpu = argc > 1 && strcmp(argv[1], "gpu") == 0;
  const int dev = gpu ? kMXGPU : kMXCPU;
  int version = 0, ngpu = -1;
  OK(MXGetVersion(&version));
  OK(MXGetGPUCount(&ngpu));
  CHECK(version >= 20000 && ngpu >= 0, "version %d gpus %d", version, ngpu);
  if (gpu && ngpu < 1) { fprintf(stderr, "no GPU\n"); return 2; }

  /* ---- create, copy, shape, slice, reshape ---- */
  const uint32_t shape[2] = {4, 8};
  float host[32], back[32];
  for (int i = 0; i < 32; ++i) host[i] = (float)(i % 7) - 3.0f;
  NDArrayHandle a = make(shape, 2, dev, kMXFloat32, host, 32);
  int ndim = 0, dtype = -1, dev_type = 0, dev_id = -1;
  const int* dims = NULL;
  OK(MXNDArrayGetShapeEx(a, &ndim, &dims));
  OK(MXNDArrayGetDType(a, &dtype));
  OK(MXNDArrayGetContext(a, &dev_type, &dev_id));
  CHECK(ndim == 2 && dims[0] == 4 && dims[1] == 8 && dtype == kMXFloat32 && dev_type == dev && dev_id == 0, "metadata");
  OK(MXNDArraySyncCopyToCPU(a, back, 32));
  CHECK(memcmp(host, back, sizeof(host)) == 0, "round trip through the device");
  CHECK(MXNDArraySyncCopyToCPU(a, back, 31) != 0 && strstr(MXGetLastError(), "size mismatch") != NULL, "a wrong size must be refused");
  NDArrayHandle rows = NULL, flat = NULL;
  OK(MXNDArraySlice(a, 1, 3, &rows));
  OK(MXNDArraySyncCopyToCPU(rows, back, 16));
  CHECK(memcmp(host + 8, back, 16 * sizeof(float)) == 0, "slice views rows 1..2");
  const int64_t newshape[2] = {-1, 4};
  OK(MXNDArrayReshape64(a, 2, newshape, 0, &flat));
  OK(MXNDArrayGetShapeEx(flat, &ndim, &dims));
  CHECK(ndim == 2 && dims[0] == 8 && dims[1] == 4, "reshape with an inferred dimension");

  /* ---- save / load ---- */
  const char* fname = argc > 2 ? argv[2] : "/tmp/mxb_c_api_test.params";
  NDArrayHandle to_save[2] = {a, rows};
  const char* keys[2] = {"arg:whole", "arg:rows"};
  OK(MXNDArraySave(fname, 2, to_save, keys));
  uint32_t n_loaded = 0, n_names = 0;
  NDArrayHandle* loaded = NULL;
  const char** names = NULL;
  OK(MXNDArrayLoad(fname, &n_loaded, &loaded, &n_names, &names));
  CHECK(n_loaded == 2 && n_names == 2 && strcmp(names[1], "arg:rows") == 0, "loaded %u arrays, %u names", n_loaded, n_names);
  if (n_loaded == 2) {
    OK(MXNDArraySyncCopyToCPU(loaded[0], back, 32));
    CHECK(memcmp(host, back, sizeof(host)) == 0, "file round trip");
    OK(MXNDArrayFree(loaded[0]));
    OK(MXNDArrayFree(loaded[1]));
  }

  /* ---- operators ---- */
  uint32_t n_ops = 0;
  const char** op_names = NULL;
  OK(MXListAllOpNames(&n_ops, &op_names));
  CHECK(n_ops >= 8, "%u native operators", n_ops);
  OpHandle missing = NULL;
  CHECK(NNGetOpHandle("no_such_operator", &missing) != 0, "an unknown operator must be refused");
  {
    NDArrayHandle in1[1] = {a};
    NDArrayHandle sm = invoke1("softmax", 1, in1, 0, NULL, NULL);
    if (sm) {
      OK(MXNDArraySyncCopyToCPU(sm, back, 32));
      for (int r = 0; r < 4; ++r) {
        float s = 0.f;
        for (int j = 0; j < 8; ++j) s += back[r * 8 + j];
        CHECK(fabsf(s - 1.f) < 1e-4f, "softmax row %d sums to %f", r, s);
      }
      CHECK(back[0] < back[1], "softmax is monotone in its input");
      OK(MXNDArrayFree(sm));
    }
    NDArrayHandle in3[3] = {a, a, a};
    NDArrayHandle sum = invoke1("add_n", 3, in3, 0, NULL, NULL);
    if (sum) {
      OK(MXNDArraySyncCopyToCPU(sum, back, 32));
      int ok = 1;
      for (int i = 0; i < 32; ++i) ok &= back[i] == 3.f * host[i];
      CHECK(ok, "add_n of three copies");
      OK(MXNDArrayFree(sum));
    }
  }
  {
    /* FullyConnected: float32 on the host; float16 through the tensor-core GEMM on the GPU */
    const uint32_t xs[2] = {4, 8}, ws[2] = {16, 8}, bs[1] = {16};
    float xw[4 * 8], ww[16 * 8], bw[16], ref[4 * 16];
    for (int i = 0; i < 32; ++i) xw[i] = (float)((i * 3) % 5) - 2.f;
    for (int i = 0; i < 128; ++i) ww[i] = (float)((i * 7) % 3) - 1.f;
    for (int i = 0; i < 16; ++i) bw[i] = (float)i * 0.5f;
    for (int i = 0; i < 4; ++i)
      for (int j = 0; j < 16; ++j) {
        float s = bw[j];
        for (int k = 0; k < 8; ++k) s += xw[i * 8 + k] * ww[j * 8 + k];
        ref[i * 16 + j] = s;
      }
    NDArrayHandle x, w, b, y;
    const char* pk[1] = {"num_hidden"};
    const char* pv[1] = {"16"};
    if (!gpu) {
      x = make(xs, 2, dev, kMXFloat32, xw, 32); w = make(ws, 2, dev, kMXFloat32, ww, 128); b = make(bs, 1, dev, kMXFloat32, bw, 16);
      NDArrayHandle in[3] = {x, w, b};
      y = invoke1("FullyConnected", 3, in, 1, pk, pv);
      float out[64];
      if (y) { OK(MXNDArraySyncCopyToCPU(y, out, 64)); int ok = 1; for (int i = 0; i < 64; ++i) ok &= fabsf(out[i] - ref[i]) < 1e-4f; CHECK(ok, "FullyConnected (host)"); }
    } else {
      uint16_t xh[32], wh[128], bh[16], out[64];
      for (int i = 0; i < 32; ++i) xh[i] = f2h(xw[i]);
      for (int i = 0; i < 128; ++i) wh[i] = f2h(ww[i]);
      for (int i = 0; i < 16; ++i) bh[i] = f2h(bw[i]);
      x = make(xs, 2, dev, kMXFloat16, xh, 32); w = make(ws, 2, dev, kMXFloat16, wh, 128); b = make(bs, 1, dev, kMXFloat16, bh, 16);
      NDArrayHandle in[3] = {x, w, b};
      y = invoke1("FullyConnected", 3, in, 1, pk, pv);
      if (y) { OK(MXNDArraySyncCopyToCPU(y, out, 64)); int ok = 1; for (int i = 0; i < 64; ++i) ok &= fabsf(h2f(out[i]) - ref[i]) < 0.05f; CHECK(ok, "FullyConnected (tcgen05 GEMM)"); }
      /* Cast float32 -> float16 on the device */
      NDArrayHandle in1[1] = {a};
      const char* ck[1] = {"dtype"};
      const char* cv[1] = {"float16"};
      NDArrayHandle half = invoke1("Cast", 1, in1, 1, ck, cv);
      if (half) { uint16_t hb[32]; OK(MXNDArraySyncCopyToCPU(half, hb, 32)); int ok = 1; for (int i = 0; i < 32; ++i) ok &= h2f(hb[i]) == host[i]; CHECK(ok, "Cast to float16"); OK(MXNDArrayFree(half)); }
    }
    if (y) OK(MXNDArrayFree(y));
    OK(MXNDArrayFree(x)); OK(MXNDArrayFree(w)); OK(MXNDArrayFree(b));
  }
  {
    NDArrayHandle in1[1] = {a};
    NDArrayHandle t = invoke1("transpose", 1, in1, 0, NULL, NULL);
    if (t) {
      OK(MXNDArrayGetShapeEx(t, &ndim, &dims));
      CHECK(ndim == 2 && dims[0] == 8 && dims[1] == 4, "transpose shape");
      OK(MXNDArraySyncCopyToCPU(t, back, 32));
      int ok = 1;
      for (int r = 0; r < 4; ++r) for (int c = 0; c < 8; ++c) ok &= back[c * 4 + r] == host[r * 8 + c];
      CHECK(ok, "transpose values");
      OK(MXNDArrayFree(t));
    }
  }

  /* ---- engine: a host function that writes an array, ordered by the array's variable ---- */
  {
    const uint32_t s1[1] = {16};
    NDArrayHandle h = make(s1, 1, kMXCPU, kMXFloat32, NULL, 0);
    void* data = NULL;
    EngineVarHandle var = NULL;
    OK(MXNDArrayGetData(h, &data));
    OK(MXNDArrayGetEngineVar(h, &var));
    struct fill_param p1 = {(float*)data, 16, 1.f}, p2 = {(float*)data, 16, 2.f};
    EngineVarHandle mut[1] = {var};
    OK(MXEnginePushSync(fill_fn, &p1, count_delete, NULL, NULL, 0, mut, 1, NULL, 0, "fill1"));
    OK(MXEnginePushSync(fill_fn, &p2, count_delete, NULL, NULL, 0, mut, 1, NULL, 0, "fill2"));
    float got[16];
    OK(MXNDArraySyncCopyToCPU(h, got, 16));      /* waits for both writers */
    CHECK(got[0] == 2.f && got[15] == 2.f && deleted == 2, "engine order: got %f, %d deleters ran", got[0], deleted);
    int prev = 0;
    OK(MXEngineSetBulkSize(4, &prev));
    OK(MXNDArrayFree(h));
  }

  /* ---- key-value store ---- */
  {
    KVStoreHandle kv = NULL;
    OK(MXKVStoreCreate("local", &kv));
    const char* type = NULL;
    int rank = -1, size = 0;
    OK(MXKVStoreGetType(kv, &type));
    OK(MXKVStoreGetRank(kv, &rank));
    OK(MXKVStoreGetGroupSize(kv, &size));
    CHECK(strcmp(type, "local") == 0 && rank == 0 && size == 1, "store identity");
    const char* k1[1] = {"w"};
    NDArrayHandle v1[1] = {a};
    OK(MXKVStoreInitEx(kv, 1, k1, v1));
    const char* k2[2] = {"w", "w"};
    NDArrayHandle v2[2] = {a, a};
    NDArrayHandle out = make(shape, 2, dev, kMXFloat32, NULL, 0);
    NDArrayHandle o1[1] = {out};
    OK(MXKVStorePushPullEx(kv, 2, k2, 1, k1, v2, o1, 0));
    OK(MXNDArraySyncCopyToCPU(out, back, 32));
    int ok = 1;
    for (int i = 0; i < 32; ++i) ok &= back[i] == 2.f * host[i];
    CHECK(ok, "push of two values for one key sums them");
    const char* kbad[1] = {"missing"};
    CHECK(MXKVStorePullEx(kv, 1, kbad, o1, 0) != 0, "pulling an unknown key must fail");
    OK(MXNDArrayFree(out));
    OK(MXKVStoreFree(kv));
  }
  OK(MXNDArrayFree(rows));
  OK(MXNDArrayFree(flat));
  OK(MXNDArrayFree(a));
  OK(MXNDArrayWaitAll());
  OK(MXNotifyShutdown());
  if (failures) { fprintf(stderr, "c_api_test: %d checks failed\n", failures); return 1; }
  printf("c_api_test(%s): all checks passed\n", gpu ? "gpu" : "cpu");
  return 0;
}

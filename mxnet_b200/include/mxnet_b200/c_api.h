/*
 * C interface of the native runtime: arrays on host and device memory, their file format, the dependency engine, a
 * local key-value store and the imperative invocation of the operators that exist as native kernels.  Names, argument
 * orders and conventions follow include/mxnet/c_api.h of the reference (every function returns 0 on success and -1 on
 * failure, with the message available from MXGetLastError on the calling thread; handles are opaque pointers; returned
 * arrays of handles / strings / shapes stay valid until the next call of the same function on the same thread), so that
 * a program written against that header links against libmxb200_rt.so for the part covered here.  No Python
 * interpreter is involved: host code is C++, device code is the sm_100a kernel library (loaded on first use on a
 * machine with a GPU).
 *
 * Covered: MXGetLastError, MXGetVersion, MXGetGPUCount, MXGetGPUMemoryInformation64, MXRandomSeed, MXNotifyShutdown,
 * MXNDArrayCreateNone / Create / CreateEx / Free / GetShapeEx / GetShape / GetDType / GetContext / GetData /
 * SyncCopyFromCPU / SyncCopyToCPU / WaitToRead / WaitToWrite / WaitAll / Save / Load / Slice / At / Reshape64,
 * MXListAllOpNames, NNGetOpHandle, MXImperativeInvoke (operators listed by MXListAllOpNames),
 * MXEnginePushSync / MXEnginePushAsync / MXEngineSetBulkSize,
 * MXKVStoreCreate / Free / InitEx / PushEx / PullEx / PushPullEx / GetType / GetRank / GetGroupSize / Barrier,
 * MXStorageEmptyCache.
 */
#ifndef MXNET_B200_C_API_H_
#define MXNET_B200_C_API_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MXNET_DLL __attribute__((visibility("default")))

typedef void* NDArrayHandle;
typedef void* AtomicSymbolCreator; /* operator handle */
typedef void* OpHandle;
typedef void* KVStoreHandle;
typedef void* EngineVarHandle;
typedef void* ContextHandle;
typedef void* EngineFnPropertyHandle;

/* device types (include/mxnet/base.h Context::DeviceType) */
enum { kMXCPU = 1, kMXGPU = 2, kMXCPUPinned = 3 };
/* element types (mshadow type flags) */
enum { kMXFloat32 = 0, kMXFloat64 = 1, kMXFloat16 = 2, kMXUint8 = 3, kMXInt32 = 4, kMXInt8 = 5, kMXInt64 = 6, kMXBool = 7,
       kMXBfloat16 = 12 };

MXNET_DLL const char* MXGetLastError(void);
MXNET_DLL int MXGetVersion(int* out);
MXNET_DLL int MXGetGPUCount(int* out);
MXNET_DLL int MXGetGPUMemoryInformation64(int dev, uint64_t* free_mem, uint64_t* total_mem);
MXNET_DLL int MXRandomSeed(int seed);
MXNET_DLL int MXNotifyShutdown(void);
MXNET_DLL int MXStorageEmptyCache(int dev_type, int dev_id);

/* ---- arrays ---- */
MXNET_DLL int MXNDArrayCreateNone(NDArrayHandle* out);
MXNET_DLL int MXNDArrayCreate(const uint32_t* shape, uint32_t ndim, int dev_type, int dev_id, int delay_alloc, NDArrayHandle* out);
MXNET_DLL int MXNDArrayCreateEx(const uint32_t* shape, uint32_t ndim, int dev_type, int dev_id, int delay_alloc, int dtype,
                                NDArrayHandle* out);
MXNET_DLL int MXNDArrayFree(NDArrayHandle handle);
MXNET_DLL int MXNDArrayGetShape(NDArrayHandle handle, uint32_t* out_dim, const uint32_t** out_pdata);
MXNET_DLL int MXNDArrayGetShapeEx(NDArrayHandle handle, int* out_dim, const int** out_pdata);
MXNET_DLL int MXNDArrayGetDType(NDArrayHandle handle, int* out_dtype);
MXNET_DLL int MXNDArrayGetContext(NDArrayHandle handle, int* out_dev_type, int* out_dev_id);
MXNET_DLL int MXNDArrayGetData(NDArrayHandle handle, void** out_pdata);
MXNET_DLL int MXNDArraySyncCopyFromCPU(NDArrayHandle handle, const void* data, size_t size); /* size in elements */
MXNET_DLL int MXNDArraySyncCopyToCPU(NDArrayHandle handle, void* data, size_t size);
MXNET_DLL int MXNDArrayWaitToRead(NDArrayHandle handle);
MXNET_DLL int MXNDArrayWaitToWrite(NDArrayHandle handle);
MXNET_DLL int MXNDArrayWaitAll(void);
MXNET_DLL int MXNDArraySave(const char* fname, uint32_t num_args, NDArrayHandle* args, const char** keys);
MXNET_DLL int MXNDArrayLoad(const char* fname, uint32_t* out_size, NDArrayHandle** out_arr, uint32_t* out_name_size,
                            const char*** out_names);
MXNET_DLL int MXNDArraySlice(NDArrayHandle handle, uint32_t slice_begin, uint32_t slice_end, NDArrayHandle* out);
MXNET_DLL int MXNDArrayAt(NDArrayHandle handle, uint32_t idx, NDArrayHandle* out);
MXNET_DLL int MXNDArrayReshape64(NDArrayHandle handle, int ndim, const int64_t* dims, int reverse, NDArrayHandle* out);

/* ---- operators ---- */
MXNET_DLL int MXListAllOpNames(uint32_t* out_size, const char*** out_array);
MXNET_DLL int NNGetOpHandle(const char* op_name, OpHandle* op_out);
/* *outputs == NULL: the outputs are created and returned in an array owned by the library; otherwise the caller's
 * arrays are written. */
MXNET_DLL int MXImperativeInvoke(AtomicSymbolCreator creator, int num_inputs, NDArrayHandle* inputs, int* num_outputs,
                                 NDArrayHandle** outputs, int num_params, const char** param_keys, const char** param_vals);

/* ---- engine ---- */
typedef void (*EngineSyncFunc)(void* rctx, void* param);
typedef void (*EngineAsyncFunc)(void* rctx, void* on_complete, void* param); /* must call MXEngineAsyncComplete(on_complete) */
typedef void (*EngineFuncParamDeleter)(void* param);
MXNET_DLL int MXEnginePushSync(EngineSyncFunc sync_func, void* func_param, EngineFuncParamDeleter deleter, ContextHandle ctx_handle,
                               EngineVarHandle const_vars_handle, int num_const_vars, EngineVarHandle mutable_vars_handle,
                               int num_mutable_vars, EngineFnPropertyHandle prop_handle, int priority, const char* opr_name);
MXNET_DLL int MXEnginePushAsync(EngineAsyncFunc async_func, void* func_param, EngineFuncParamDeleter deleter,
                                ContextHandle ctx_handle, EngineVarHandle const_vars_handle, int num_const_vars,
                                EngineVarHandle mutable_vars_handle, int num_mutable_vars, EngineFnPropertyHandle prop_handle,
                                int priority, const char* opr_name, int wait);
MXNET_DLL int MXEngineAsyncComplete(void* on_complete);
MXNET_DLL int MXEngineSetBulkSize(int bulk_size, int* prev_bulk_size);
/* the engine variable of an array, for the const_vars / mutable_vars lists above (arrays of EngineVarHandle) */
MXNET_DLL int MXNDArrayGetEngineVar(NDArrayHandle handle, EngineVarHandle* out);

/* ---- key-value store (type "local" or "device": values summed over the pushes of one key) ---- */
MXNET_DLL int MXKVStoreCreate(const char* type, KVStoreHandle* out);
MXNET_DLL int MXKVStoreFree(KVStoreHandle handle);
MXNET_DLL int MXKVStoreInitEx(KVStoreHandle handle, uint32_t num, const char** keys, NDArrayHandle* vals);
MXNET_DLL int MXKVStorePushEx(KVStoreHandle handle, uint32_t num, const char** keys, NDArrayHandle* vals, int priority);
MXNET_DLL int MXKVStorePullEx(KVStoreHandle handle, uint32_t num, const char** keys, NDArrayHandle* vals, int priority);
MXNET_DLL int MXKVStorePushPullEx(KVStoreHandle handle, uint32_t vnum, const char** vkeys, uint32_t onum, const char** okeys,
                                  NDArrayHandle* vals, NDArrayHandle* outs, int priority);
MXNET_DLL int MXKVStoreGetType(KVStoreHandle handle, const char** type);
MXNET_DLL int MXKVStoreGetRank(KVStoreHandle handle, int* ret);
MXNET_DLL int MXKVStoreGetGroupSize(KVStoreHandle handle, int* ret);
MXNET_DLL int MXKVStoreBarrier(KVStoreHandle handle);

#ifdef __cplusplus
}
#endif
#endif /* MXNET_B200_C_API_H_ */

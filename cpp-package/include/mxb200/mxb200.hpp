// C++ front end over the native runtime library (libmxb200_rt.so): RAII wrappers of the dependency engine, the
// .params reader/writer and RecordIO, for host programs that do not embed Python.
// (The reference's counterpart is cpp-package/include/mxnet-cpp/*.h on top of libmxnet's C API.)
#pragma once
#include <cstdint>
#include <cstring>
#include <functional>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

extern "C" {
typedef int (*mxb_task_fn)(void* arg, char* err, int errlen);
void* mxb_engine_create(int naive, int nworkers);
void mxb_engine_destroy(void* e);
void* mxb_engine_new_var(void* e);
void mxb_engine_delete_var(void* e, void* v);
uint64_t mxb_engine_var_version(void* v);
void mxb_engine_push(void* e, mxb_task_fn fn, void* arg, void** reads, int nreads, void** writes, int nwrites, int priority,
                     const char* name);
int mxb_engine_wait_var(void* e, void* v, char* err, int errlen);
int mxb_engine_wait_all(void* e, char* err, int errlen);
int64_t mxb_engine_num_pending(void* e);
void* mxb_ndlist_load_file(const char* path);
void mxb_ndlist_free(void* l);
const char* mxb_ndlist_error(void* l);
int64_t mxb_ndlist_count(void* l);
int64_t mxb_ndlist_num_names(void* l);
const char* mxb_ndlist_name(void* l, int64_t i, int64_t* len);
void mxb_ndlist_meta(void* l, int64_t i, int64_t* out8);     // none, stype, ndim, dev type, dev id, dtype flag, n aux, storage ndim
void mxb_ndlist_shape(void* l, int64_t i, int64_t* out);
const void* mxb_ndlist_data(void* l, int64_t i, uint64_t* nbytes);
void* mxb_ndwriter_create();
void mxb_ndwriter_free(void* w);
void mxb_ndwriter_add_dense(void* w, int np_shape, const int64_t* shape, int ndim, int dev_type, int dev_id, int dtype_flag,
                            const void* data, uint64_t nbytes, int is_none);
void mxb_ndwriter_add_name(void* w, const char* name, uint64_t len);
int mxb_ndwriter_save(void* w, const char* path);
void* mxb_rec_writer_open(const char* path, int append);
int mxb_rec_writer_write(void* w, const void* data, uint64_t len);
void mxb_rec_writer_close(void* w);
void* mxb_rec_reader_open(const char* path);
const void* mxb_rec_reader_next(void* r, uint64_t* len);
void mxb_rec_reader_close(void* r);
}

namespace mxb200 {

// dtype flags of the .params format (mshadow type flags)
enum DType { kFloat32 = 0, kFloat64 = 1, kFloat16 = 2, kUint8 = 3, kInt32 = 4, kInt8 = 5, kInt64 = 6, kBool = 7, kBfloat16 = 12 };

class Engine {
 public:
  using Var = void*;
  explicit Engine(int workers = 4, bool naive = false) : h_(mxb_engine_create(naive ? 1 : 0, workers)) {}
  ~Engine() { if (h_) mxb_engine_destroy(h_); }
  Engine(const Engine&) = delete;
  Engine& operator=(const Engine&) = delete;
  Var NewVar() { return mxb_engine_new_var(h_); }
  void DeleteVar(Var v) { mxb_engine_delete_var(h_, v); }
  // Schedules fn after every earlier writer of `reads` and every earlier user of `writes`.
  void Push(std::function<void()> fn, std::vector<Var> reads, std::vector<Var> writes, int priority = 0,
            const char* name = "task") {
    auto* boxed = new std::function<void()>(std::move(fn));
    mxb_engine_push(h_, &Engine::Trampoline, boxed, reads.empty() ? nullptr : reads.data(), (int)reads.size(),
                    writes.empty() ? nullptr : writes.data(), (int)writes.size(), priority, name);
  }
  void WaitForVar(Var v) { char e[1024]; if (mxb_engine_wait_var(h_, v, e, sizeof(e))) throw std::runtime_error(e); }
  void WaitForAll() { char e[1024]; if (mxb_engine_wait_all(h_, e, sizeof(e))) throw std::runtime_error(e); }
  int64_t NumPending() const { return mxb_engine_num_pending(h_); }

 private:
  static int Trampoline(void* arg, char* err, int errlen) {
    std::unique_ptr<std::function<void()>> fn(static_cast<std::function<void()>*>(arg));
    try {
      (*fn)();
      return 0;
    } catch (const std::exception& ex) {
      if (err && errlen > 0) { std::strncpy(err, ex.what(), errlen - 1); err[errlen - 1] = 0; }
      return 1;
    }
  }
  void* h_;
};

struct Array {
  std::string name;            // empty for list files
  std::vector<int64_t> shape;
  int dtype = kFloat32;
  const void* data = nullptr;  // owned by the ParamsFile it came from
  uint64_t nbytes = 0;
};

// Reader of `.params` / `nd.save` files (all on-disk versions the Python front end reads).
class ParamsFile {
 public:
  explicit ParamsFile(const std::string& path) : h_(mxb_ndlist_load_file(path.c_str())) {
    const char* err = h_ ? mxb_ndlist_error(h_) : "cannot open file";
    if (!h_ || (err && err[0])) {
      std::string msg = err ? err : "load failed";
      if (h_) mxb_ndlist_free(h_);
      throw std::runtime_error(msg);
    }
    const int64_t n = mxb_ndlist_count(h_), nn = mxb_ndlist_num_names(h_);
    for (int64_t i = 0; i < n; ++i) {
      Array a;
      int64_t meta[8];
      mxb_ndlist_meta(h_, i, meta);
      a.shape.resize((size_t)meta[2]);
      if (meta[2] > 0) mxb_ndlist_shape(h_, i, a.shape.data());
      a.dtype = (int)meta[5];
      a.data = mxb_ndlist_data(h_, i, &a.nbytes);
      if (i < nn) {
        int64_t len = 0;
        const char* p = mxb_ndlist_name(h_, i, &len);
        a.name.assign(p, (size_t)len);
      }
      arrays_.push_back(std::move(a));
    }
  }
  ~ParamsFile() { if (h_) mxb_ndlist_free(h_); }
  ParamsFile(const ParamsFile&) = delete;
  ParamsFile& operator=(const ParamsFile&) = delete;
  const std::vector<Array>& arrays() const { return arrays_; }
  const Array* find(const std::string& name) const {
    for (const auto& a : arrays_) if (a.name == name) return &a;
    return nullptr;
  }

 private:
  void* h_;
  std::vector<Array> arrays_;
};

class ParamsWriter {
 public:
  ParamsWriter() : h_(mxb_ndwriter_create()) {}
  ~ParamsWriter() { mxb_ndwriter_free(h_); }
  void Add(const std::string& name, const std::vector<int64_t>& shape, int dtype, const void* data, uint64_t nbytes) {
    mxb_ndwriter_add_dense(h_, 0, shape.data(), (int)shape.size(), 1, 0, dtype, data, nbytes, 0);
    if (!name.empty()) mxb_ndwriter_add_name(h_, name.data(), name.size());
  }
  void Save(const std::string& path) { if (mxb_ndwriter_save(h_, path.c_str())) throw std::runtime_error("cannot write " + path); }

 private:
  void* h_;
};

class RecordWriter {
 public:
  explicit RecordWriter(const std::string& path) : h_(mxb_rec_writer_open(path.c_str(), 0)) {
    if (!h_) throw std::runtime_error("cannot open " + path);
  }
  ~RecordWriter() { if (h_) mxb_rec_writer_close(h_); }
  void Write(const std::string& rec) { mxb_rec_writer_write(h_, rec.data(), rec.size()); }

 private:
  void* h_;
};

class RecordReader {
 public:
  explicit RecordReader(const std::string& path) : h_(mxb_rec_reader_open(path.c_str())) {
    if (!h_) throw std::runtime_error("cannot open " + path);
  }
  ~RecordReader() { if (h_) mxb_rec_reader_close(h_); }
  bool Next(std::string* out) {
    uint64_t len = 0;
    const void* p = mxb_rec_reader_next(h_, &len);
    if (!p) return false;
    out->assign(static_cast<const char*>(p), (size_t)len);
    return true;
  }

 private:
  void* h_;
};

}  // namespace mxb200

// Pooled storage manager for host, pinned-host and device memory, plus POSIX shared-memory segments.
//
// Behaviour kept from the reference (src/storage/storage.cc:64-210, pooled_storage_manager.h:175-397):
// three strategies selected per device type -- "Naive" rounds a request up to a multiple of the page
// size (large requests to a multiple of the large-allocation granule) and keeps exact-size free
// lists, "Round" rounds to the next power of two below a cut-off and linearly above it, "Unpooled"
// goes straight to the driver; a configurable percentage of device memory is never pooled; when the
// driver reports out-of-memory the pool is released and the request retried once; a fail-safe
// request returns null instead of raising.  Shared segments (cpu_shared_storage_manager.h) carry a
// cross-process reference count in their first cache line so data-loader workers can hand batches
// to the trainer process without copies.
//
// The CUDA runtime is resolved at run time with dlopen so the same library serves CPU-only hosts.
#include <dlfcn.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

namespace mxb {

enum DevType { kCPU = 1, kGPU = 2, kCPUPinned = 3, kCPUShared = 5 };
enum Strategy { kNaive = 0, kRound = 1, kUnpooled = 2 };

struct CudaRT {
  int (*Malloc)(void**, size_t) = nullptr;
  int (*Free)(void*) = nullptr;
  int (*HostAlloc)(void**, size_t, unsigned) = nullptr;
  int (*FreeHost)(void*) = nullptr;
  int (*MemGetInfo)(size_t*, size_t*) = nullptr;
  int (*SetDevice)(int) = nullptr;
  int (*GetDevice)(int*) = nullptr;
  int (*GetLastError)() = nullptr;
  bool ok = false;
  CudaRT() {
    const char* names[] = {"libcudart.so.12", "libcudart.so", "libcudart.so.13"};
    void* h = nullptr;
    for (const char* n : names) { h = dlopen(n, RTLD_NOW | RTLD_GLOBAL); if (h) break; }
    if (!h) return;
    Malloc = reinterpret_cast<int (*)(void**, size_t)>(dlsym(h, "cudaMalloc"));
    Free = reinterpret_cast<int (*)(void*)>(dlsym(h, "cudaFree"));
    HostAlloc = reinterpret_cast<int (*)(void**, size_t, unsigned)>(dlsym(h, "cudaHostAlloc"));
    FreeHost = reinterpret_cast<int (*)(void*)>(dlsym(h, "cudaFreeHost"));
    MemGetInfo = reinterpret_cast<int (*)(size_t*, size_t*)>(dlsym(h, "cudaMemGetInfo"));
    SetDevice = reinterpret_cast<int (*)(int)>(dlsym(h, "cudaSetDevice"));
    GetDevice = reinterpret_cast<int (*)(int*)>(dlsym(h, "cudaGetDevice"));
    GetLastError = reinterpret_cast<int (*)()>(dlsym(h, "cudaGetLastError"));
    ok = Malloc && Free && HostAlloc && FreeHost && MemGetInfo && SetDevice && GetDevice;
  }
};

static CudaRT& RT() { static CudaRT rt; return rt; }

struct DeviceGuard {
  int prev = -1;
  bool active = false;
  explicit DeviceGuard(int dev) {
    if (RT().ok && dev >= 0) { RT().GetDevice(&prev); if (prev != dev) { RT().SetDevice(dev); active = true; } }
  }
  ~DeviceGuard() { if (active) RT().SetDevice(prev); }
};

class Pool {
 public:
  Pool(int dev_type, int dev_id, int strategy, size_t page, size_t large_round, int reserve_pct, int cutoff)
      : dev_type_(dev_type), dev_id_(dev_id), strategy_(strategy), page_(page ? page : 4096),
        large_round_(large_round ? large_round : (2u << 20)), reserve_pct_(reserve_pct), cutoff_(cutoff) {}
  ~Pool() { ReleaseAll(); }

  size_t RoundSize(size_t n) const {
    if (n == 0) n = 1;
    if (strategy_ == kUnpooled) return n;
    if (strategy_ == kRound) {
      size_t cut = size_t(1) << cutoff_;
      if (n <= cut) {
        size_t p = page_;
        while (p < n) p <<= 1;
        return p;
      }
      return (n + cut - 1) / cut * cut;
    }
    size_t g = n >= large_round_ ? large_round_ : page_;
    return (n + g - 1) / g * g;
  }

  void* Alloc(size_t nbytes, bool failsafe, size_t* rounded) {
    size_t sz = RoundSize(nbytes);
    *rounded = sz;
    std::lock_guard<std::mutex> lk(mu_);
    if (strategy_ != kUnpooled) {
      auto it = free_.find(sz);
      if (it != free_.end() && !it->second.empty()) {
        void* p = it->second.back();
        it->second.pop_back();
        pooled_bytes_ -= sz;
        used_bytes_ += sz;
        ++hits_;
        return p;
      }
    }
    if (dev_type_ == kGPU && strategy_ != kUnpooled && RT().ok && reserve_pct_ > 0) {
      DeviceGuard g(dev_id_);
      size_t fr = 0, tot = 0;
      RT().MemGetInfo(&fr, &tot);
      if (fr < sz || fr - sz < tot / 100 * reserve_pct_) ReleaseAllLocked();
    }
    void* p = RawAlloc(sz);
    if (!p) {                       // out of memory: give the cache back and retry once
      ReleaseAllLocked();
      p = RawAlloc(sz);
    }
    if (!p) {
      if (failsafe) return nullptr;
      return nullptr;
    }
    ++misses_;
    used_bytes_ += sz;
    total_bytes_ += sz;
    if (used_bytes_ > peak_bytes_) peak_bytes_ = used_bytes_;
    return p;
  }

  void Free(void* p, size_t rounded) {
    std::lock_guard<std::mutex> lk(mu_);
    used_bytes_ -= rounded;
    if (strategy_ == kUnpooled) { RawFree(p); total_bytes_ -= rounded; return; }
    free_[rounded].push_back(p);
    pooled_bytes_ += rounded;
  }

  void DirectFree(void* p, size_t rounded) {
    std::lock_guard<std::mutex> lk(mu_);
    used_bytes_ -= rounded;
    total_bytes_ -= rounded;
    RawFree(p);
  }

  void ReleaseAll() { std::lock_guard<std::mutex> lk(mu_); ReleaseAllLocked(); }

  void Stats(int64_t* out) {
    std::lock_guard<std::mutex> lk(mu_);
    out[0] = used_bytes_; out[1] = pooled_bytes_; out[2] = total_bytes_; out[3] = peak_bytes_;
    out[4] = hits_; out[5] = misses_;
  }

 private:
  void ReleaseAllLocked() {
    for (auto& kv : free_) {
      for (void* p : kv.second) { RawFree(p); total_bytes_ -= kv.first; }
      kv.second.clear();
    }
    pooled_bytes_ = 0;
  }
  void* RawAlloc(size_t sz) {
    void* p = nullptr;
    if (dev_type_ == kGPU) {
      if (!RT().ok) return nullptr;
      DeviceGuard g(dev_id_);
      if (RT().Malloc(&p, sz) != 0) { if (RT().GetLastError) RT().GetLastError(); return nullptr; }
      return p;
    }
    if (dev_type_ == kCPUPinned && RT().ok) {
      if (RT().HostAlloc(&p, sz, 0x01 /*portable*/) != 0) { if (RT().GetLastError) RT().GetLastError(); return nullptr; }
      return p;
    }
    if (posix_memalign(&p, 256, sz) != 0) return nullptr;
    return p;
  }
  void RawFree(void* p) {
    if (dev_type_ == kGPU) { if (RT().ok) { DeviceGuard g(dev_id_); RT().Free(p); } return; }
    if (dev_type_ == kCPUPinned && RT().ok) { RT().FreeHost(p); return; }
    free(p);
  }

  int dev_type_, dev_id_, strategy_;
  size_t page_, large_round_;
  int reserve_pct_, cutoff_;
  std::mutex mu_;
  std::unordered_map<size_t, std::vector<void*>> free_;
  int64_t used_bytes_ = 0, pooled_bytes_ = 0, total_bytes_ = 0, peak_bytes_ = 0, hits_ = 0, misses_ = 0;
};

// ---- shared memory segments ---------------------------------------------------------------------
struct ShmHeader { std::atomic<int> refcount; uint64_t size; char pad[48]; };

}  // namespace mxb

extern "C" {

void* mxb_pool_create(int dev_type, int dev_id, int strategy, uint64_t page, uint64_t large_round, int reserve_pct,
                      int cutoff) {
  return new mxb::Pool(dev_type, dev_id, strategy, page, large_round, reserve_pct, cutoff);
}
void mxb_pool_destroy(void* p) { delete static_cast<mxb::Pool*>(p); }
void* mxb_pool_alloc(void* p, uint64_t nbytes, int failsafe, uint64_t* rounded) {
  size_t r = 0;
  void* ptr = static_cast<mxb::Pool*>(p)->Alloc(nbytes, failsafe != 0, &r);
  *rounded = r;
  return ptr;
}
void mxb_pool_free(void* p, void* ptr, uint64_t rounded) { static_cast<mxb::Pool*>(p)->Free(ptr, rounded); }
void mxb_pool_direct_free(void* p, void* ptr, uint64_t rounded) { static_cast<mxb::Pool*>(p)->DirectFree(ptr, rounded); }
void mxb_pool_release_all(void* p) { static_cast<mxb::Pool*>(p)->ReleaseAll(); }
uint64_t mxb_pool_round(void* p, uint64_t n) { return static_cast<mxb::Pool*>(p)->RoundSize(n); }
void mxb_pool_stats(void* p, int64_t* out6) { static_cast<mxb::Pool*>(p)->Stats(out6); }
int mxb_cuda_runtime_found() { return mxb::RT().ok ? 1 : 0; }

// Creates (create=1) or attaches to a named shared segment; returns the payload address.
void* mxb_shm_open(const char* name, uint64_t size, int create, uint64_t* out_size) {
  int fd = shm_open(name, create ? (O_CREAT | O_EXCL | O_RDWR) : O_RDWR, 0600);
  if (fd < 0) return nullptr;
  uint64_t total = size + sizeof(mxb::ShmHeader);
  if (create) {
    if (ftruncate(fd, total) != 0) { close(fd); shm_unlink(name); return nullptr; }
  } else {
    struct stat st;
    if (fstat(fd, &st) != 0) { close(fd); return nullptr; }
    total = st.st_size;
  }
  void* base = mmap(nullptr, total, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (base == MAP_FAILED) return nullptr;
  auto* h = static_cast<mxb::ShmHeader*>(base);
  if (create) { new (&h->refcount) std::atomic<int>(1); h->size = size; } else { h->refcount.fetch_add(1); }
  if (out_size) *out_size = h->size;
  return static_cast<char*>(base) + sizeof(mxb::ShmHeader);
}

// Drops one reference; the last one unlinks the name.  Returns the remaining count.
int mxb_shm_close(const char* name, void* payload) {
  auto* h = reinterpret_cast<mxb::ShmHeader*>(static_cast<char*>(payload) - sizeof(mxb::ShmHeader));
  uint64_t total = h->size + sizeof(mxb::ShmHeader);
  int left = h->refcount.fetch_sub(1) - 1;
  munmap(h, total);
  if (left == 0) shm_unlink(name);
  return left;
}

// Unmaps a segment WITHOUT dropping its reference: the segment stays alive for a process that attaches later and takes
// the reference over with mxb_shm_adopt (a data-loader worker hands a finished batch to its parent this way).
int mxb_shm_detach(void* payload) {
  auto* h = reinterpret_cast<mxb::ShmHeader*>(static_cast<char*>(payload) - sizeof(mxb::ShmHeader));
  return munmap(h, h->size + sizeof(mxb::ShmHeader));
}

// Attaches to an existing segment and takes over the reference its creator left behind (no increment): the adopter's
// mxb_shm_close is then the one that unlinks the name.
void* mxb_shm_adopt(const char* name, uint64_t* out_size) {
  int fd = shm_open(name, O_RDWR, 0600);
  if (fd < 0) return nullptr;
  struct stat st;
  if (fstat(fd, &st) != 0) { close(fd); return nullptr; }
  void* base = mmap(nullptr, st.st_size, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (base == MAP_FAILED) return nullptr;
  auto* h = static_cast<mxb::ShmHeader*>(base);
  if (out_size) *out_size = h->size;
  return static_cast<char*>(base) + sizeof(mxb::ShmHeader);
}

}  // extern "C"

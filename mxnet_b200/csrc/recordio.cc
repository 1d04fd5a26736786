// RecordIO container reader/writer with a prefetching thread, and text-format parsers (CSV, LibSVM).
//
// Container format (dmlc recordio, used by tools/im2rec and ImageRecordIter in the reference,
// src/io/iter_image_recordio_2.cc): every record starts with the magic word 0xced7230a followed by
// a length word whose upper 3 bits are a continuation flag (0 whole, 1 first, 2 middle, 3 last
// part) and lower 29 bits the part length; payloads are padded to 4 bytes.  A payload that
// contains the magic word at a 4-byte aligned offset is split there (the magic itself is dropped
// and re-inserted by the reader).
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace mxb {

static const uint32_t kRecMagic = 0xced7230a;

struct RecWriter {
  FILE* f = nullptr;
};

struct RecReader {
  FILE* f = nullptr;
  std::vector<char> rec;
  // returns false at end of file
  bool Next() {
    rec.clear();
    bool started = false;
    for (;;) {
      uint32_t head[2];
      if (std::fread(head, 4, 2, f) != 2) return false;
      if (head[0] != kRecMagic) return false;
      uint32_t cflag = head[1] >> 29, len = head[1] & ((1u << 29) - 1);
      uint32_t padded = (len + 3u) & ~3u;
      size_t off = rec.size();
      if (started) {                       // re-insert the magic dropped at the split point
        rec.resize(off + 4);
        std::memcpy(rec.data() + off, &kRecMagic, 4);
        off += 4;
      }
      rec.resize(off + padded);
      if (padded && std::fread(rec.data() + off, 1, padded, f) != padded) return false;
      rec.resize(off + len);
      if (cflag == 0 || cflag == 3) return true;
      started = true;
    }
  }
};

// Sequential or index-driven prefetcher: one thread reads records ahead of the consumer.
struct Prefetcher {
  RecReader reader;
  std::vector<int64_t> offsets;       // empty: sequential
  size_t cursor = 0;
  size_t depth = 64;
  std::deque<std::vector<char>> queue;
  std::vector<char> current;
  std::mutex mu;
  std::condition_variable cv_put, cv_get;
  bool done = false, stop = false;
  std::thread th;

  void Run() {
    for (;;) {
      if (!offsets.empty()) {
        if (cursor >= offsets.size()) break;
        std::fseek(reader.f, offsets[cursor++], SEEK_SET);
      }
      if (!reader.Next()) break;
      std::unique_lock<std::mutex> lk(mu);
      cv_put.wait(lk, [this] { return stop || queue.size() < depth; });
      if (stop) return;
      queue.push_back(std::move(reader.rec));
      reader.rec = std::vector<char>();
      cv_get.notify_one();
    }
    std::lock_guard<std::mutex> lk(mu);
    done = true;
    cv_get.notify_all();
  }
  ~Prefetcher() {
    { std::lock_guard<std::mutex> lk(mu); stop = true; }
    cv_put.notify_all();
    if (th.joinable()) th.join();
    if (reader.f) std::fclose(reader.f);
  }
};

}  // namespace mxb

extern "C" {

void* mxb_rec_writer_open(const char* path, int append) {
  FILE* f = std::fopen(path, append ? "ab" : "wb");
  if (!f) return nullptr;
  auto* w = new mxb::RecWriter();
  w->f = f;
  return w;
}
int64_t mxb_rec_writer_tell(void* h) { return std::ftell(static_cast<mxb::RecWriter*>(h)->f); }
int mxb_rec_writer_write(void* h, const void* buf, uint64_t size) {
  FILE* f = static_cast<mxb::RecWriter*>(h)->f;
  if (size >= (1u << 29)) return 1;
  const char* b = static_cast<const char*>(buf);
  const uint32_t magic = mxb::kRecMagic;
  uint32_t len = static_cast<uint32_t>(size), lower = (len >> 2) << 2, upper = ((len + 3) >> 2) << 2, dptr = 0;
  for (uint32_t i = 0; i < lower; i += 4) {
    if (std::memcmp(b + i, &magic, 4) == 0) {
      uint32_t lrec = ((dptr == 0 ? 1u : 2u) << 29) | (i - dptr);
      std::fwrite(&magic, 4, 1, f);
      std::fwrite(&lrec, 4, 1, f);
      if (i != dptr) std::fwrite(b + dptr, 1, i - dptr, f);
      dptr = i + 4;
    }
  }
  uint32_t lrec = ((dptr != 0 ? 3u : 0u) << 29) | (len - dptr);
  std::fwrite(&magic, 4, 1, f);
  std::fwrite(&lrec, 4, 1, f);
  if (len != dptr) std::fwrite(b + dptr, 1, len - dptr, f);
  uint32_t zero = 0;
  if (upper != len) std::fwrite(&zero, 1, upper - len, f);
  return 0;
}
void mxb_rec_writer_close(void* h) {
  auto* w = static_cast<mxb::RecWriter*>(h);
  if (w->f) std::fclose(w->f);
  delete w;
}

void* mxb_rec_reader_open(const char* path) {
  FILE* f = std::fopen(path, "rb");
  if (!f) return nullptr;
  auto* r = new mxb::RecReader();
  r->f = f;
  return r;
}
// returns pointer to an internal buffer valid until the next call; null at end of file
const void* mxb_rec_reader_next(void* h, uint64_t* size) {
  auto* r = static_cast<mxb::RecReader*>(h);
  if (!r->Next()) { *size = 0; return nullptr; }
  *size = r->rec.size();
  return r->rec.empty() ? static_cast<const void*>("") : r->rec.data();
}
void mxb_rec_reader_seek(void* h, int64_t pos) { std::fseek(static_cast<mxb::RecReader*>(h)->f, pos, SEEK_SET); }
int64_t mxb_rec_reader_tell(void* h) { return std::ftell(static_cast<mxb::RecReader*>(h)->f); }
void mxb_rec_reader_close(void* h) {
  auto* r = static_cast<mxb::RecReader*>(h);
  if (r->f) std::fclose(r->f);
  delete r;
}

void* mxb_rec_prefetch_open(const char* path, const int64_t* offsets, int64_t n, int depth) {
  FILE* f = std::fopen(path, "rb");
  if (!f) return nullptr;
  auto* p = new mxb::Prefetcher();
  p->reader.f = f;
  if (offsets && n > 0) p->offsets.assign(offsets, offsets + n);
  p->depth = depth > 0 ? depth : 64;
  p->th = std::thread([p] { p->Run(); });
  return p;
}
const void* mxb_rec_prefetch_next(void* h, uint64_t* size) {
  auto* p = static_cast<mxb::Prefetcher*>(h);
  std::unique_lock<std::mutex> lk(p->mu);
  p->cv_get.wait(lk, [p] { return p->done || !p->queue.empty(); });
  if (p->queue.empty()) { *size = 0; return nullptr; }
  p->current = std::move(p->queue.front());
  p->queue.pop_front();
  p->cv_put.notify_one();
  *size = p->current.size();
  return p->current.empty() ? static_cast<const void*>("") : p->current.data();
}
void mxb_rec_prefetch_close(void* h) { delete static_cast<mxb::Prefetcher*>(h); }

// ---- text parsers ------------------------------------------------------------------------------
// CSV of floats: returns a malloc'd row-major float32 matrix (caller frees with mxb_free).
float* mxb_csv_load(const char* path, int64_t* rows, int64_t* cols) {
  FILE* f = std::fopen(path, "rb");
  if (!f) return nullptr;
  std::fseek(f, 0, SEEK_END);
  long n = std::ftell(f);
  std::fseek(f, 0, SEEK_SET);
  std::vector<char> buf(n + 1);
  if (n > 0 && std::fread(buf.data(), 1, n, f) != static_cast<size_t>(n)) { std::fclose(f); return nullptr; }
  std::fclose(f);
  buf[n] = 0;
  std::vector<float> vals;
  int64_t r = 0, c = 0, cur = 0;
  char* p = buf.data();
  char* end = p + n;
  while (p < end) {
    while (p < end && (*p == ' ' || *p == '\t' || *p == '\r')) ++p;
    if (p >= end) break;
    if (*p == '\n') { if (cur) { if (!c) c = cur; ++r; cur = 0; } ++p; continue; }
    char* q;
    float v = std::strtof(p, &q);
    if (q == p) { ++p; continue; }
    vals.push_back(v);
    ++cur;
    p = q;
    while (p < end && (*p == ',' || *p == ' ' || *p == '\t' || *p == '\r')) ++p;
  }
  if (cur) { if (!c) c = cur; ++r; }
  *rows = r; *cols = c;
  float* out = static_cast<float*>(std::malloc(sizeof(float) * (vals.empty() ? 1 : vals.size())));
  std::memcpy(out, vals.data(), sizeof(float) * vals.size());
  return out;
}

// LibSVM: "label idx:val idx:val ..." per line.  Outputs CSR triplet + labels, all malloc'd.
int mxb_libsvm_load(const char* path, float** labels, float** values, int64_t** indices, int64_t** indptr,
                    int64_t* rows, int64_t* nnz) {
  FILE* f = std::fopen(path, "rb");
  if (!f) return 1;
  std::vector<float> lab, val;
  std::vector<int64_t> idx, ptr(1, 0);
  char* line = nullptr;
  size_t cap = 0;
  while (getline(&line, &cap, f) > 0) {
    char* p = line;
    char* q;
    float l = std::strtof(p, &q);
    if (q == p) continue;
    lab.push_back(l);
    p = q;
    for (;;) {
      long i = std::strtol(p, &q, 10);
      if (q == p || *q != ':') break;
      p = q + 1;
      float v = std::strtof(p, &q);
      if (q == p) break;
      idx.push_back(i);
      val.push_back(v);
      p = q;
    }
    ptr.push_back(static_cast<int64_t>(idx.size()));
  }
  std::free(line);
  std::fclose(f);
  auto dup = [](const void* src, size_t bytes) { void* d = std::malloc(bytes ? bytes : 1); std::memcpy(d, src, bytes); return d; };
  *labels = static_cast<float*>(dup(lab.data(), lab.size() * 4));
  *values = static_cast<float*>(dup(val.data(), val.size() * 4));
  *indices = static_cast<int64_t*>(dup(idx.data(), idx.size() * 8));
  *indptr = static_cast<int64_t*>(dup(ptr.data(), ptr.size() * 8));
  *rows = static_cast<int64_t>(lab.size());
  *nnz = static_cast<int64_t>(idx.size());
  return 0;
}

void mxb_free(void* p) { std::free(p); }

}  // extern "C"

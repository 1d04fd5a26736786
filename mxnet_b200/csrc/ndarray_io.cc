// Reader and writer of the NDArray list container (".params" files), byte-compatible with the
// reference's format (src/ndarray/ndarray.cc:1865-2148):
//
//   file   := u64 0x112 | u64 0 | u64 n_arrays | array* | u64 n_names | (u64 len | bytes)*
//   array  := u32 magic | i32 stype | [storage_shape if sparse] | shape | (end if shape is "none")
//             | i32 dev_type | i32 dev_id | i32 type_flag | (i32 aux_type | aux_shape)* | data | aux_data*
//   shape  := i32 ndim | i64 dims[ndim]
//   magic  := 0xF993fac9 (V2, legacy shape semantics: ndim 0 = none)
//           | 0xF993faca (V3, NumPy shape semantics: ndim -1 = none, ndim 0 = scalar)
//           | 0xF993fac8 (V1: no stype field) | anything else = pre-V1 where the word is ndim and
//             dims are u32.
// Sparse arrays: row_sparse has one aux array (row indices), csr has two (indptr, column indices).
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace mxb {

static const uint64_t kListMagic = 0x112;
static const uint32_t kV1 = 0xF993fac8, kV2 = 0xF993fac9, kV3 = 0xF993faca;

static size_t TypeSize(int flag) {
  switch (flag) {
    case 0: return 4;   // float32
    case 1: return 8;   // float64
    case 2: return 2;   // float16
    case 3: return 1;   // uint8
    case 4: return 4;   // int32
    case 5: return 1;   // int8
    case 6: return 8;   // int64
    case 7: return 1;   // bool
    case 8: return 2;   // int16
    case 9: return 2;   // uint16
    case 10: return 4;  // uint32
    case 11: return 8;  // uint64
    case 12: return 2;  // bfloat16
    default: return 0;
  }
}

struct Entry {
  int32_t stype = 0;
  bool none = false;
  std::vector<int64_t> shape, storage_shape;
  int32_t dev_type = 1, dev_id = 0, type_flag = 0;
  std::vector<int32_t> aux_types;
  std::vector<std::vector<int64_t>> aux_shapes;
  size_t data_off = 0, data_bytes = 0;             // into the file buffer (reader)
  std::vector<size_t> aux_off, aux_bytes;
};

struct List {
  std::vector<char> buf;
  std::vector<Entry> entries;
  std::vector<std::string> names;
  std::string error;
};

struct Cursor {
  const char* p;
  size_t n, pos = 0;
  bool ok = true;
  bool Read(void* dst, size_t k) {
    if (!ok || pos + k > n) { ok = false; return false; }
    std::memcpy(dst, p + pos, k);
    pos += k;
    return true;
  }
  template <typename T> T Get() { T v{}; Read(&v, sizeof(T)); return v; }
};

static int64_t Prod(const std::vector<int64_t>& s) {
  int64_t r = 1;
  for (auto d : s) r *= d;
  return r;
}

static bool ReadShape(Cursor* c, std::vector<int64_t>* shape, int32_t* ndim_out) {
  int32_t ndim = c->Get<int32_t>();
  *ndim_out = ndim;
  if (!c->ok || ndim > 64) { c->ok = false; return false; }
  shape->assign(ndim > 0 ? ndim : 0, 0);
  for (int i = 0; i < ndim; ++i) (*shape)[i] = c->Get<int64_t>();
  return c->ok;
}

static bool ReadArray(Cursor* c, Entry* e) {
  uint32_t magic = c->Get<uint32_t>();
  if (!c->ok) return false;
  int32_t ndim = 0;
  if (magic == kV2 || magic == kV3) {
    e->stype = c->Get<int32_t>();
    int nad = e->stype == 1 ? 1 : (e->stype == 2 ? 2 : 0);
    if (nad > 0) { int32_t nd; if (!ReadShape(c, &e->storage_shape, &nd)) return false; }
    if (!ReadShape(c, &e->shape, &ndim)) return false;
    bool none = (magic == kV3) ? (ndim < 0) : (ndim == 0);
    if (none) { e->none = true; return true; }
    e->dev_type = c->Get<int32_t>();
    e->dev_id = c->Get<int32_t>();
    e->type_flag = c->Get<int32_t>();
    for (int i = 0; i < nad; ++i) {
      e->aux_types.push_back(c->Get<int32_t>());
      std::vector<int64_t> s; int32_t nd;
      if (!ReadShape(c, &s, &nd)) return false;
      e->aux_shapes.push_back(s);
    }
    size_t ts = TypeSize(e->type_flag);
    if (!ts) { c->ok = false; return false; }
    e->data_bytes = ts * static_cast<size_t>(Prod(nad > 0 ? e->storage_shape : e->shape));
    e->data_off = c->pos;
    if (c->pos + e->data_bytes > c->n) { c->ok = false; return false; }
    c->pos += e->data_bytes;
    for (int i = 0; i < nad; ++i) {
      size_t ab = TypeSize(e->aux_types[i]) * static_cast<size_t>(Prod(e->aux_shapes[i]));
      e->aux_off.push_back(c->pos);
      e->aux_bytes.push_back(ab);
      if (c->pos + ab > c->n) { c->ok = false; return false; }
      c->pos += ab;
    }
    return true;
  }
  // legacy layouts
  if (magic == kV1) {
    if (!ReadShape(c, &e->shape, &ndim)) return false;
  } else {
    ndim = static_cast<int32_t>(magic);
    if (ndim > 64) { c->ok = false; return false; }
    e->shape.assign(ndim, 0);
    for (int i = 0; i < ndim; ++i) e->shape[i] = c->Get<uint32_t>();
  }
  if (ndim == 0) { e->none = true; return c->ok; }
  e->dev_type = c->Get<int32_t>();
  e->dev_id = c->Get<int32_t>();
  e->type_flag = c->Get<int32_t>();
  size_t ts = TypeSize(e->type_flag);
  if (!c->ok || !ts) { c->ok = false; return false; }
  e->data_bytes = ts * static_cast<size_t>(Prod(e->shape));
  e->data_off = c->pos;
  if (c->pos + e->data_bytes > c->n) { c->ok = false; return false; }
  c->pos += e->data_bytes;
  return true;
}

static bool Parse(List* l) {
  Cursor c{l->buf.data(), l->buf.size()};
  uint64_t header = c.Get<uint64_t>();
  uint64_t reserved = c.Get<uint64_t>();
  (void)reserved;
  if (!c.ok || header != kListMagic) { l->error = "Invalid NDArray file format"; return false; }
  uint64_t n = c.Get<uint64_t>();
  if (!c.ok || n > (1ull << 32)) { l->error = "Invalid NDArray file format"; return false; }
  l->entries.resize(n);
  for (uint64_t i = 0; i < n; ++i) {
    if (!ReadArray(&c, &l->entries[i])) { l->error = "Invalid NDArray file format"; return false; }
  }
  uint64_t k = c.Get<uint64_t>();
  if (!c.ok) { l->error = "Invalid NDArray file format"; return false; }
  l->names.resize(k);
  for (uint64_t i = 0; i < k; ++i) {
    uint64_t len = c.Get<uint64_t>();
    if (!c.ok || c.pos + len > c.n) { l->error = "Invalid NDArray file format"; return false; }
    l->names[i].assign(c.p + c.pos, len);
    c.pos += len;
  }
  if (k != 0 && k != n) { l->error = "Invalid NDArray file format"; return false; }
  return true;
}

// ---- writer ----------------------------------------------------------------------------------
struct Writer {
  std::vector<char> body;
  std::vector<std::string> names;
  uint64_t count = 0;
  template <typename T> void Put(T v) { const char* p = reinterpret_cast<const char*>(&v); body.insert(body.end(), p, p + sizeof(T)); }
  void PutBytes(const void* p, size_t n) { const char* c = static_cast<const char*>(p); body.insert(body.end(), c, c + n); }
  void PutShape(const int64_t* s, int ndim) { Put<int32_t>(ndim); for (int i = 0; i < ndim; ++i) Put<int64_t>(s[i]); }
};

}  // namespace mxb

extern "C" {

// ---- reading ----
void* mxb_ndlist_load_file(const char* path) {
  auto* l = new mxb::List();
  FILE* f = std::fopen(path, "rb");
  if (!f) { l->error = std::string("cannot open ") + path; return l; }
  std::fseek(f, 0, SEEK_END);
  long n = std::ftell(f);
  std::fseek(f, 0, SEEK_SET);
  l->buf.resize(n > 0 ? n : 0);
  if (n > 0 && std::fread(l->buf.data(), 1, n, f) != static_cast<size_t>(n)) l->error = "short read";
  std::fclose(f);
  if (l->error.empty()) mxb::Parse(l);
  return l;
}
void* mxb_ndlist_load_buffer(const void* data, uint64_t n) {
  auto* l = new mxb::List();
  l->buf.assign(static_cast<const char*>(data), static_cast<const char*>(data) + n);
  mxb::Parse(l);
  return l;
}
void mxb_ndlist_free(void* h) { delete static_cast<mxb::List*>(h); }
const char* mxb_ndlist_error(void* h) { auto* l = static_cast<mxb::List*>(h); return l->error.empty() ? nullptr : l->error.c_str(); }
int64_t mxb_ndlist_count(void* h) { return static_cast<int64_t>(static_cast<mxb::List*>(h)->entries.size()); }
int64_t mxb_ndlist_num_names(void* h) { return static_cast<int64_t>(static_cast<mxb::List*>(h)->names.size()); }
const char* mxb_ndlist_name(void* h, int64_t i, int64_t* len) {
  auto& s = static_cast<mxb::List*>(h)->names[i];
  *len = static_cast<int64_t>(s.size());
  return s.data();
}
// meta: [none, stype, ndim, dev_type, dev_id, type_flag, n_aux, storage_ndim]
void mxb_ndlist_meta(void* h, int64_t i, int64_t* meta8) {
  auto& e = static_cast<mxb::List*>(h)->entries[i];
  meta8[0] = e.none; meta8[1] = e.stype; meta8[2] = static_cast<int64_t>(e.shape.size());
  meta8[3] = e.dev_type; meta8[4] = e.dev_id; meta8[5] = e.type_flag;
  meta8[6] = static_cast<int64_t>(e.aux_types.size()); meta8[7] = static_cast<int64_t>(e.storage_shape.size());
}
void mxb_ndlist_shape(void* h, int64_t i, int64_t* out) {
  auto& e = static_cast<mxb::List*>(h)->entries[i];
  for (size_t k = 0; k < e.shape.size(); ++k) out[k] = e.shape[k];
}
void mxb_ndlist_storage_shape(void* h, int64_t i, int64_t* out) {
  auto& e = static_cast<mxb::List*>(h)->entries[i];
  for (size_t k = 0; k < e.storage_shape.size(); ++k) out[k] = e.storage_shape[k];
}
const void* mxb_ndlist_data(void* h, int64_t i, uint64_t* nbytes) {
  auto* l = static_cast<mxb::List*>(h);
  auto& e = l->entries[i];
  *nbytes = e.data_bytes;
  return l->buf.data() + e.data_off;
}
// aux meta: [type_flag, ndim]; shape written to out
const void* mxb_ndlist_aux(void* h, int64_t i, int k, int64_t* meta2, int64_t* shape_out, uint64_t* nbytes) {
  auto* l = static_cast<mxb::List*>(h);
  auto& e = l->entries[i];
  meta2[0] = e.aux_types[k];
  meta2[1] = static_cast<int64_t>(e.aux_shapes[k].size());
  for (size_t d = 0; d < e.aux_shapes[k].size(); ++d) shape_out[d] = e.aux_shapes[k][d];
  *nbytes = e.aux_bytes[k];
  return l->buf.data() + e.aux_off[k];
}

// ---- writing ----
void* mxb_ndwriter_create() { return new mxb::Writer(); }
void mxb_ndwriter_free(void* w) { delete static_cast<mxb::Writer*>(w); }
// np_shape selects the V3 magic.  ndim < 0 (np) / ndim == 0 (legacy) with data == null writes a "none" array.
void mxb_ndwriter_add_dense(void* wh, int np_shape, const int64_t* shape, int ndim, int dev_type, int dev_id,
                            int type_flag, const void* data, uint64_t nbytes, int is_none) {
  auto* w = static_cast<mxb::Writer*>(wh);
  w->Put<uint32_t>(np_shape ? mxb::kV3 : mxb::kV2);
  w->Put<int32_t>(0);
  if (is_none) { w->Put<int32_t>(np_shape ? -1 : 0); ++w->count; return; }
  w->PutShape(shape, ndim);
  w->Put<int32_t>(dev_type);
  w->Put<int32_t>(dev_id);
  w->Put<int32_t>(type_flag);
  w->PutBytes(data, nbytes);
  ++w->count;
}
// sparse: stype 1 (row_sparse: aux0 = row ids) or 2 (csr: aux0 = indptr, aux1 = column ids); aux arrays are int64
void mxb_ndwriter_add_sparse(void* wh, int stype, const int64_t* shape, int ndim, const int64_t* storage_shape,
                             int storage_ndim, int dev_type, int dev_id, int type_flag, const void* data,
                             uint64_t nbytes, int n_aux, const int64_t* const* aux_data, const int64_t* aux_len) {
  auto* w = static_cast<mxb::Writer*>(wh);
  w->Put<uint32_t>(mxb::kV2);
  w->Put<int32_t>(stype);
  w->PutShape(storage_shape, storage_ndim);
  w->PutShape(shape, ndim);
  w->Put<int32_t>(dev_type);
  w->Put<int32_t>(dev_id);
  w->Put<int32_t>(type_flag);
  for (int i = 0; i < n_aux; ++i) {
    w->Put<int32_t>(6);   // int64
    w->PutShape(&aux_len[i], 1);
  }
  w->PutBytes(data, nbytes);
  for (int i = 0; i < n_aux; ++i) w->PutBytes(aux_data[i], sizeof(int64_t) * aux_len[i]);
  ++w->count;
}
void mxb_ndwriter_add_name(void* wh, const char* name, uint64_t len) { static_cast<mxb::Writer*>(wh)->names.emplace_back(name, len); }

static void Finish(mxb::Writer* w, std::vector<char>* out) {
  auto put64 = [out](uint64_t v) { const char* p = reinterpret_cast<const char*>(&v); out->insert(out->end(), p, p + 8); };
  put64(mxb::kListMagic);
  put64(0);
  put64(w->count);
  out->insert(out->end(), w->body.begin(), w->body.end());
  put64(w->names.size());
  for (auto& s : w->names) { put64(s.size()); out->insert(out->end(), s.begin(), s.end()); }
}
int mxb_ndwriter_save(void* wh, const char* path) {
  std::vector<char> out;
  Finish(static_cast<mxb::Writer*>(wh), &out);
  FILE* f = std::fopen(path, "wb");
  if (!f) return 1;
  size_t n = std::fwrite(out.data(), 1, out.size(), f);
  std::fclose(f);
  return n == out.size() ? 0 : 2;
}
uint64_t mxb_ndwriter_size(void* wh) {
  auto* w = static_cast<mxb::Writer*>(wh);
  uint64_t n = 24 + w->body.size() + 8;
  for (auto& s : w->names) n += 8 + s.size();
  return n;
}
void mxb_ndwriter_to_buffer(void* wh, void* dst) {
  std::vector<char> out;
  Finish(static_cast<mxb::Writer*>(wh), &out);
  std::memcpy(dst, out.data(), out.size());
}

}  // extern "C"

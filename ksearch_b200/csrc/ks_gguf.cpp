// GGUF container reader: the on-disk format on the load side of the decode path.
//
// Mirrors Gguf::open and its accessors (crates/ksearch_gguf/src/gguf_impl.rs:130-417): little-endian header
// (magic "GGUF", version 2 or 3, tensor count, key/value count), typed key/value metadata, tensor infos
// (name, dims, ggml type, offset), tensor data from the first multiple of general.alignment (default 32) behind
// the infos.  The file is mapped read-only; tensor bytes are handed out as pointers into the mapping
// (tensor_raw, gguf_impl.rs:277-281).  Where the reference panics (bad magic, unsupported version, unknown tensor,
// unknown ggml type) the C entry points return an error; a file that ends inside its own header is an error
// too (the reference would index past its mapping).  Host code only: no GPU is touched here.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "ks_internal.h"

namespace {

constexpr uint32_t GGUF_MAGIC = 0x46554747u;  // "GGUF"
constexpr size_t GGUF_DEFAULT_ALIGNMENT = 32;

// gguf_impl.rs:20-31 ggml_type ids and gguf_impl.rs:50-64 block_spec: (elements per block, bytes per block)
bool block_spec(uint32_t t, size_t* epb, size_t* bpb) {
  switch (t) {
    case 0: *epb = 1; *bpb = 4; return true;       // F32
    case 1: *epb = 1; *bpb = 2; return true;       // F16
    case 30: *epb = 1; *bpb = 2; return true;      // BF16
    case 2: *epb = 32; *bpb = 18; return true;     // Q4_0
    case 3: *epb = 32; *bpb = 20; return true;     // Q4_1
    case 7: *epb = 32; *bpb = 24; return true;     // Q5_1
    case 8: *epb = 32; *bpb = 34; return true;     // Q8_0
    case 12: *epb = 256; *bpb = 144; return true;  // Q4_K
    case 13: *epb = 256; *bpb = 176; return true;  // Q5_K
    case 14: *epb = 256; *bpb = 210; return true;  // Q6_K
    default: return false;
  }
}

struct Meta {  // gguf_impl.rs:66-90 MetaValue
  uint32_t type = 0;       // value type id of the file; arrays: 9
  uint32_t elem_type = 0;  // arrays: element type id
  uint64_t u = 0;          // unsigned scalars, bool
  int64_t i = 0;           // signed scalars
  double f = 0.0;          // F32 / F64
  std::string s;
  std::vector<uint32_t> au;     // ArrU32
  std::vector<int32_t> ai;      // ArrI32
  std::vector<float> af;        // ArrF32
  std::vector<uint8_t> ab;      // ArrBool
  std::vector<std::string> as;  // ArrStr
  uint64_t n = 0;               // array length (ArrOther keeps only this)
};

struct TensorInfo {  // gguf_impl.rs:92-120
  std::string name;
  uint32_t ggml_type = 0;
  std::vector<uint64_t> dims;
  uint64_t offset = 0;   // from the start of the data section
  uint64_t nbytes = 0;
};

struct Cursor {
  const uint8_t* buf;
  size_t len, pos = 0;
  bool bad = false;
  const uint8_t* read(size_t n) {
    if (bad || n > len - pos) {
      bad = true;
      return nullptr;
    }
    const uint8_t* p = buf + pos;
    pos += n;
    return p;
  }
  template <typename T>
  T get() {
    T v{};
    if (const uint8_t* p = read(sizeof(T))) memcpy(&v, p, sizeof(T));
    return v;
  }
  std::string gstr() {
    const uint64_t n = get<uint64_t>();
    if (bad || n > len - pos) {
      bad = true;
      return std::string();
    }
    const uint8_t* p = read((size_t)n);
    return std::string(reinterpret_cast<const char*>(p), (size_t)n);
  }
};

// One scalar of value type vt (gguf_impl.rs:175-192); false for a type id that is not a scalar.
bool read_scalar(Cursor& c, uint32_t vt, Meta& m) {
  switch (vt) {
    case 0: m.u = c.get<uint8_t>(); return true;
    case 1: m.i = c.get<int8_t>(); return true;
    case 2: m.u = c.get<uint16_t>(); return true;
    case 3: m.i = c.get<int16_t>(); return true;
    case 4: m.u = c.get<uint32_t>(); return true;
    case 5: m.i = c.get<int32_t>(); return true;
    case 6: m.f = c.get<float>(); return true;
    case 7: m.u = c.get<uint8_t>() != 0; return true;
    case 8: m.s = c.gstr(); return true;
    case 10: m.u = c.get<uint64_t>(); return true;
    case 11: m.i = c.get<int64_t>(); return true;
    case 12: m.f = c.get<double>(); return true;
    default: return false;
  }
}

void set_err(char* err, size_t n, const char* fmt, ...) {
  if (!err || !n) return;
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(err, n, fmt, ap);
  va_end(ap);
}

}  // namespace

struct ks_gguf {
  const uint8_t* map = nullptr;
  size_t map_len = 0;
  uint32_t version = 0;
  std::map<std::string, Meta> meta;
  std::map<std::string, TensorInfo> tensors;
  std::vector<std::string> order;  // tensor names in file order
  size_t data_offset = 0;
};

extern "C" {

void ks_gguf_close(ks_gguf* g) {
  if (!g) return;
  if (g->map) munmap(const_cast<uint8_t*>(g->map), g->map_len);
  delete g;
}

ks_gguf* ks_gguf_open(const char* path, char* err, size_t err_len) {
  if (!path) {
    set_err(err, err_len, "gguf_open: null path");
    return nullptr;
  }
  const int fd = open(path, O_RDONLY);
  if (fd < 0) {
    set_err(err, err_len, "failed to open gguf file %s", path);
    return nullptr;
  }
  struct stat st{};
  if (fstat(fd, &st) != 0 || st.st_size <= 0) {
    close(fd);
    set_err(err, err_len, "failed to mmap gguf file %s", path);
    return nullptr;
  }
  void* p = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  close(fd);
  if (p == MAP_FAILED) {
    set_err(err, err_len, "failed to mmap gguf file %s", path);
    return nullptr;
  }
  ks_gguf* g = new ks_gguf();
  g->map = static_cast<const uint8_t*>(p);
  g->map_len = (size_t)st.st_size;
  Cursor c{g->map, g->map_len};
  const uint32_t magic = c.get<uint32_t>();
  if (c.bad || magic != GGUF_MAGIC) {
    set_err(err, err_len, "not a GGUF file (bad magic)");
    ks_gguf_close(g);
    return nullptr;
  }
  g->version = c.get<uint32_t>();
  if (c.bad || (g->version != 2 && g->version != 3)) {
    set_err(err, err_len, "unsupported GGUF version %u", g->version);
    ks_gguf_close(g);
    return nullptr;
  }
  const uint64_t tensor_count = c.get<uint64_t>(), kv_count = c.get<uint64_t>();
  // every key/value and every tensor info takes at least a dozen bytes: counts beyond the file size are corrupt
  if (c.bad || tensor_count > g->map_len || kv_count > g->map_len) {
    set_err(err, err_len, "truncated GGUF file");
    ks_gguf_close(g);
    return nullptr;
  }
  for (uint64_t k = 0; k < kv_count && !c.bad; k++) {
    const std::string key = c.gstr();
    Meta m;
    m.type = c.get<uint32_t>();
    if (m.type != 9) {
      if (!read_scalar(c, m.type, m)) {
        set_err(err, err_len, "unexpected scalar value type %u", m.type);
        ks_gguf_close(g);
        return nullptr;
      }
    } else {  // ARRAY (gguf_impl.rs:197-215): u32 / i32 / f32 / bool / string arrays are kept, others only counted
      m.elem_type = c.get<uint32_t>();
      m.n = c.get<uint64_t>();
      if (c.bad || m.n > g->map_len) {
        c.bad = true;
        break;
      }
      for (uint64_t e = 0; e < m.n && !c.bad; e++) {
        Meta v;
        if (!read_scalar(c, m.elem_type, v)) {
          set_err(err, err_len, "unexpected scalar value type %u", m.elem_type);
          ks_gguf_close(g);
          return nullptr;
        }
        switch (m.elem_type) {
          case 4: m.au.push_back((uint32_t)v.u); break;
          case 5: m.ai.push_back((int32_t)v.i); break;
          case 6: m.af.push_back((float)v.f); break;
          case 7: m.ab.push_back((uint8_t)v.u); break;
          case 8: m.as.push_back(v.s); break;
          default: break;
        }
      }
    }
    g->meta[key] = std::move(m);
  }
  for (uint64_t t = 0; t < tensor_count && !c.bad; t++) {
    TensorInfo ti;
    ti.name = c.gstr();
    const uint32_t n_dims = c.get<uint32_t>();
    if (c.bad || n_dims > 8) {
      c.bad = true;
      break;
    }
    for (uint32_t d = 0; d < n_dims; d++) ti.dims.push_back(c.get<uint64_t>());
    ti.ggml_type = c.get<uint32_t>();
    ti.offset = c.get<uint64_t>();
    g->order.push_back(ti.name);
    g->tensors[ti.name] = std::move(ti);
  }
  if (c.bad) {
    set_err(err, err_len, "truncated GGUF file");
    ks_gguf_close(g);
    return nullptr;
  }
  size_t alignment = GGUF_DEFAULT_ALIGNMENT;  // gguf_impl.rs:246-250: general.alignment as U32 or U64
  auto al = g->meta.find("general.alignment");
  if (al != g->meta.end() && (al->second.type == 4 || al->second.type == 10) && al->second.u > 0) alignment = (size_t)al->second.u;
  g->data_offset = (c.pos + alignment - 1) / alignment * alignment;
  // byte lengths (gguf_impl.rs:114-119) and bounds, so that tensor_raw can never point outside the mapping
  for (auto& kv : g->tensors) {
    TensorInfo& ti = kv.second;
    size_t epb = 0, bpb = 0;
    uint64_t n = 1;
    for (uint64_t d : ti.dims) n *= d;
    if (!block_spec(ti.ggml_type, &epb, &bpb)) {
      ti.nbytes = 0;  // unknown type: listed, but its bytes cannot be handed out
      continue;
    }
    if (n % epb) {
      set_err(err, err_len, "tensor %s elems %llu not divisible by block %zu", ti.name.c_str(), (unsigned long long)n, epb);
      ks_gguf_close(g);
      return nullptr;
    }
    ti.nbytes = n / epb * bpb;
    if (g->data_offset > g->map_len || ti.offset > g->map_len - g->data_offset || ti.nbytes > g->map_len - g->data_offset - ti.offset) {
      set_err(err, err_len, "tensor %s lies outside the file", ti.name.c_str());
      ks_gguf_close(g);
      return nullptr;
    }
  }
  return g;
}

int ks_gguf_version(const ks_gguf* g) { return g ? (int)g->version : 0; }
size_t ks_gguf_n_tensors(const ks_gguf* g) { return g ? g->tensors.size() : 0; }
size_t ks_gguf_n_kv(const ks_gguf* g) { return g ? g->meta.size() : 0; }
uint64_t ks_gguf_data_offset(const ks_gguf* g) { return g ? g->data_offset : 0; }
const char* ks_gguf_tensor_name(const ks_gguf* g, size_t i) { return g && i < g->order.size() ? g->order[i].c_str() : nullptr; }

// Type, dims (up to 4 returned, n_dims says how many there are), absolute file offset (tensor_file_offset,
// gguf_impl.rs:309-314) and byte length of a tensor.  KS_ERR_INVALID: "tensor not found".
int ks_gguf_tensor(const ks_gguf* g, const char* name, uint32_t* ggml_type, uint32_t* n_dims, uint64_t* dims4, uint64_t* file_offset,
                   uint64_t* nbytes) {
  if (!g || !name) return KS_ERR_INVALID;
  auto it = g->tensors.find(name);
  if (it == g->tensors.end()) return KS_ERR_INVALID;
  const TensorInfo& ti = it->second;
  if (ggml_type) *ggml_type = ti.ggml_type;
  if (n_dims) *n_dims = (uint32_t)ti.dims.size();
  if (dims4)
    for (size_t d = 0; d < 4; d++) dims4[d] = d < ti.dims.size() ? ti.dims[d] : 1;
  if (file_offset) *file_offset = g->data_offset + ti.offset;
  if (nbytes) *nbytes = ti.nbytes;
  return KS_OK;
}

// tensor_raw (gguf_impl.rs:277-281): the tensor's bytes inside the mapping; NULL for an unknown tensor or ggml type.
const void* ks_gguf_tensor_raw(const ks_gguf* g, const char* name) {
  if (!g || !name) return nullptr;
  auto it = g->tensors.find(name);
  if (it == g->tensors.end() || !it->second.nbytes) return nullptr;
  return g->map + g->data_offset + it->second.offset;
}

// ---- metadata accessors, with the reference's coercions (gguf_impl.rs:330-417); 1 = found, 0 = absent or another type
int ks_gguf_has_key(const ks_gguf* g, const char* key) { return g && key && g->meta.count(key) ? 1 : 0; }
int ks_gguf_get_u32(const ks_gguf* g, const char* key, uint32_t* out) {
  if (!g || !key || !out) return 0;
  auto it = g->meta.find(key);
  if (it == g->meta.end()) return 0;
  const Meta& m = it->second;
  if (m.type == 4 || m.type == 10 || m.type == 2) *out = (uint32_t)m.u;
  else if (m.type == 5) *out = (uint32_t)m.i;
  else return 0;
  return 1;
}
int ks_gguf_get_u64(const ks_gguf* g, const char* key, uint64_t* out) {
  if (!g || !key || !out) return 0;
  auto it = g->meta.find(key);
  if (it == g->meta.end()) return 0;
  const Meta& m = it->second;
  if (m.type == 10 || m.type == 4) *out = m.u;
  else if (m.type == 5) *out = (uint64_t)m.i;
  else return 0;
  return 1;
}
int ks_gguf_get_f32(const ks_gguf* g, const char* key, float* out) {
  if (!g || !key || !out) return 0;
  auto it = g->meta.find(key);
  if (it == g->meta.end() || (it->second.type != 6 && it->second.type != 12)) return 0;
  *out = (float)it->second.f;
  return 1;
}
int ks_gguf_get_bool(const ks_gguf* g, const char* key, int* out) {
  if (!g || !key || !out) return 0;
  auto it = g->meta.find(key);
  if (it == g->meta.end() || it->second.type != 7) return 0;
  *out = it->second.u != 0;
  return 1;
}
const char* ks_gguf_get_str(const ks_gguf* g, const char* key) {
  if (!g || !key) return nullptr;
  auto it = g->meta.find(key);
  return it == g->meta.end() || it->second.type != 8 ? nullptr : it->second.s.c_str();
}
// Arrays: length and element type id (-1 when the key is absent or not an array), then typed copies of up to `max`
// elements that return the element count, or -1 when the array has another element type.
long long ks_gguf_arr_len(const ks_gguf* g, const char* key, uint32_t* elem_type) {
  if (!g || !key) return -1;
  auto it = g->meta.find(key);
  if (it == g->meta.end() || it->second.type != 9) return -1;
  if (elem_type) *elem_type = it->second.elem_type;
  return (long long)it->second.n;
}
long long ks_gguf_get_arr_u32(const ks_gguf* g, const char* key, uint32_t* out, size_t max) {
  if (!g || !key) return -1;
  auto it = g->meta.find(key);
  if (it == g->meta.end() || it->second.type != 9 || it->second.elem_type != 4) return -1;
  for (size_t i = 0; i < it->second.au.size() && i < max && out; i++) out[i] = it->second.au[i];
  return (long long)it->second.au.size();
}
long long ks_gguf_get_arr_i32(const ks_gguf* g, const char* key, int32_t* out, size_t max) {
  if (!g || !key) return -1;
  auto it = g->meta.find(key);
  if (it == g->meta.end() || it->second.type != 9 || it->second.elem_type != 5) return -1;
  for (size_t i = 0; i < it->second.ai.size() && i < max && out; i++) out[i] = it->second.ai[i];
  return (long long)it->second.ai.size();
}
long long ks_gguf_get_arr_f32(const ks_gguf* g, const char* key, float* out, size_t max) {
  if (!g || !key) return -1;
  auto it = g->meta.find(key);
  if (it == g->meta.end() || it->second.type != 9 || it->second.elem_type != 6) return -1;
  for (size_t i = 0; i < it->second.af.size() && i < max && out; i++) out[i] = it->second.af[i];
  return (long long)it->second.af.size();
}
long long ks_gguf_get_arr_bool(const ks_gguf* g, const char* key, uint8_t* out, size_t max) {
  if (!g || !key) return -1;
  auto it = g->meta.find(key);
  if (it == g->meta.end() || it->second.type != 9 || it->second.elem_type != 7) return -1;
  for (size_t i = 0; i < it->second.ab.size() && i < max && out; i++) out[i] = it->second.ab[i];
  return (long long)it->second.ab.size();
}
const char* ks_gguf_get_arr_str(const ks_gguf* g, const char* key, size_t i) {
  if (!g || !key) return nullptr;
  auto it = g->meta.find(key);
  if (it == g->meta.end() || it->second.type != 9 || it->second.elem_type != 8 || i >= it->second.as.size()) return nullptr;
  return it->second.as[i].c_str();
}

}  // extern "C"

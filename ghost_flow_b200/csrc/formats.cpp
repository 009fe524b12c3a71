// Checkpoint formats of GhostFlow, read and written bit-exactly, behind a small C ABI.
//
//  GHOSTFLW state dict (ghostflow-core/src/serialize.rs:11-200):
//    "GHOSTFLW" | u32 version = 1 | u32 n | per tensor: u32 name_len, name, u8 dtype code, u32 ndim,
//    ndim x u64 dims, numel x f32 payload (always f32, whatever the dtype code says).
//  GFCP checkpoint (ghostflow-nn/src/serialization.rs:75-284):
//    "GFCP" | bytes 0,4,0 | 3 strings (model name, version, framework version) | u64 epoch | f32 loss |
//    u32 n_extra | n x (key, value) strings | u32 n_params | per param: name, u32 ndim, ndim x u64,
//    u64 data_len, data_len x f32 | u8 has_optimizer | if 1: u32 n, per entry: name, u64 len, len x f32.
//  SafeTensors (serialize.rs:223-456): u64 header length, JSON header, raw little-endian data; the writer
//    emits F32 only and no __metadata__, the reader accepts F32 (and converts F16/BF16/F64/I64/I32 to f32).
//
// All integers little-endian. A loaded file is an in-memory handle queried through accessors.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#define GFIO_API extern "C" __attribute__((visibility("default")))

namespace {

struct Entry {
  std::string name;
  uint8_t dtype = 2;
  std::vector<uint64_t> dims;
  std::vector<float> data;
};

struct File {
  int kind = 0;  // 1 GHOSTFLW, 2 GFCP, 3 safetensors
  std::vector<Entry> tensors;
  std::vector<Entry> optimizer;  // GFCP optimizer entries (1-D)
  std::string meta[3];
  uint64_t epoch = 0;
  float loss = 0.f;
  std::vector<std::pair<std::string, std::string>> extra;
  std::string error;
};

thread_local std::string g_error;

struct Reader {
  FILE* f;
  bool ok = true;
  explicit Reader(FILE* fp) : f(fp) {}
  void raw(void* p, size_t n) {
    if (ok && fread(p, 1, n, f) != n) ok = false;
  }
  uint8_t u8() { uint8_t v = 0; raw(&v, 1); return v; }
  uint32_t u32() { uint32_t v = 0; raw(&v, 4); return v; }
  uint64_t u64() { uint64_t v = 0; raw(&v, 8); return v; }
  float f32() { float v = 0; raw(&v, 4); return v; }
  std::string str() {
    uint32_t n = u32();
    if (!ok || n > (1u << 28)) { ok = false; return {}; }
    std::string s(n, '\0');
    raw(s.data(), n);
    return s;
  }
};

struct Writer {
  FILE* f;
  bool ok = true;
  explicit Writer(FILE* fp) : f(fp) {}
  void raw(const void* p, size_t n) {
    if (ok && fwrite(p, 1, n, f) != n) ok = false;
  }
  void u8(uint8_t v) { raw(&v, 1); }
  void u32(uint32_t v) { raw(&v, 4); }
  void u64(uint64_t v) { raw(&v, 8); }
  void f32(float v) { raw(&v, 4); }
  void str(const std::string& s) { u32((uint32_t)s.size()); raw(s.data(), s.size()); }
};

uint64_t numel(const std::vector<uint64_t>& d) {
  uint64_t n = 1;
  for (auto v : d) n *= v;
  return n;
}

bool read_ghostflw(Reader& r, File& out) {
  uint32_t version = r.u32();
  if (!r.ok || version > 1) { g_error = "unsupported GHOSTFLW version"; return false; }
  uint32_t n = r.u32();
  for (uint32_t i = 0; i < n && r.ok; ++i) {
    Entry e;
    e.name = r.str();
    e.dtype = r.u8();
    uint32_t nd = r.u32();
    if (nd > 16) { r.ok = false; break; }
    for (uint32_t k = 0; k < nd; ++k) e.dims.push_back(r.u64());
    uint64_t ne = numel(e.dims);
    if (!r.ok || ne > (1ull << 36)) { r.ok = false; break; }
    e.data.resize(ne);
    r.raw(e.data.data(), ne * 4);
    out.tensors.push_back(std::move(e));
  }
  if (!r.ok) g_error = "truncated GHOSTFLW file";
  return r.ok;
}

bool read_gfcp(Reader& r, File& out) {
  uint8_t ver[3];
  r.raw(ver, 3);
  for (auto& m : out.meta) m = r.str();
  out.epoch = r.u64();
  out.loss = r.f32();
  uint32_t nx = r.u32();
  for (uint32_t i = 0; i < nx && r.ok; ++i) {
    std::string k = r.str(), v = r.str();
    out.extra.emplace_back(k, v);
  }
  uint32_t np = r.u32();
  for (uint32_t i = 0; i < np && r.ok; ++i) {
    Entry e;
    e.name = r.str();
    uint32_t nd = r.u32();
    if (nd > 16) { r.ok = false; break; }
    for (uint32_t k = 0; k < nd; ++k) e.dims.push_back(r.u64());
    uint64_t len = r.u64();
    if (!r.ok || len > (1ull << 36)) { r.ok = false; break; }
    e.data.resize(len);
    r.raw(e.data.data(), len * 4);
    out.tensors.push_back(std::move(e));
  }
  uint8_t has_opt = r.u8();
  if (r.ok && has_opt == 1) {
    uint32_t no = r.u32();
    for (uint32_t i = 0; i < no && r.ok; ++i) {
      Entry e;
      e.name = r.str();
      uint64_t len = r.u64();
      if (!r.ok || len > (1ull << 36)) { r.ok = false; break; }
      e.dims = {len};
      e.data.resize(len);
      r.raw(e.data.data(), len * 4);
      out.optimizer.push_back(std::move(e));
    }
  }
  if (!r.ok) g_error = "truncated GFCP file";
  return r.ok;
}

// ---- minimal JSON scanning for the safetensors header: {"name": {"dtype": "F32", "shape": [..], "data_offsets": [a, b]}, ...}
struct JsonCur {
  const std::string& s;
  size_t i = 0;
  explicit JsonCur(const std::string& t) : s(t) {}
  void ws() { while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i; }
  bool eat(char c) { ws(); if (i < s.size() && s[i] == c) { ++i; return true; } return false; }
  bool str(std::string& out) {
    ws();
    if (i >= s.size() || s[i] != '"') return false;
    ++i;
    out.clear();
    while (i < s.size() && s[i] != '"') {
      if (s[i] == '\\' && i + 1 < s.size()) { ++i; }
      out.push_back(s[i++]);
    }
    if (i >= s.size()) return false;
    ++i;
    return true;
  }
  bool num(uint64_t& v) {
    ws();
    if (i >= s.size() || s[i] < '0' || s[i] > '9') return false;
    v = 0;
    while (i < s.size() && s[i] >= '0' && s[i] <= '9') v = v * 10 + (uint64_t)(s[i++] - '0');
    return true;
  }
  bool skip_value() {  // skips any JSON value
    ws();
    if (i >= s.size()) return false;
    if (s[i] == '"') { std::string t; return str(t); }
    if (s[i] == '{' || s[i] == '[') {
      char open = s[i], close = open == '{' ? '}' : ']';
      int depth = 0;
      bool in_str = false;
      for (; i < s.size(); ++i) {
        if (in_str) { if (s[i] == '\\') ++i; else if (s[i] == '"') in_str = false; continue; }
        if (s[i] == '"') in_str = true;
        else if (s[i] == open) ++depth;
        else if (s[i] == close) { if (--depth == 0) { ++i; return true; } }
      }
      return false;
    }
    while (i < s.size() && s[i] != ',' && s[i] != '}' && s[i] != ']') ++i;
    return true;
  }
};

float half_to_float(uint16_t h) {
  uint32_t sign = (h >> 15) & 1, exp = (h >> 10) & 0x1f, man = h & 0x3ff, bits;
  if (exp == 0) {
    if (man == 0) bits = sign << 31;
    else {
      int e = -1;
      do { ++e; man <<= 1; } while (!(man & 0x400));
      bits = (sign << 31) | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ff) << 13);
    }
  } else if (exp == 31) bits = (sign << 31) | 0x7f800000u | (man << 13);
  else bits = (sign << 31) | ((exp + 112) << 23) | (man << 13);
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

bool read_safetensors(FILE* fp, File& out) {
  Reader r(fp);
  uint64_t hlen = r.u64();
  if (!r.ok || hlen > (1ull << 30)) { g_error = "bad safetensors header length"; return false; }
  std::string hdr(hlen, '\0');
  r.raw(hdr.data(), hlen);
  if (!r.ok) { g_error = "truncated safetensors header"; return false; }
  long data_start = ftell(fp);
  JsonCur c(hdr);
  if (!c.eat('{')) { g_error = "safetensors header is not an object"; return false; }
  while (true) {
    std::string name;
    if (!c.str(name)) break;
    if (!c.eat(':')) { g_error = "bad safetensors header"; return false; }
    if (name == "__metadata__") {
      if (!c.skip_value()) return false;
    } else {
      if (!c.eat('{')) { g_error = "bad tensor record"; return false; }
      Entry e;
      e.name = name;
      std::string dtype;
      uint64_t off0 = 0, off1 = 0;
      while (true) {
        std::string key;
        if (!c.str(key)) break;
        c.eat(':');
        if (key == "dtype") c.str(dtype);
        else if (key == "shape") {
          c.eat('[');
          uint64_t v;
          while (c.num(v)) { e.dims.push_back(v); if (!c.eat(',')) break; }
          c.eat(']');
        } else if (key == "data_offsets") {
          c.eat('[');
          c.num(off0); c.eat(','); c.num(off1);
          c.eat(']');
        } else c.skip_value();
        if (!c.eat(',')) break;
      }
      c.eat('}');
      uint64_t ne = numel(e.dims);
      size_t esz = dtype == "F32" ? 4 : dtype == "F64" || dtype == "I64" ? 8 : dtype == "I32" ? 4 :
                   (dtype == "F16" || dtype == "BF16") ? 2 : 0;
      if (esz == 0 || off1 - off0 != ne * esz) { g_error = "unsupported safetensors dtype " + dtype; return false; }
      std::vector<uint8_t> rawb(ne * esz);
      fseek(fp, data_start + (long)off0, SEEK_SET);
      if (fread(rawb.data(), 1, rawb.size(), fp) != rawb.size()) { g_error = "truncated safetensors data"; return false; }
      e.data.resize(ne);
      for (uint64_t k = 0; k < ne; ++k) {
        if (dtype == "F32") memcpy(&e.data[k], &rawb[k * 4], 4);
        else if (dtype == "F64") { double d; memcpy(&d, &rawb[k * 8], 8); e.data[k] = (float)d; }
        else if (dtype == "I64") { int64_t d; memcpy(&d, &rawb[k * 8], 8); e.data[k] = (float)d; }
        else if (dtype == "I32") { int32_t d; memcpy(&d, &rawb[k * 4], 4); e.data[k] = (float)d; }
        else if (dtype == "F16") { uint16_t h; memcpy(&h, &rawb[k * 2], 2); e.data[k] = half_to_float(h); }
        else { uint16_t h; memcpy(&h, &rawb[k * 2], 2); uint32_t b = (uint32_t)h << 16; memcpy(&e.data[k], &b, 4); }
      }
      e.dtype = dtype == "F16" ? 0 : dtype == "BF16" ? 1 : dtype == "F64" ? 3 : dtype == "I32" ? 6 : dtype == "I64" ? 7 : 2;
      out.tensors.push_back(std::move(e));
    }
    if (!c.eat(',')) break;
  }
  return true;
}

}  // namespace

GFIO_API const char* gfio_last_error() { return g_error.c_str(); }

// Opens any of the three formats (detected by magic). Returns a handle or null.
GFIO_API void* gfio_open(const char* path) {
  FILE* fp = fopen(path, "rb");
  if (!fp) { g_error = std::string("cannot open ") + path; return nullptr; }
  File* f = new File();
  char magic[8] = {0};
  size_t got = fread(magic, 1, 8, fp);
  bool ok = false;
  if (got == 8 && memcmp(magic, "GHOSTFLW", 8) == 0) {
    f->kind = 1;
    Reader r(fp);
    ok = read_ghostflw(r, *f);
  } else if (got >= 4 && memcmp(magic, "GFCP", 4) == 0) {
    f->kind = 2;
    fseek(fp, 4, SEEK_SET);
    Reader r(fp);
    ok = read_gfcp(r, *f);
  } else {
    f->kind = 3;
    fseek(fp, 0, SEEK_SET);
    ok = read_safetensors(fp, *f);
  }
  fclose(fp);
  if (!ok) { delete f; return nullptr; }
  return f;
}
GFIO_API void gfio_close(void* h) { delete static_cast<File*>(h); }
GFIO_API int gfio_kind(void* h) { return static_cast<File*>(h)->kind; }
GFIO_API int gfio_count(void* h, int section) {
  File* f = static_cast<File*>(h);
  return (int)(section == 0 ? f->tensors.size() : f->optimizer.size());
}
static Entry& ent(void* h, int section, int i) {
  File* f = static_cast<File*>(h);
  return section == 0 ? f->tensors[i] : f->optimizer[i];
}
GFIO_API const char* gfio_name(void* h, int section, int i) { return ent(h, section, i).name.c_str(); }
GFIO_API int gfio_dtype(void* h, int section, int i) { return ent(h, section, i).dtype; }
GFIO_API int gfio_ndim(void* h, int section, int i) { return (int)ent(h, section, i).dims.size(); }
GFIO_API void gfio_dims(void* h, int section, int i, uint64_t* out) {
  auto& d = ent(h, section, i).dims;
  for (size_t k = 0; k < d.size(); ++k) out[k] = d[k];
}
GFIO_API uint64_t gfio_numel(void* h, int section, int i) { return ent(h, section, i).data.size(); }
GFIO_API const float* gfio_data(void* h, int section, int i) { return ent(h, section, i).data.data(); }
GFIO_API const char* gfio_meta(void* h, int which) { return static_cast<File*>(h)->meta[which].c_str(); }
GFIO_API uint64_t gfio_epoch(void* h) { return static_cast<File*>(h)->epoch; }
GFIO_API float gfio_loss(void* h) { return static_cast<File*>(h)->loss; }
GFIO_API int gfio_extra_count(void* h) { return (int)static_cast<File*>(h)->extra.size(); }
GFIO_API const char* gfio_extra_key(void* h, int i) { return static_cast<File*>(h)->extra[i].first.c_str(); }
GFIO_API const char* gfio_extra_value(void* h, int i) { return static_cast<File*>(h)->extra[i].second.c_str(); }

// ---- writers: tensors are described by parallel arrays; dims_flat holds all dims back to back.
GFIO_API int gfio_write_ghostflw(const char* path, int n, const char* const* names, const uint8_t* dtypes,
                                 const int* ndims, const uint64_t* dims_flat, const float* const* data) {
  FILE* fp = fopen(path, "wb");
  if (!fp) { g_error = std::string("cannot create ") + path; return -1; }
  Writer w(fp);
  w.raw("GHOSTFLW", 8);
  w.u32(1);
  w.u32((uint32_t)n);
  size_t dpos = 0;
  for (int i = 0; i < n; ++i) {
    w.str(names[i]);
    w.u8(dtypes[i]);
    w.u32((uint32_t)ndims[i]);
    uint64_t ne = 1;
    for (int k = 0; k < ndims[i]; ++k) { w.u64(dims_flat[dpos + k]); ne *= dims_flat[dpos + k]; }
    dpos += ndims[i];
    w.raw(data[i], ne * 4);
  }
  fclose(fp);
  if (!w.ok) { g_error = "short write"; return -1; }
  return 0;
}

GFIO_API int gfio_write_gfcp(const char* path, const char* model_name, const char* version, const char* fw_version,
                             uint64_t epoch, float loss, int n_extra, const char* const* extra_keys,
                             const char* const* extra_vals, int n, const char* const* names, const int* ndims,
                             const uint64_t* dims_flat, const float* const* data, int n_opt,
                             const char* const* opt_names, const uint64_t* opt_lens, const float* const* opt_data) {
  FILE* fp = fopen(path, "wb");
  if (!fp) { g_error = std::string("cannot create ") + path; return -1; }
  Writer w(fp);
  w.raw("GFCP", 4);
  const uint8_t ver[3] = {0, 4, 0};
  w.raw(ver, 3);
  w.str(model_name); w.str(version); w.str(fw_version);
  w.u64(epoch);
  w.f32(loss);
  w.u32((uint32_t)n_extra);
  for (int i = 0; i < n_extra; ++i) { w.str(extra_keys[i]); w.str(extra_vals[i]); }
  w.u32((uint32_t)n);
  size_t dpos = 0;
  for (int i = 0; i < n; ++i) {
    w.str(names[i]);
    w.u32((uint32_t)ndims[i]);
    uint64_t ne = 1;
    for (int k = 0; k < ndims[i]; ++k) { w.u64(dims_flat[dpos + k]); ne *= dims_flat[dpos + k]; }
    dpos += ndims[i];
    w.u64(ne);
    w.raw(data[i], ne * 4);
  }
  w.u8(n_opt >= 0 ? 1 : 0);
  if (n_opt >= 0) {
    w.u32((uint32_t)n_opt);
    for (int i = 0; i < n_opt; ++i) { w.str(opt_names[i]); w.u64(opt_lens[i]); w.raw(opt_data[i], opt_lens[i] * 4); }
  }
  fclose(fp);
  if (!w.ok) { g_error = "short write"; return -1; }
  return 0;
}

GFIO_API int gfio_write_safetensors(const char* path, int n, const char* const* names, const int* ndims,
                                    const uint64_t* dims_flat, const float* const* data) {
  std::string hdr = "{";
  uint64_t off = 0;
  size_t dpos = 0;
  std::vector<uint64_t> sizes(n);
  for (int i = 0; i < n; ++i) {
    uint64_t ne = 1;
    std::string shape = "[";
    for (int k = 0; k < ndims[i]; ++k) {
      ne *= dims_flat[dpos + k];
      shape += std::to_string(dims_flat[dpos + k]);
      if (k + 1 < ndims[i]) shape += ",";
    }
    shape += "]";
    dpos += ndims[i];
    sizes[i] = ne * 4;
    std::string nm;
    for (const char* p = names[i]; *p; ++p) { if (*p == '"' || *p == '\\') nm.push_back('\\'); nm.push_back(*p); }
    hdr += "\"" + nm + "\":{\"dtype\":\"F32\",\"shape\":" + shape + ",\"data_offsets\":[" + std::to_string(off) + "," +
           std::to_string(off + sizes[i]) + "]}";
    if (i + 1 < n) hdr += ",";
    off += sizes[i];
  }
  hdr += "}";
  while (hdr.size() % 8) hdr.push_back(' ');
  FILE* fp = fopen(path, "wb");
  if (!fp) { g_error = std::string("cannot create ") + path; return -1; }
  Writer w(fp);
  w.u64(hdr.size());
  w.raw(hdr.data(), hdr.size());
  for (int i = 0; i < n; ++i) w.raw(data[i], sizes[i]);
  fclose(fp);
  if (!w.ok) { g_error = "short write"; return -1; }
  return 0;
}

// GGUF v2/v3 container parser over an mmap'd file or a caller-owned byte buffer.
// Produces a JSON description (metadata + tensor index) for the Python layer and hands out
// zero-copy tensor pointers into the mapping.
//
// Format rules mirrored from the reference parser (src/gguf/loader_parse.rs:2-300,
// src/gguf/types.rs:18-120): magic 0x46554747, versions 2..3, tensor_count <= 100000,
// metadata entries <= 10000, arrays <= 10M elements, n_dims <= 8, tensor data start aligned
// to `general.alignment` (default 32).  Dimensions are stored innermost-first on disk and are
// reported both ways ("ne" as stored, "shape" reversed to row-major).
#include "quant_blocks.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <stdexcept>
#include <string>
#include <vector>

namespace {

struct TensorInfo { std::string name; std::vector<uint64_t> ne; uint32_t qtype; uint64_t offset; uint64_t nbytes; };

struct Gguf {
  const uint8_t* base = nullptr; size_t size = 0; bool mapped = false; int fd = -1;
  uint32_t version = 0; uint64_t data_start = 0; uint32_t alignment = 32;
  std::vector<TensorInfo> tensors; std::string json;
};

struct Reader {
  const uint8_t* p; size_t n; size_t pos = 0;
  void need(size_t k) const { if (k > n - pos || pos > n) throw std::runtime_error("unexpected end of file at offset " + std::to_string(pos)); }
  template <class T> T get() { need(sizeof(T)); T v; memcpy(&v, p + pos, sizeof(T)); pos += sizeof(T); return v; }
  std::string str() {
    uint64_t len = get<uint64_t>();
    if (len > n - pos) throw std::runtime_error("string length " + std::to_string(len) + " exceeds file size");
    std::string s((const char*)p + pos, (size_t)len); pos += (size_t)len; return s;
  }
};

void json_escape(const std::string& s, std::string& out) {
  out.push_back('"');
  for (unsigned char c : s) {
    switch (c) {
      case '"': out += "\\\""; break; case '\\': out += "\\\\"; break;
      case '\n': out += "\\n"; break; case '\r': out += "\\r"; break; case '\t': out += "\\t"; break;
      default:
        if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); out += b; }
        else out.push_back((char)c);
    }
  }
  out.push_back('"');
}

void fmt_float(double v, std::string& out) {
  if (v != v) { out += "\"nan\""; return; }
  if (v > 1.7e308 || v < -1.7e308) { out += v > 0 ? "\"inf\"" : "\"-inf\""; return; }
  char b[40]; snprintf(b, sizeof b, "%.9g", v); out += b;
}

// value types: 0 u8,1 i8,2 u16,3 i16,4 u32,5 i32,6 f32,7 bool,8 string,9 array,10 u64,11 i64,12 f64
void read_scalar(Reader& r, uint32_t t, std::string& out, uint32_t* as_u32 = nullptr) {
  switch (t) {
    case 0: out += std::to_string(r.get<uint8_t>()); break;
    case 1: out += std::to_string(r.get<int8_t>()); break;
    case 2: out += std::to_string(r.get<uint16_t>()); break;
    case 3: out += std::to_string(r.get<int16_t>()); break;
    case 4: { uint32_t v = r.get<uint32_t>(); if (as_u32) *as_u32 = v; out += std::to_string(v); break; }
    case 5: out += std::to_string(r.get<int32_t>()); break;
    case 6: fmt_float(r.get<float>(), out); break;
    case 7: { uint8_t v = r.get<uint8_t>(); if (v > 1) throw std::runtime_error("invalid bool value"); out += v ? "true" : "false"; break; }
    case 8: json_escape(r.str(), out); break;
    case 10: out += std::to_string(r.get<uint64_t>()); break;
    case 11: out += std::to_string(r.get<int64_t>()); break;
    case 12: fmt_float(r.get<double>(), out); break;
    default: throw std::runtime_error("unknown metadata value type " + std::to_string(t));
  }
}

void parse(Gguf& g) {
  Reader r{g.base, g.size};
  if (g.size < 24) throw std::runtime_error("file too small for a GGUF header");
  uint32_t magic = r.get<uint32_t>();
  if (magic != 0x46554747u) { char b[64]; snprintf(b, sizeof b, "bad magic 0x%08x (want GGUF)", magic); throw std::runtime_error(b); }
  g.version = r.get<uint32_t>();
  if (g.version < 2 || g.version > 3) throw std::runtime_error("unsupported GGUF version " + std::to_string(g.version));
  uint64_t n_tensors = r.get<uint64_t>(), n_kv = r.get<uint64_t>();
  if (n_tensors > 100000) throw std::runtime_error("tensor_count " + std::to_string(n_tensors) + " exceeds limit 100000");
  if (n_kv > 10000) throw std::runtime_error("metadata_count " + std::to_string(n_kv) + " exceeds limit 10000");
  std::string& j = g.json;
  j = "{\"version\":" + std::to_string(g.version) + ",\"metadata\":{";
  for (uint64_t i = 0; i < n_kv; ++i) {
    std::string key = r.str();
    if (key.size() > 65535) throw std::runtime_error("metadata key too long");
    uint32_t t = r.get<uint32_t>();
    if (i) j.push_back(',');
    json_escape(key, j); j += ":{\"t\":" + std::to_string(t);
    if (t == 9) {
      uint32_t et = r.get<uint32_t>(); uint64_t len = r.get<uint64_t>();
      if (et == 9) throw std::runtime_error("nested arrays are not supported");
      if (len > 10000000ull) throw std::runtime_error("array length " + std::to_string(len) + " exceeds limit 10000000");
      j += ",\"et\":" + std::to_string(et) + ",\"v\":[";
      for (uint64_t e = 0; e < len; ++e) { if (e) j.push_back(','); read_scalar(r, et, j); }
      j += "]}";
    } else {
      j += ",\"v\":";
      uint32_t u = 0; read_scalar(r, t, j, &u);
      if (key == "general.alignment" && t == 4) { if (u == 0 || (u & (u - 1))) throw std::runtime_error("alignment must be a power of two"); g.alignment = u; }
      j += "}";
    }
  }
  j += "},\"tensors\":[";
  g.tensors.reserve((size_t)n_tensors);
  for (uint64_t i = 0; i < n_tensors; ++i) {
    TensorInfo ti; ti.name = r.str();
    uint32_t nd = r.get<uint32_t>();
    if (nd > 8) throw std::runtime_error("tensor '" + ti.name + "' has " + std::to_string(nd) + " dims (max 8)");
    uint64_t elems = 1;
    for (uint32_t d = 0; d < nd; ++d) {
      uint64_t e = r.get<uint64_t>();
      if (e != 0 && elems > UINT64_MAX / e) throw std::runtime_error("tensor '" + ti.name + "' element count overflows");
      elems *= e; ti.ne.push_back(e);
    }
    ti.qtype = r.get<uint32_t>(); ti.offset = r.get<uint64_t>();
    const int be = rlz::qtype_block_elems((int)ti.qtype), bb = rlz::qtype_block_bytes((int)ti.qtype);
    if (be == 0) ti.nbytes = 0;  // unknown type: listed but not readable
    else {
      if (!ti.ne.empty() && ti.ne[0] % (uint64_t)be) throw std::runtime_error("tensor '" + ti.name + "' row length not a multiple of its block size");
      ti.nbytes = elems / (uint64_t)be * (uint64_t)bb;
    }
    g.tensors.push_back(std::move(ti));
  }
  g.data_start = (r.pos + g.alignment - 1) / g.alignment * g.alignment;
  for (size_t i = 0; i < g.tensors.size(); ++i) {
    TensorInfo& ti = g.tensors[i];
    if (ti.nbytes && (ti.offset > g.size || g.data_start > g.size - ti.offset || ti.nbytes > g.size - g.data_start - ti.offset))
      throw std::runtime_error("tensor '" + ti.name + "' data exceeds file size");
    if (i) j.push_back(',');
    j += "{\"name\":"; json_escape(ti.name, j);
    j += ",\"ne\":[";
    for (size_t d = 0; d < ti.ne.size(); ++d) { if (d) j.push_back(','); j += std::to_string(ti.ne[d]); }
    j += "],\"shape\":[";
    for (size_t d = 0; d < ti.ne.size(); ++d) { if (d) j.push_back(','); j += std::to_string(ti.ne[ti.ne.size() - 1 - d]); }
    j += "],\"qtype\":" + std::to_string(ti.qtype) + ",\"offset\":" + std::to_string(g.data_start + ti.offset) + ",\"nbytes\":" + std::to_string(ti.nbytes) + "}";
  }
  j += "],\"data_start\":" + std::to_string(g.data_start) + ",\"alignment\":" + std::to_string(g.alignment) + "}";
}

void set_err(char* err, int errlen, const std::string& msg) { if (err && errlen > 0) snprintf(err, (size_t)errlen, "%s", msg.c_str()); }

}  // namespace

extern "C" {

void* rlz_gguf_open_buffer(const void* data, uint64_t size, char* err, int errlen) {
  Gguf* g = new Gguf(); g->base = (const uint8_t*)data; g->size = (size_t)size;
  try { parse(*g); } catch (const std::exception& e) { set_err(err, errlen, e.what()); delete g; return nullptr; }
  return g;
}

void* rlz_gguf_open_file(const char* path, char* err, int errlen) {
  int fd = open(path, O_RDONLY);
  if (fd < 0) { set_err(err, errlen, std::string("cannot open ") + path); return nullptr; }
  struct stat st; if (fstat(fd, &st) || st.st_size <= 0) { close(fd); set_err(err, errlen, "cannot stat file or file is empty"); return nullptr; }
  void* p = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  if (p == MAP_FAILED) { close(fd); set_err(err, errlen, "mmap failed"); return nullptr; }
  Gguf* g = new Gguf(); g->base = (const uint8_t*)p; g->size = (size_t)st.st_size; g->mapped = true; g->fd = fd;
  try { parse(*g); } catch (const std::exception& e) { set_err(err, errlen, e.what()); munmap(p, g->size); close(fd); delete g; return nullptr; }
  return g;
}

void rlz_gguf_close(void* h) {
  Gguf* g = (Gguf*)h; if (!g) return;
  if (g->mapped) { munmap((void*)g->base, g->size); close(g->fd); }
  delete g;
}

const char* rlz_gguf_json(void* h, uint64_t* len) { Gguf* g = (Gguf*)h; if (len) *len = g->json.size(); return g->json.c_str(); }
const void* rlz_gguf_base(void* h) { return ((Gguf*)h)->base; }
uint64_t rlz_gguf_size(void* h) { return ((Gguf*)h)->size; }

// madvise hints over the whole mapping: 0 normal, 1 sequential, 2 random, 3 willneed
int rlz_gguf_advise(void* h, int mode) {
  Gguf* g = (Gguf*)h; if (!g->mapped) return 0;
  int adv = mode == 1 ? MADV_SEQUENTIAL : mode == 2 ? MADV_RANDOM : mode == 3 ? MADV_WILLNEED : MADV_NORMAL;
  return madvise((void*)g->base, g->size, adv);
}
int rlz_gguf_lock(void* h) { Gguf* g = (Gguf*)h; return g->mapped ? mlock(g->base, g->size) : 0; }

}  // extern "C"

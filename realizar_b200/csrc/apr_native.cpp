// APR v2 container parser: 64-byte header, JSON metadata span, binary tensor index.
// Produces a JSON description of the index for the Python layer.
//
// Layout (reference: src/apr/mod.rs:80-403): magic "APR\0" or "APR2" ("APR1" is refused), version
// (2 bytes), flags u16 @6, tensor_count u32 @8, metadata_offset u64 @12, metadata_size u32 @20,
// tensor_index_offset u64 @24, data_offset u64 @32, checksum u32 @40.  Index entries:
// name_len u16, name, dtype u8 (ggml ids; 128/129 and legacy 8/9 = APR-native q4/q8), ndim u8,
// dims u64 x ndim, offset u64 (relative to data_offset), size u64.
#include <stdint.h>
#include <string.h>

#include <cstdio>
#include <stdexcept>
#include <string>

namespace {
template <class T> T rd(const uint8_t* p) { T v; memcpy(&v, p, sizeof(T)); return v; }

void esc(const std::string& s, std::string& out) {
  out.push_back('"');
  for (unsigned char c : s) {
    if (c == '"' || c == '\\') { out.push_back('\\'); out.push_back((char)c); }
    else if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); out += b; }
    else out.push_back((char)c);
  }
  out.push_back('"');
}
}  // namespace

extern "C" {

// Parses `data[0..size)`.  On success returns a malloc'd JSON string (free with rlz_apr_free) and 0 in *rc.
char* rlz_apr_parse(const uint8_t* data, uint64_t size, int* rc, char* err, int errlen) {
  auto fail = [&](int code, const std::string& msg) -> char* {
    *rc = code;
    if (err && errlen > 0) snprintf(err, (size_t)errlen, "%s", msg.c_str());
    return nullptr;
  };
  if (size < 64) return fail(-1, ".apr header too small: " + std::to_string(size) + " bytes (need 64)");
  if (memcmp(data, "APR", 3) != 0) return fail(-2, "invalid .apr magic");
  const uint8_t vb = data[3];
  if (vb == '1') return fail(-3, "APR v1 is not supported for inference; convert to APR v2");
  if (vb != 0 && vb != '2') return fail(-2, "invalid .apr version byte " + std::to_string(vb));
  const uint16_t flags = rd<uint16_t>(data + 6);
  const uint32_t n_tensors = rd<uint32_t>(data + 8);
  const uint64_t meta_off = rd<uint64_t>(data + 12);
  const uint32_t meta_size = rd<uint32_t>(data + 20);
  const uint64_t index_off = rd<uint64_t>(data + 24);
  const uint64_t data_off = rd<uint64_t>(data + 32);
  const uint32_t checksum = rd<uint32_t>(data + 40);
  if (n_tensors > 100000) return fail(-4, "tensor_count exceeds limit 100000");
  if (meta_off > size || meta_size > size - meta_off) return fail(-5, "metadata section exceeds file size");
  if (index_off > size || data_off > size) return fail(-5, "section offset exceeds file size");
  std::string j = "{\"version\":[" + std::to_string(data[4]) + "," + std::to_string(data[5]) + "],\"flags\":" + std::to_string(flags) +
                  ",\"tensor_count\":" + std::to_string(n_tensors) + ",\"metadata_offset\":" + std::to_string(meta_off) +
                  ",\"metadata_size\":" + std::to_string(meta_size) + ",\"tensor_index_offset\":" + std::to_string(index_off) +
                  ",\"data_offset\":" + std::to_string(data_off) + ",\"checksum\":" + std::to_string(checksum) + ",\"tensors\":[";
  uint64_t pos = index_off;
  for (uint32_t i = 0; i < n_tensors; ++i) {
    if (pos + 4 > size) return fail(-6, "tensor entry too short");
    const uint16_t nl = rd<uint16_t>(data + pos); pos += 2;
    if (nl == 0) return fail(-6, "tensor entry " + std::to_string(i) + " has an empty name (index shorter than tensor_count)");
    if (pos + nl + 2 > size) return fail(-6, "tensor entry truncated at name");
    std::string name((const char*)data + pos, nl); pos += nl;
    const uint8_t dtype = data[pos++]; const uint8_t nd = data[pos++];
    if (nd > 8) return fail(-7, "tensor '" + name + "' has more than 8 dims");
    if (pos + (uint64_t)nd * 8 + 16 > size) return fail(-6, "tensor entry truncated at shape");
    if (i) j.push_back(',');
    j += "{\"name\":"; esc(name, j); j += ",\"dtype\":" + std::to_string(dtype) + ",\"shape\":[";
    for (int d = 0; d < nd; ++d) { if (d) j.push_back(','); j += std::to_string(rd<uint64_t>(data + pos)); pos += 8; }
    const uint64_t off = rd<uint64_t>(data + pos), sz = rd<uint64_t>(data + pos + 8); pos += 16;
    if (data_off + off > size || sz > size - data_off - off) return fail(-8, "tensor '" + name + "' data exceeds file size");
    if (data_off >= index_off && pos > data_off) return fail(-6, "tensor index runs into the data section");
    j += "],\"offset\":" + std::to_string(data_off + off) + ",\"size\":" + std::to_string(sz) + "}";
  }
  j += "]}";
  char* out = (char*)malloc(j.size() + 1);
  memcpy(out, j.c_str(), j.size() + 1);
  *rc = 0;
  return out;
}

void rlz_apr_free(char* p) { free(p); }

// CRC32 (IEEE, reflected) used for the header checksum and file integrity checks
uint32_t rlz_crc32(const uint8_t* data, uint64_t n) {
  static uint32_t table[256]; static bool init = false;
  if (!init) { for (uint32_t i = 0; i < 256; ++i) { uint32_t c = i; for (int k = 0; k < 8; ++k) c = (c & 1) ? 0xEDB88320u ^ (c >> 1) : c >> 1; table[i] = c; } init = true; }
  uint32_t c = 0xFFFFFFFFu;
  for (uint64_t i = 0; i < n; ++i) c = table[(c ^ data[i]) & 0xFF] ^ (c >> 8);
  return c ^ 0xFFFFFFFFu;
}

}  // extern "C"

// Memory-mapped safetensors reader (host side).
//
// File format: 8-byte little-endian header length, a JSON object mapping tensor names to
// {"dtype", "shape", "data_offsets": [begin, end]} plus an optional "__metadata__" object of
// strings, then the raw tensor bytes. The file is mapped read-only; tensor data is handed to the
// caller as pointers into the mapping so that a device upload reads straight from the page cache.
//
// Same role as the reference's SafeTensorsLoader.Load / GetTensor
// (src/HartsyInference.ModelAssets/SafeTensors/SafeTensorsLoader.cs:23,52) and its MmapHandle
// (src/HartsyInference.Core/Memory/MmapHandle.cs).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#define B200_API extern "C" __attribute__((visibility("default")))

namespace {

struct TensorInfo {
  std::string name;
  std::string dtype;
  std::vector<int64_t> shape;
  uint64_t begin = 0, end = 0;
};

struct StFile {
  int fd = -1;
  uint8_t* map = nullptr;
  size_t size = 0;
  uint64_t header_len = 0;
  std::vector<TensorInfo> tensors;
  std::string metadata_json;   // the raw "__metadata__" object text ("{}" if absent)
  std::string error;
};

// Minimal JSON scanner for the restricted header grammar (objects, arrays, strings, integers).
struct Scanner {
  const char* p;
  const char* end;
  bool ok = true;
  void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool eat(char c) { ws(); if (p < end && *p == c) { ++p; return true; } return false; }
  std::string str() {
    ws();
    std::string out;
    if (p >= end || *p != '"') { ok = false; return out; }
    ++p;
    while (p < end && *p != '"') {
      if (*p == '\\' && p + 1 < end) {
        ++p;
        switch (*p) {
          case 'n': out.push_back('\n'); break;
          case 't': out.push_back('\t'); break;
          case 'r': out.push_back('\r'); break;
          case 'b': out.push_back('\b'); break;
          case 'f': out.push_back('\f'); break;
          case 'u': {
            // keep BMP code points as UTF-8
            if (p + 4 < end) {
              unsigned cp = 0;
              for (int i = 1; i <= 4; ++i) {
                char c = p[i];
                cp = cp * 16 + (c >= '0' && c <= '9' ? c - '0' : (c | 32) - 'a' + 10);
              }
              p += 4;
              if (cp < 0x80) out.push_back(static_cast<char>(cp));
              else if (cp < 0x800) { out.push_back(static_cast<char>(0xC0 | (cp >> 6))); out.push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
              else { out.push_back(static_cast<char>(0xE0 | (cp >> 12))); out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F))); out.push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
            }
            break;
          }
          default: out.push_back(*p);
        }
        ++p;
      } else {
        out.push_back(*p++);
      }
    }
    if (p >= end) { ok = false; return out; }
    ++p;
    return out;
  }
  int64_t integer() {
    ws();
    bool neg = false;
    if (p < end && *p == '-') { neg = true; ++p; }
    int64_t v = 0;
    bool any = false;
    while (p < end && *p >= '0' && *p <= '9') { v = v * 10 + (*p - '0'); ++p; any = true; }
    if (!any) ok = false;
    return neg ? -v : v;
  }
  // skips any JSON value, returns its raw text span
  std::string skip_value() {
    ws();
    const char* s = p;
    int depth = 0;
    bool in_str = false;
    while (p < end) {
      char c = *p;
      if (in_str) {
        if (c == '\\') { ++p; }
        else if (c == '"') in_str = false;
      } else {
        if (c == '"') in_str = true;
        else if (c == '{' || c == '[') ++depth;
        else if (c == '}' || c == ']') { if (depth == 0) break; --depth; if (depth == 0) { ++p; break; } }
        else if ((c == ',') && depth == 0) break;
      }
      ++p;
    }
    return std::string(s, p);
  }
};

bool parse_header(StFile& f, const char* text, size_t len) {
  Scanner sc{text, text + len};
  if (!sc.eat('{')) return false;
  if (sc.eat('}')) return true;
  while (sc.ok) {
    std::string key = sc.str();
    if (!sc.ok || !sc.eat(':')) return false;
    if (key == "__metadata__") {
      f.metadata_json = sc.skip_value();
    } else {
      TensorInfo t;
      t.name = key;
      if (!sc.eat('{')) return false;
      while (sc.ok) {
        std::string k = sc.str();
        if (!sc.eat(':')) return false;
        if (k == "dtype") t.dtype = sc.str();
        else if (k == "shape") {
          if (!sc.eat('[')) return false;
          if (!sc.eat(']')) {
            do { t.shape.push_back(sc.integer()); } while (sc.eat(','));
            if (!sc.eat(']')) return false;
          }
        } else if (k == "data_offsets") {
          if (!sc.eat('[')) return false;
          t.begin = static_cast<uint64_t>(sc.integer());
          if (!sc.eat(',')) return false;
          t.end = static_cast<uint64_t>(sc.integer());
          if (!sc.eat(']')) return false;
        } else {
          sc.skip_value();
        }
        if (sc.eat(',')) continue;
        if (sc.eat('}')) break;
        return false;
      }
      f.tensors.push_back(std::move(t));
    }
    if (sc.eat(',')) continue;
    if (sc.eat('}')) break;
    return false;
  }
  return sc.ok;
}

}  // namespace

B200_API void* b200_st_open(const char* path) {
  auto* f = new StFile();
  f->metadata_json = "{}";
  f->fd = ::open(path, O_RDONLY);
  if (f->fd < 0) { f->error = std::string("cannot open ") + path; return f; }
  struct stat st;
  if (fstat(f->fd, &st) != 0 || st.st_size < 8) { f->error = "file too small"; return f; }
  f->size = static_cast<size_t>(st.st_size);
  void* m = mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, f->fd, 0);
  if (m == MAP_FAILED) { f->error = "mmap failed"; return f; }
  f->map = static_cast<uint8_t*>(m);
  uint64_t hl = 0;
  memcpy(&hl, f->map, 8);
  if (hl > f->size - 8 || hl > (1ull << 30)) { f->error = "bad header length"; return f; }
  f->header_len = hl;
  if (!parse_header(*f, reinterpret_cast<const char*>(f->map + 8), static_cast<size_t>(hl))) {
    f->error = "malformed header";
    f->tensors.clear();
    return f;
  }
  const uint64_t data_size = f->size - 8 - hl;
  for (auto& t : f->tensors)
    if (t.begin > t.end || t.end > data_size) { f->error = "tensor " + t.name + " out of bounds"; f->tensors.clear(); break; }
  return f;
}
B200_API const char* b200_st_error(void* h) {
  auto* f = static_cast<StFile*>(h);
  return f->error.empty() ? nullptr : f->error.c_str();
}
B200_API void b200_st_close(void* h) {
  auto* f = static_cast<StFile*>(h);
  if (f->map) munmap(f->map, f->size);
  if (f->fd >= 0) ::close(f->fd);
  delete f;
}
B200_API int32_t b200_st_count(void* h) { return static_cast<int32_t>(static_cast<StFile*>(h)->tensors.size()); }
B200_API const char* b200_st_name(void* h, int32_t i) { return static_cast<StFile*>(h)->tensors[static_cast<size_t>(i)].name.c_str(); }
B200_API const char* b200_st_dtype(void* h, int32_t i) { return static_cast<StFile*>(h)->tensors[static_cast<size_t>(i)].dtype.c_str(); }
B200_API int32_t b200_st_ndim(void* h, int32_t i) { return static_cast<int32_t>(static_cast<StFile*>(h)->tensors[static_cast<size_t>(i)].shape.size()); }
B200_API void b200_st_shape(void* h, int32_t i, int64_t* out) {
  const auto& s = static_cast<StFile*>(h)->tensors[static_cast<size_t>(i)].shape;
  for (size_t k = 0; k < s.size(); ++k) out[k] = s[k];
}
B200_API const void* b200_st_data(void* h, int32_t i, uint64_t* nbytes) {
  auto* f = static_cast<StFile*>(h);
  const auto& t = f->tensors[static_cast<size_t>(i)];
  if (nbytes) *nbytes = t.end - t.begin;
  return f->map + 8 + f->header_len + t.begin;
}
B200_API const char* b200_st_metadata(void* h) { return static_cast<StFile*>(h)->metadata_json.c_str(); }

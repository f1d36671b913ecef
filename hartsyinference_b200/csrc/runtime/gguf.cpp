// GGUF container reader (v2 / v3) and host-side block codecs.
//
// The file is memory-mapped; metadata is handed to Python as one JSON document, tensor data as
// pointers into the mapping. The codecs are the fp32 oracle of the device dequant-GEMM kernels and
// the implementation of the CPU path: dequantise Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q8_1, Q2_K, Q3_K, Q4_K,
// Q5_K, Q6_K, Q8_K, IQ4_NL, MXFP4, F16, BF16 to fp32 and quantise fp32 to Q8_0 / Q4_0 / Q4_K.
//
// Counterparts in the reference: GgufLoader (header / KV / tensor-info parser;
// src/HartsyInference.ModelAssets/Gguf/GgufLoader.cs), the per-format codecs
// (src/HartsyInference.ModelAssets/Gguf/Codecs/Codec_Q8_0.cs:5-60, Codec_Q4_K.cs:5-45, ...) and
// GgufQuantizer / GgufWriter. Block geometry follows the ggml definitions those files restate.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#define B200_API extern "C" __attribute__((visibility("default")))

namespace {

float f16_to_f32(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ff;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) bits = sign;
    else {
      exp = 127 - 15 + 1;
      while ((man & 0x400) == 0) { man <<= 1; --exp; }
      man &= 0x3ff;
      bits = sign | (exp << 23) | (man << 13);
    }
  } else if (exp == 31) bits = sign | 0x7f800000u | (man << 13);
  else bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  float f;
  memcpy(&f, &bits, 4);
  return f;
}
uint16_t f32_to_f16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000;
  int32_t exp = static_cast<int32_t>((x >> 23) & 0xff) - 127 + 15;
  uint32_t man = x & 0x7fffff;
  if (exp >= 31) return static_cast<uint16_t>(sign | 0x7c00 | (((x >> 23) & 0xff) == 255 && man ? 0x200 : 0));
  if (exp <= 0) {
    if (exp < -10) return static_cast<uint16_t>(sign);
    man |= 0x800000;
    const int shift = 14 - exp;
    uint32_t r = man >> shift;
    if ((man >> (shift - 1)) & 1) ++r;
    return static_cast<uint16_t>(sign | r);
  }
  uint32_t r = (static_cast<uint32_t>(exp) << 10) | (man >> 13);
  if (man & 0x1000) ++r;
  return static_cast<uint16_t>(sign | r);
}

struct TypeInfo { int id; const char* name; int block; int bytes; };
const TypeInfo kTypes[] = {
    {0, "F32", 1, 4},     {1, "F16", 1, 2},     {2, "Q4_0", 32, 18},   {3, "Q4_1", 32, 20},
    {6, "Q5_0", 32, 22},  {7, "Q5_1", 32, 24},  {8, "Q8_0", 32, 34},   {9, "Q8_1", 32, 36},
    {10, "Q2_K", 256, 84}, {11, "Q3_K", 256, 110}, {12, "Q4_K", 256, 144}, {13, "Q5_K", 256, 176},
    {14, "Q6_K", 256, 210}, {15, "Q8_K", 256, 292}, {20, "IQ4_NL", 32, 18}, {24, "I8", 1, 1},
    {25, "I16", 1, 2},    {26, "I32", 1, 4},    {27, "I64", 1, 8},     {28, "F64", 1, 8},
    {30, "BF16", 1, 2},   {39, "MXFP4", 32, 17},
};
const TypeInfo* find_type(int id) {
  for (const auto& t : kTypes) if (t.id == id) return &t;
  return nullptr;
}

struct GTensor {
  std::string name;
  std::vector<int64_t> dims;   // ggml order: dims[0] is the contiguous dimension
  int type = 0;
  uint64_t offset = 0;
  uint64_t nbytes = 0;
};

struct GFile {
  int fd = -1;
  uint8_t* map = nullptr;
  size_t size = 0;
  uint32_t version = 0;
  uint64_t data_start = 0;
  std::vector<GTensor> tensors;
  std::string meta_json;
  std::string error;
};

struct Reader {
  const uint8_t* p;
  const uint8_t* end;
  bool ok = true;
  template <typename T> T get() {
    T v{};
    if (p + sizeof(T) > end) { ok = false; return v; }
    memcpy(&v, p, sizeof(T));
    p += sizeof(T);
    return v;
  }
  std::string str() {
    const uint64_t n = get<uint64_t>();
    if (!ok || n > static_cast<uint64_t>(end - p)) { ok = false; return {}; }
    std::string s(reinterpret_cast<const char*>(p), static_cast<size_t>(n));
    p += n;
    return s;
  }
};

void json_escape(const std::string& s, std::string& out) {
  out.push_back('"');
  for (unsigned char c : s) {
    switch (c) {
      case '"': out += "\\\""; break;
      case '\\': out += "\\\\"; break;
      case '\n': out += "\\n"; break;
      case '\r': out += "\\r"; break;
      case '\t': out += "\\t"; break;
      default:
        if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); out += b; }
        else out.push_back(static_cast<char>(c));
    }
  }
  out.push_back('"');
}

bool value_json(Reader& r, uint32_t type, std::string& out, int depth = 0) {
  char buf[64];
  switch (type) {
    case 0: snprintf(buf, sizeof buf, "%u", r.get<uint8_t>()); out += buf; break;
    case 1: snprintf(buf, sizeof buf, "%d", r.get<int8_t>()); out += buf; break;
    case 2: snprintf(buf, sizeof buf, "%u", r.get<uint16_t>()); out += buf; break;
    case 3: snprintf(buf, sizeof buf, "%d", r.get<int16_t>()); out += buf; break;
    case 4: snprintf(buf, sizeof buf, "%u", r.get<uint32_t>()); out += buf; break;
    case 5: snprintf(buf, sizeof buf, "%d", r.get<int32_t>()); out += buf; break;
    case 6: {
      const float f = r.get<float>();
      if (std::isfinite(f)) { snprintf(buf, sizeof buf, "%.9g", f); out += buf; } else out += "null";
      break;
    }
    case 7: out += r.get<uint8_t>() ? "true" : "false"; break;
    case 8: json_escape(r.str(), out); break;
    case 9: {
      if (depth > 2) return false;
      const uint32_t et = r.get<uint32_t>();
      const uint64_t n = r.get<uint64_t>();
      if (!r.ok || n > (1ull << 28)) return false;
      out.push_back('[');
      for (uint64_t i = 0; i < n; ++i) {
        if (i) out.push_back(',');
        if (!value_json(r, et, out, depth + 1) || !r.ok) return false;
      }
      out.push_back(']');
      break;
    }
    case 10: snprintf(buf, sizeof buf, "%llu", static_cast<unsigned long long>(r.get<uint64_t>())); out += buf; break;
    case 11: snprintf(buf, sizeof buf, "%lld", static_cast<long long>(r.get<int64_t>())); out += buf; break;
    case 12: {
      const double d = r.get<double>();
      if (std::isfinite(d)) { snprintf(buf, sizeof buf, "%.17g", d); out += buf; } else out += "null";
      break;
    }
    default: return false;
  }
  return r.ok;
}

}  // namespace

B200_API void* b200_gguf_open(const char* path) {
  auto* f = new GFile();
  f->fd = ::open(path, O_RDONLY);
  if (f->fd < 0) { f->error = std::string("cannot open ") + path; return f; }
  struct stat st;
  if (fstat(f->fd, &st) != 0 || st.st_size < 24) { f->error = "file too small"; return f; }
  f->size = static_cast<size_t>(st.st_size);
  void* m = mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, f->fd, 0);
  if (m == MAP_FAILED) { f->error = "mmap failed"; return f; }
  f->map = static_cast<uint8_t*>(m);
  Reader r{f->map, f->map + f->size};
  if (r.get<uint32_t>() != 0x46554747u) { f->error = "not a GGUF file"; return f; }
  f->version = r.get<uint32_t>();
  if (f->version < 2 || f->version > 3) { f->error = "unsupported GGUF version"; return f; }
  const uint64_t n_tensors = r.get<uint64_t>();
  const uint64_t n_kv = r.get<uint64_t>();
  if (!r.ok || n_tensors > (1u << 24) || n_kv > (1u << 24)) { f->error = "corrupt header"; return f; }
  uint64_t alignment = 32;
  std::string& js = f->meta_json;
  js = "{";
  for (uint64_t i = 0; i < n_kv; ++i) {
    const std::string key = r.str();
    const uint32_t type = r.get<uint32_t>();
    if (!r.ok) { f->error = "corrupt metadata"; return f; }
    if (i) js.push_back(',');
    json_escape(key, js);
    js.push_back(':');
    const uint8_t* before = r.p;
    if (!value_json(r, type, js)) { f->error = "corrupt metadata value for " + key; return f; }
    if (key == "general.alignment" && type == 4) { uint32_t a; memcpy(&a, before, 4); if (a) alignment = a; }
  }
  js.push_back('}');
  for (uint64_t i = 0; i < n_tensors; ++i) {
    GTensor t;
    t.name = r.str();
    const uint32_t nd = r.get<uint32_t>();
    if (!r.ok || nd > 8) { f->error = "corrupt tensor table"; f->tensors.clear(); return f; }
    uint64_t elems = 1;
    bool bad_dims = false;
    for (uint32_t d = 0; d < nd; ++d) {
      const int64_t v = static_cast<int64_t>(r.get<uint64_t>());
      t.dims.push_back(v);
      // a crafted file must not wrap the element count (and with it the bounds check below)
      if (v <= 0 || __builtin_mul_overflow(elems, static_cast<uint64_t>(v), &elems)) bad_dims = true;
    }
    if (bad_dims) { f->error = "bad dimensions in " + t.name; f->tensors.clear(); return f; }
    t.type = static_cast<int>(r.get<uint32_t>());
    t.offset = r.get<uint64_t>();
    const TypeInfo* ti = find_type(t.type);
    if (!r.ok || !ti) { f->error = "unknown tensor type in " + t.name; f->tensors.clear(); return f; }
    if (__builtin_mul_overflow(elems / static_cast<uint64_t>(ti->block), static_cast<uint64_t>(ti->bytes), &t.nbytes)) {
      f->error = "tensor size overflow in " + t.name; f->tensors.clear(); return f;
    }
    f->tensors.push_back(std::move(t));
  }
  const uint64_t pos = static_cast<uint64_t>(r.p - f->map);
  f->data_start = (pos + alignment - 1) / alignment * alignment;
  if (f->data_start > f->size) { f->error = "tensor data starts past the end of the file"; f->tensors.clear(); return f; }
  const uint64_t room = f->size - f->data_start;
  for (const auto& t : f->tensors)
    // written so that no sum can wrap: offset and size are each checked against what is left
    if (t.offset > room || t.nbytes > room - t.offset) { f->error = "tensor " + t.name + " out of bounds"; f->tensors.clear(); break; }
  return f;
}
B200_API const char* b200_gguf_error(void* h) { auto* f = static_cast<GFile*>(h); return f->error.empty() ? nullptr : f->error.c_str(); }
B200_API void b200_gguf_close(void* h) {
  auto* f = static_cast<GFile*>(h);
  if (f->map) munmap(f->map, f->size);
  if (f->fd >= 0) ::close(f->fd);
  delete f;
}
B200_API const char* b200_gguf_metadata(void* h) { return static_cast<GFile*>(h)->meta_json.c_str(); }
B200_API int32_t b200_gguf_version(void* h) { return static_cast<int32_t>(static_cast<GFile*>(h)->version); }
B200_API int32_t b200_gguf_count(void* h) { return static_cast<int32_t>(static_cast<GFile*>(h)->tensors.size()); }
B200_API const char* b200_gguf_name(void* h, int32_t i) { return static_cast<GFile*>(h)->tensors[static_cast<size_t>(i)].name.c_str(); }
B200_API int32_t b200_gguf_type(void* h, int32_t i) { return static_cast<GFile*>(h)->tensors[static_cast<size_t>(i)].type; }
B200_API int32_t b200_gguf_ndim(void* h, int32_t i) { return static_cast<int32_t>(static_cast<GFile*>(h)->tensors[static_cast<size_t>(i)].dims.size()); }
B200_API void b200_gguf_dims(void* h, int32_t i, int64_t* out) {
  const auto& d = static_cast<GFile*>(h)->tensors[static_cast<size_t>(i)].dims;
  for (size_t k = 0; k < d.size(); ++k) out[k] = d[k];
}
B200_API const void* b200_gguf_data(void* h, int32_t i, uint64_t* nbytes) {
  auto* f = static_cast<GFile*>(h);
  const auto& t = f->tensors[static_cast<size_t>(i)];
  if (nbytes) *nbytes = t.nbytes;
  return f->map + f->data_start + t.offset;
}
B200_API int32_t b200_ggml_type_info(int32_t type, int32_t* block, int32_t* bytes, char* name, int32_t cap) {
  const TypeInfo* t = find_type(type);
  if (!t) return -1;
  if (block) *block = t->block;
  if (bytes) *bytes = t->bytes;
  if (name && cap > 0) { strncpy(name, t->name, static_cast<size_t>(cap - 1)); name[cap - 1] = 0; }
  return 0;
}

// ------------------------------------------------------------------------------------------
// codecs
// ------------------------------------------------------------------------------------------
namespace {
inline void scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
  if (j < 4) { *d = q[j] & 63; *m = q[j + 4] & 63; }
  else { *d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); *m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}
const int8_t kIq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
inline uint16_t rd16(const uint8_t* p) { uint16_t v; memcpy(&v, p, 2); return v; }
}  // namespace

// Dequantise `n` elements (a multiple of the block size) of ggml type `type` to fp32.
B200_API int32_t b200_ggml_dequant(int32_t type, const void* src, float* y, int64_t n) {
  const uint8_t* p = static_cast<const uint8_t*>(src);
  const TypeInfo* ti = find_type(type);
  if (!ti || n % ti->block != 0) return -1;
  const int64_t nb = n / ti->block;
  switch (type) {
    case 0: memcpy(y, p, static_cast<size_t>(n) * 4); return 0;
    case 1: for (int64_t i = 0; i < n; ++i) y[i] = f16_to_f32(rd16(p + 2 * i)); return 0;
    case 30: for (int64_t i = 0; i < n; ++i) { uint32_t b = static_cast<uint32_t>(rd16(p + 2 * i)) << 16; memcpy(&y[i], &b, 4); } return 0;
    case 39: {   // one E8M0 scale byte, then E2M1 nibbles: element j low, element j + 16 high
      static const float kE2m1[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};
      for (int64_t b = 0; b < nb; ++b, p += 17, y += 32) {
        const float d = std::ldexp(1.0f, static_cast<int>(p[0]) - 127);
        const uint8_t* qs = p + 1;
        for (int j = 0; j < 16; ++j) { y[j] = kE2m1[qs[j] & 0xF] * d; y[j + 16] = kE2m1[qs[j] >> 4] * d; }
      }
      return 0;
    }
    case 2: case 20:
      for (int64_t b = 0; b < nb; ++b, p += 18, y += 32) {
        const float d = f16_to_f32(rd16(p));
        const uint8_t* qs = p + 2;
        for (int j = 0; j < 16; ++j) {
          if (type == 2) { y[j] = ((qs[j] & 0xF) - 8) * d; y[j + 16] = ((qs[j] >> 4) - 8) * d; }
          else { y[j] = kIq4nl[qs[j] & 0xF] * d; y[j + 16] = kIq4nl[qs[j] >> 4] * d; }
        }
      }
      return 0;
    case 3:
      for (int64_t b = 0; b < nb; ++b, p += 20, y += 32) {
        const float d = f16_to_f32(rd16(p)), m = f16_to_f32(rd16(p + 2));
        const uint8_t* qs = p + 4;
        for (int j = 0; j < 16; ++j) { y[j] = (qs[j] & 0xF) * d + m; y[j + 16] = (qs[j] >> 4) * d + m; }
      }
      return 0;
    case 6: case 7: {
      const int hdr = type == 6 ? 2 : 4;
      for (int64_t b = 0; b < nb; ++b, p += ti->bytes, y += 32) {
        const float d = f16_to_f32(rd16(p));
        const float m = type == 7 ? f16_to_f32(rd16(p + 2)) : 0.f;
        uint32_t qh; memcpy(&qh, p + hdr, 4);
        const uint8_t* qs = p + hdr + 4;
        for (int j = 0; j < 16; ++j) {
          const int x0 = (qs[j] & 0xF) | (((qh >> j) & 1) << 4);
          const int x1 = (qs[j] >> 4) | (((qh >> (j + 16)) & 1) << 4);
          if (type == 6) { y[j] = (x0 - 16) * d; y[j + 16] = (x1 - 16) * d; }
          else { y[j] = x0 * d + m; y[j + 16] = x1 * d + m; }
        }
      }
      return 0;
    }
    case 8:
      for (int64_t b = 0; b < nb; ++b, p += 34, y += 32) {
        const float d = f16_to_f32(rd16(p));
        const int8_t* q = reinterpret_cast<const int8_t*>(p + 2);
        for (int j = 0; j < 32; ++j) y[j] = q[j] * d;
      }
      return 0;
    case 10:
      for (int64_t b = 0; b < nb; ++b, p += 84) {
        const uint8_t* sc = p; const uint8_t* q = p + 16;
        const float d = f16_to_f32(rd16(p + 80)), dmin = f16_to_f32(rd16(p + 82));
        int is = 0;
        for (int n0 = 0; n0 < 256; n0 += 128) {
          int shift = 0;
          for (int j = 0; j < 4; ++j) {
            uint8_t s = sc[is++]; float dl = d * (s & 0xF), ml = dmin * (s >> 4);
            for (int l = 0; l < 16; ++l) *y++ = dl * ((q[l] >> shift) & 3) - ml;
            s = sc[is++]; dl = d * (s & 0xF); ml = dmin * (s >> 4);
            for (int l = 0; l < 16; ++l) *y++ = dl * ((q[l + 16] >> shift) & 3) - ml;
            shift += 2;
          }
          q += 32;
        }
      }
      return 0;
    case 9:    // Q8_1: scale, precomputed sum (unused when dequantising), 32 int8
      for (int64_t b = 0; b < nb; ++b, p += 36, y += 32) {
        const float d = f16_to_f32(rd16(p));
        const int8_t* q = reinterpret_cast<const int8_t*>(p + 4);
        for (int j = 0; j < 32; ++j) y[j] = q[j] * d;
      }
      return 0;
    case 15:   // Q8_K: fp32 scale, 256 int8, 16 block sums (unused when dequantising)
      for (int64_t b = 0; b < nb; ++b, p += 292, y += 256) {
        float d; memcpy(&d, p, 4);
        const int8_t* q = reinterpret_cast<const int8_t*>(p + 4);
        for (int j = 0; j < 256; ++j) y[j] = q[j] * d;
      }
      return 0;
    case 11:   // Q3_K: high-bit mask [32], 2-bit quants [64], sixteen 6-bit scales in 12 bytes, f16 scale
      for (int64_t b = 0; b < nb; ++b, p += 110) {
        const uint8_t* hm = p; const uint8_t* q = p + 32; const uint8_t* packed = p + 96;
        const float d = f16_to_f32(rd16(p + 108));
        // scale i: low 4 bits from bytes 0..7 (low nibble for i < 8, high nibble for i >= 8), top 2
        // bits from bytes 8..11 (byte 8 + i % 4, bit pair i / 4); stored with a bias of 32
        int sc[16];
        for (int i = 0; i < 16; ++i) {
          const int lo = i < 8 ? (packed[i] & 0xF) : (packed[i - 8] >> 4);
          const int hi = (packed[8 + (i & 3)] >> (2 * (i >> 2))) & 3;
          sc[i] = (lo | (hi << 4)) - 32;
        }
        int is = 0;
        uint8_t bit = 1;
        for (int half = 0; half < 2; ++half, q += 32) {
          for (int shift = 0; shift < 8; shift += 2, bit = static_cast<uint8_t>(bit << 1)) {
            for (int part = 0; part < 2; ++part) {
              const float dl = d * sc[is++];
              for (int l = 0; l < 16; ++l) {
                const int idx = part * 16 + l;
                const int v = ((q[idx] >> shift) & 3) - ((hm[idx] & bit) ? 0 : 4);
                *y++ = dl * v;
              }
            }
          }
        }
      }
      return 0;
    case 12:
      for (int64_t b = 0; b < nb; ++b, p += 144) {
        const float d = f16_to_f32(rd16(p)), dmin = f16_to_f32(rd16(p + 2));
        const uint8_t* sc = p + 4; const uint8_t* q = p + 16;
        int is = 0;
        for (int j = 0; j < 256; j += 64) {
          uint8_t s, m;
          scale_min_k4(is, sc, &s, &m); const float d1 = d * s, m1 = dmin * m;
          scale_min_k4(is + 1, sc, &s, &m); const float d2 = d * s, m2 = dmin * m;
          for (int l = 0; l < 32; ++l) *y++ = d1 * (q[l] & 0xF) - m1;
          for (int l = 0; l < 32; ++l) *y++ = d2 * (q[l] >> 4) - m2;
          q += 32; is += 2;
        }
      }
      return 0;
    case 13:
      for (int64_t b = 0; b < nb; ++b, p += 176) {
        const float d = f16_to_f32(rd16(p)), dmin = f16_to_f32(rd16(p + 2));
        const uint8_t* sc = p + 4; const uint8_t* qh = p + 16; const uint8_t* ql = p + 48;
        int is = 0; uint8_t u1 = 1, u2 = 2;
        for (int j = 0; j < 256; j += 64) {
          uint8_t s, m;
          scale_min_k4(is, sc, &s, &m); const float d1 = d * s, m1 = dmin * m;
          scale_min_k4(is + 1, sc, &s, &m); const float d2 = d * s, m2 = dmin * m;
          for (int l = 0; l < 32; ++l) *y++ = d1 * ((ql[l] & 0xF) + (qh[l] & u1 ? 16 : 0)) - m1;
          for (int l = 0; l < 32; ++l) *y++ = d2 * ((ql[l] >> 4) + (qh[l] & u2 ? 16 : 0)) - m2;
          ql += 32; is += 2; u1 <<= 2; u2 <<= 2;
        }
      }
      return 0;
    case 14:
      for (int64_t b = 0; b < nb; ++b, p += 210) {
        const uint8_t* ql = p; const uint8_t* qh = p + 128;
        const int8_t* sc = reinterpret_cast<const int8_t*>(p + 192);
        const float d = f16_to_f32(rd16(p + 208));
        for (int n0 = 0; n0 < 256; n0 += 128) {
          for (int l = 0; l < 32; ++l) {
            const int is = l / 16;
            const int q1 = static_cast<int>((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
            const int q2 = static_cast<int>((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
            const int q3 = static_cast<int>((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            const int q4 = static_cast<int>((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            y[l] = d * sc[is] * q1; y[l + 32] = d * sc[is + 2] * q2;
            y[l + 64] = d * sc[is + 4] * q3; y[l + 96] = d * sc[is + 6] * q4;
          }
          y += 128; ql += 64; qh += 32; sc += 8;
        }
      }
      return 0;
    default: return -2;
  }
}

// Quantise fp32 -> Q8_0 (type 8), Q4_0 (type 2) or Q4_K (type 12). n must be a block multiple.
B200_API int32_t b200_ggml_quant(int32_t type, const float* x, void* dst, int64_t n) {
  uint8_t* p = static_cast<uint8_t*>(dst);
  if (type == 8) {
    if (n % 32) return -1;
    for (int64_t b = 0; b < n / 32; ++b, x += 32, p += 34) {
      float amax = 0.f;
      for (int j = 0; j < 32; ++j) amax = std::fmax(amax, std::fabs(x[j]));
      const float d = amax / 127.f, id = d ? 1.f / d : 0.f;
      const uint16_t dh = f32_to_f16(d);
      memcpy(p, &dh, 2);
      int8_t* q = reinterpret_cast<int8_t*>(p + 2);
      for (int j = 0; j < 32; ++j) { int v = static_cast<int>(std::lround(x[j] * id)); q[j] = static_cast<int8_t>(v > 127 ? 127 : v < -127 ? -127 : v); }
    }
    return 0;
  }
  if (type == 2) {
    if (n % 32) return -1;
    for (int64_t b = 0; b < n / 32; ++b, x += 32, p += 18) {
      float amax = 0.f, mx = 0.f;
      for (int j = 0; j < 32; ++j) if (std::fabs(x[j]) > amax) { amax = std::fabs(x[j]); mx = x[j]; }
      const float d = mx / -8.f, id = d ? 1.f / d : 0.f;
      const uint16_t dh = f32_to_f16(d);
      memcpy(p, &dh, 2);
      for (int j = 0; j < 16; ++j) {
        int a = static_cast<int>(x[j] * id + 8.5f), c = static_cast<int>(x[j + 16] * id + 8.5f);
        a = a < 0 ? 0 : a > 15 ? 15 : a; c = c < 0 ? 0 : c > 15 ? 15 : c;
        p[2 + j] = static_cast<uint8_t>(a | (c << 4));
      }
    }
    return 0;
  }
  if (type == 12) {
    if (n % 256) return -1;
    for (int64_t b = 0; b < n / 256; ++b, x += 256, p += 144) {
      float scales[8], mins[8], max_scale = 0.f, max_min = 0.f;
      for (int j = 0; j < 8; ++j) {
        float lo = x[32 * j], hi = x[32 * j];
        for (int l = 1; l < 32; ++l) { lo = std::fmin(lo, x[32 * j + l]); hi = std::fmax(hi, x[32 * j + l]); }
        if (lo > 0) lo = 0;
        scales[j] = (hi - lo) / 15.f;
        mins[j] = -lo;
        max_scale = std::fmax(max_scale, scales[j]);
        max_min = std::fmax(max_min, mins[j]);
      }
      const float d = max_scale / 63.f, dmin = max_min / 63.f;
      const float id = d ? 1.f / d : 0.f, idmin = dmin ? 1.f / dmin : 0.f;
      const uint16_t dh = f32_to_f16(d), mh = f32_to_f16(dmin);
      memcpy(p, &dh, 2); memcpy(p + 2, &mh, 2);
      uint8_t* sc = p + 4;
      memset(sc, 0, 12);
      uint8_t ls[8], lm[8];
      for (int j = 0; j < 8; ++j) {
        int a = static_cast<int>(std::lround(scales[j] * id)), c = static_cast<int>(std::lround(mins[j] * idmin));
        ls[j] = static_cast<uint8_t>(a > 63 ? 63 : a); lm[j] = static_cast<uint8_t>(c > 63 ? 63 : c);
        if (j < 4) { sc[j] = ls[j]; sc[j + 4] = lm[j]; }
        else { sc[j + 4] = (ls[j] & 0xF) | ((lm[j] & 0xF) << 4); sc[j - 4] |= (ls[j] >> 4) << 6; sc[j] |= (lm[j] >> 4) << 6; }
      }
      const float df = f16_to_f32(dh), mf = f16_to_f32(mh);
      uint8_t* q = p + 16;
      for (int j = 0; j < 256; j += 64) {
        const int s0 = j / 32, s1 = s0 + 1;
        const float d0 = df * ls[s0], m0 = mf * lm[s0], d1 = df * ls[s1], m1 = mf * lm[s1];
        for (int l = 0; l < 32; ++l) {
          int a = d0 ? static_cast<int>(std::lround((x[j + l] + m0) / d0)) : 0;
          int c = d1 ? static_cast<int>(std::lround((x[j + 32 + l] + m1) / d1)) : 0;
          a = a < 0 ? 0 : a > 15 ? 15 : a; c = c < 0 ? 0 : c > 15 ? 15 : c;
          q[l] = static_cast<uint8_t>(a | (c << 4));
        }
        q += 32;
      }
    }
    return 0;
  }
  return -2;
}

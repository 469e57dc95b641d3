// Checkpoint loader: reads a GGUF file (the container the reference's client downloads and manages,
// crates/eidola-app-core/src/local_models.rs:29-34, 1310-1385) and hands its tensors to the engine, which quantises
// the linear layers to e4m3 with 128x128 block scales on the device and stores them as tiles.
//
// GGUF (version 2 and 3, little endian) as its published specification lays it out:
//   "GGUF" | u32 version | u64 tensor_count | u64 kv_count | kv_count x (string key, u32 type, value)
//   | tensor_count x (string name, u32 n_dims, n_dims x u64 extent (innermost first), u32 ggml type, u64 offset)
//   | padding to `general.alignment` (default 32) | tensor data
// Tensor types read here: F32 (0), F16 (1), BF16 (30) and three block formats of 32 elements along a row: Q4_0 (2),
// Q8_0 (8), MXFP4 (39), decoded to fp32 as their published definitions say (block_bytes / decode_block below); the other
// quantised GGUF types are refused by number.  Host code only;
// everything numeric happens in the engine.
#include "loader.h"

#include <string.h>

#include <algorithm>

namespace eb {

namespace {

struct Reader {
  FILE* f;
  bool ok = true;
  template <typename T>
  T get() {
    T v{};
    if (ok && fread(&v, sizeof(T), 1, f) != 1) ok = false;
    return v;
  }
  std::string str() {
    const uint64_t n = get<uint64_t>();
    if (!ok || n > (1u << 20)) {
      ok = false;
      return {};
    }
    std::string s((size_t)n, '\0');
    if (n && fread(&s[0], 1, (size_t)n, f) != n) ok = false;
    return s;
  }
  void skip(uint64_t n) {
    if (ok && fseeko(f, (off_t)n, SEEK_CUR) != 0) ok = false;
  }
};

// bytes of one scalar metadata value of `type`, 0 for strings and arrays
uint64_t scalar_bytes(uint32_t type) {
  switch (type) {
    case 0: case 1: case 7: return 1;
    case 2: case 3: return 2;
    case 4: case 5: case 6: return 4;
    case 10: case 11: case 12: return 8;
  }
  return 0;
}

bool skip_value(Reader& r, uint32_t type, uint32_t* as_u32) {
  if (const uint64_t b = scalar_bytes(type)) {
    if (as_u32 && type == 4) {
      *as_u32 = r.get<uint32_t>();
      return r.ok;
    }
    r.skip(b);
    return r.ok;
  }
  if (type == 8) {
    r.str();
    return r.ok;
  }
  if (type == 9) {
    const uint32_t et = r.get<uint32_t>();
    const uint64_t n = r.get<uint64_t>();
    if (!r.ok) return false;
    if (const uint64_t b = scalar_bytes(et)) {
      r.skip(b * n);
      return r.ok;
    }
    if (et != 8) return false;
    for (uint64_t i = 0; i < n && r.ok; ++i) r.str();
    return r.ok;
  }
  return false;
}

inline float half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {  // subnormal: normalise
      int e = -1;
      do {
        ++e;
        man <<= 1;
      } while (!(man & 0x400u));
      bits = sign | (uint32_t)(127 - 15 - e) << 23 | (man & 0x3FFu) << 13;
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | man << 13;
  } else {
    bits = sign | (exp + 127 - 15) << 23 | man << 13;
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

}  // namespace

GgufFile::~GgufFile() {
  if (f_) fclose(f_);
}

int32_t GgufFile::open(const char* path) {
  f_ = fopen(path, "rb");
  if (!f_) return fail(EB_ERR_ARG, "gguf: cannot open %s", path);
  Reader r{f_};
  char magic[4] = {0};
  if (fread(magic, 1, 4, f_) != 4 || memcmp(magic, "GGUF", 4) != 0) return fail(EB_ERR_ARG, "gguf: %s is not a GGUF file", path);
  const uint32_t version = r.get<uint32_t>();
  if (version != 2 && version != 3) return fail(EB_ERR_UNSUPPORTED, "gguf: version %u (2 and 3 are read)", version);
  const uint64_t n_tensors = r.get<uint64_t>(), n_kv = r.get<uint64_t>();
  if (!r.ok || n_tensors > (1u << 22) || n_kv > (1u << 22)) return fail(EB_ERR_ARG, "gguf: implausible header");
  uint32_t alignment = 32;
  for (uint64_t i = 0; i < n_kv; ++i) {
    const std::string key = r.str();
    const uint32_t type = r.get<uint32_t>();
    uint32_t v = 0;
    if (!r.ok || !skip_value(r, type, key == "general.alignment" ? &v : nullptr))
      return fail(EB_ERR_ARG, "gguf: metadata entry %llu cannot be read", (unsigned long long)i);
    if (key == "general.alignment" && type == 4 && v >= 1) alignment = v;
  }
  for (uint64_t i = 0; i < n_tensors; ++i) {
    GgufTensor t;
    const std::string name = r.str();
    const uint32_t nd = r.get<uint32_t>();
    if (!r.ok || nd < 1 || nd > 4) return fail(EB_ERR_ARG, "gguf: tensor %llu has %u dimensions", (unsigned long long)i, nd);
    t.n_dims = (int)nd;
    for (uint32_t d = 0; d < nd; ++d) t.ne[d] = (int64_t)r.get<uint64_t>();
    t.type = r.get<uint32_t>();
    t.offset = r.get<uint64_t>();
    if (!r.ok) return fail(EB_ERR_ARG, "gguf: tensor table is truncated");
    tensors_[name] = t;
  }
  const off_t here = ftello(f_);
  data_start_ = ((uint64_t)here + alignment - 1) / alignment * alignment;
  return EB_OK;
}

const GgufTensor* GgufFile::find(const std::string& name) const {
  auto it = tensors_.find(name);
  return it == tensors_.end() ? nullptr : &it->second;
}

namespace {

// Block formats: 32 consecutive elements of a row share one scale.
//   Q8_0  (34 bytes): fp16 d, int8 q[32]                      x[i] = d * q[i]
//   Q4_0  (18 bytes): fp16 d, 16 bytes of two 4-bit codes     x[i] = d * ((b[i] & 15) - 8), x[i + 16] = d * ((b[i] >> 4) - 8)
//   MXFP4 (17 bytes): e8m0 scale byte e, 16 bytes of two e2m1 codes (the OCP microscaling element: sign, 2 exponent
//                     bits, 1 mantissa bit: 0, 0.5, 1, 1.5, 2, 3, 4, 6), low nibbles the first 16 elements, high nibbles
//                     the last 16 as in Q4_0                   x = 2^(e - 127) * e2m1(code); e = 255 is NaN
int block_bytes(uint32_t type) { return type == 8 ? 34 : type == 2 ? 18 : type == 39 ? 17 : 0; }

void decode_block(uint32_t type, const uint8_t* b, float* x) {
  if (type == 8) {
    uint16_t h;
    memcpy(&h, b, 2);
    const float d = half_to_float(h);
    for (int i = 0; i < 32; ++i) x[i] = d * (float)(int8_t)b[2 + i];
  } else if (type == 2) {
    uint16_t h;
    memcpy(&h, b, 2);
    const float d = half_to_float(h);
    for (int i = 0; i < 16; ++i) {
      x[i] = d * (float)((int)(b[2 + i] & 15) - 8);
      x[i + 16] = d * (float)((int)(b[2 + i] >> 4) - 8);
    }
  } else {
    static const float kE2M1[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    const float d = b[0] == 255 ? NAN : ldexpf(1.0f, (int)b[0] - 127);
    for (int i = 0; i < 16; ++i) {
      const uint8_t lo = b[1 + i] & 15, hi = b[1 + i] >> 4;
      x[i] = d * ((lo & 8) ? -kE2M1[lo & 7] : kE2M1[lo & 7]);
      x[i + 16] = d * ((hi & 8) ? -kE2M1[hi & 7] : kE2M1[hi & 7]);
    }
  }
}

}  // namespace

int32_t GgufFile::read_f32(const GgufTensor& t, int64_t elem0, int64_t n, float* out) {
  if (elem0 < 0 || n < 0 || elem0 + n > t.elements()) return fail(EB_ERR_ARG, "gguf: elements [%lld, +%lld) outside the tensor", (long long)elem0, (long long)n);
  if (const int bb = block_bytes(t.type)) {
    if (t.ne[0] % 32) return fail(EB_ERR_UNSUPPORTED, "gguf: block-quantised rows of %lld elements (not a multiple of 32)", (long long)t.ne[0]);
    const int64_t b0 = elem0 / 32, b1 = (elem0 + n + 31) / 32;
    raw_.resize((size_t)((b1 - b0) * bb));
    if (fseeko(f_, (off_t)(data_start_ + t.offset + (uint64_t)b0 * bb), SEEK_SET) != 0) return fail(EB_ERR_ARG, "gguf: seek failed");
    if (fread(raw_.data(), 1, raw_.size(), f_) != raw_.size()) return fail(EB_ERR_ARG, "gguf: tensor data is truncated");
    float x[32];
    for (int64_t b = b0; b < b1; ++b) {
      decode_block(t.type, raw_.data() + (size_t)((b - b0) * bb), x);
      const int64_t lo = std::max<int64_t>(elem0, b * 32), hi = std::min<int64_t>(elem0 + n, b * 32 + 32);
      for (int64_t e = lo; e < hi; ++e) out[e - elem0] = x[e - b * 32];
    }
    return EB_OK;
  }
  int esz;
  switch (t.type) {
    case 0: esz = 4; break;
    case 1: case 30: esz = 2; break;
    default:
      return fail(EB_ERR_UNSUPPORTED, "gguf: tensor type %u is not F32, F16, BF16, Q4_0, Q8_0 or MXFP4 (the other quantised GGUF types are not read)", t.type);
  }
  if (fseeko(f_, (off_t)(data_start_ + t.offset + (uint64_t)elem0 * esz), SEEK_SET) != 0) return fail(EB_ERR_ARG, "gguf: seek failed");
  if (t.type == 0) {
    if (fread(out, 4, (size_t)n, f_) != (size_t)n) return fail(EB_ERR_ARG, "gguf: tensor data is truncated");
    return EB_OK;
  }
  tmp_.resize((size_t)n);
  if (fread(tmp_.data(), 2, (size_t)n, f_) != (size_t)n) return fail(EB_ERR_ARG, "gguf: tensor data is truncated");
  for (int64_t i = 0; i < n; ++i) {
    if (t.type == 30) {
      const uint32_t b = (uint32_t)tmp_[(size_t)i] << 16;
      memcpy(&out[i], &b, 4);
    } else {
      out[i] = half_to_float(tmp_[(size_t)i]);
    }
  }
  return EB_OK;
}

}  // namespace eb

extern "C" int32_t eb_gguf_read_f32(const char* path, const char* tensor, int64_t elem0, int64_t n, float* h_out, int32_t* ggml_type,
                                    int64_t* n_elements) {
  EB_REQUIRE(path && tensor, EB_ERR_ARG, "eb_gguf_read_f32: null");
  eb::GgufFile g;
  const int32_t rc = g.open(path);
  if (rc != EB_OK) return rc;
  const eb::GgufTensor* t = g.find(tensor);
  EB_REQUIRE(t, EB_ERR_ARG, "eb_gguf_read_f32: no tensor %s in %s", tensor, path);
  if (ggml_type) *ggml_type = (int32_t)t->type;
  if (n_elements) *n_elements = t->elements();
  if (n == 0) return EB_OK;
  EB_REQUIRE(h_out, EB_ERR_ARG, "eb_gguf_read_f32: null output");
  return g.read_f32(*t, elem0, n, h_out);
}

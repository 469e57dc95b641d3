// Checkpoint loader: reads a GGUF file (the container the reference's client downloads and manages,
// crates/eidola-app-core/src/local_models.rs:29-34, 1310-1385) and hands its tensors to the engine, which quantises
// the linear layers to e4m3 with 128x128 block scales on the device and stores them as tiles.
//
// GGUF (version 2 and 3, little endian) as its published specification lays it out:
//   "GGUF" | u32 version | u64 tensor_count | u64 kv_count | kv_count x (string key, u32 type, value)
//   | tensor_count x (string name, u32 n_dims, n_dims x u64 extent (innermost first), u32 ggml type, u64 offset)
//   | padding to `general.alignment` (default 32) | tensor data
// Tensor types read here: F32 (0), F16 (1), BF16 (30); quantised GGUF types are refused by name.  Host code only;
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

int32_t GgufFile::read_f32(const GgufTensor& t, int64_t elem0, int64_t n, float* out) {
  int esz;
  switch (t.type) {
    case 0: esz = 4; break;
    case 1: case 30: esz = 2; break;
    default:
      return fail(EB_ERR_UNSUPPORTED, "gguf: tensor type %u is not F32, F16 or BF16 (quantised GGUF types are not read)", t.type);
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

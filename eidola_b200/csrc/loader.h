// GGUF reader used by eb_engine_load_gguf (host only).
#pragma once

#include <stdint.h>
#include <stdio.h>

#include <map>
#include <string>
#include <vector>

#include "common.h"

namespace eb {

struct GgufTensor {
  int n_dims = 0;
  int64_t ne[4] = {1, 1, 1, 1};  // extents, innermost (columns) first
  uint32_t type = 0;            // ggml type: 0 F32, 1 F16, 30 BF16, 2 Q4_0, 8 Q8_0, 39 MXFP4
  uint64_t offset = 0;          // from the start of the data section
  int64_t elements() const { return ne[0] * ne[1] * ne[2] * ne[3]; }
};

class GgufFile {
 public:
  ~GgufFile();
  int32_t open(const char* path);
  const GgufTensor* find(const std::string& name) const;
  // n elements starting at element elem0 of the tensor, converted to fp32
  int32_t read_f32(const GgufTensor& t, int64_t elem0, int64_t n, float* out);

 private:
  FILE* f_ = nullptr;
  uint64_t data_start_ = 0;
  std::map<std::string, GgufTensor> tensors_;
  std::vector<uint16_t> tmp_;
  std::vector<uint8_t> raw_;
};

}  // namespace eb

// Shared host-side helpers of libeidola_b200: error reporting across the C ABI and the device status word.
#pragma once

#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/eidola_b200.h"

namespace eb {

// Records a message for eb_last_error() and returns `code`.
int32_t fail(int32_t code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

// Device pointer to this device's status word (allocated on first use; nullptr if CUDA is unavailable).
int32_t* status_word();

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace eb

#define EB_CUDA(expr)                                                                              \
  do {                                                                                             \
    cudaError_t _e = (expr);                                                                       \
    if (_e != cudaSuccess) return eb::fail((int32_t)_e, "%s: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

#define EB_REQUIRE(cond, code, ...) \
  do {                              \
    if (!(cond)) return eb::fail((code), __VA_ARGS__); \
  } while (0)

#define EB_LAUNCH_CHECK()                                                                        \
  do {                                                                                           \
    cudaError_t _e = cudaGetLastError();                                                         \
    if (_e != cudaSuccess) return eb::fail((int32_t)_e, "kernel launch: %s", cudaGetErrorString(_e)); \
  } while (0)

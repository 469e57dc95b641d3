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
// Status word built into the library for eb_attn_paged_sink_static on the current device; nullptr until that entry
// point has resolved it.
int32_t* static_status_word_if_ready();

// Polls a bounded device-side wait (mbarrier, flag) makes before it gives up with EB_DEV_WAIT_TIMEOUT.
// Default 1 << 22 (seconds); EIDOLA_B200_WAIT_TRIES or eb_wait_limit_set() change it for launches made afterwards.
uint32_t wait_tries();

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace eb

#ifdef __CUDACC__
#include <utility>
namespace eb {
// Programmatic dependent launch: a kernel launched through eb::launch may start (be scheduled, run its prologue)
// while its predecessor in the stream drains; it must call pdl_wait() before it touches any global memory and may
// call pdl_trigger() once its own successor is allowed to be scheduled.  EIDOLA_B200_NO_PDL=1 turns the launch
// attribute off (the device calls are then no-ops).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
bool pdl_enabled();
template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
}  // namespace eb
#endif

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

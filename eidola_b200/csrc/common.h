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

// What a consumer kernel needs to wait (bounded) for its peers' push `seq` itself, instead of behind a wait launch:
// the flag words the peers write in this rank's arena (slot seq % kPeerFlagSlots, one word per source rank).
// flags == nullptr: nothing to wait for.
constexpr int kPeerFlagSlots = 8;
constexpr int kPeerMaxRanks = 8;
struct PeerWait {
  const int32_t* flags;
  int32_t rank, size, seq;
  uint32_t tries;
  int32_t* status;
};
// Fills `out` for eb_symm `s` (peer.cu); patience 1..64 multiplies the wait limit.
int32_t symm_peer_wait(eb_symm* s, int32_t seq, int32_t patience, PeerWait* out);

// What a producer kernel needs to store its result straight into every rank's arena (its own included) and to raise the
// collective's flags itself, instead of leaving that to a push launch: dst[p] = this rank's plane in rank p's arena.
// size == 0: not in use.
struct PeerPlanes {
  uint8_t* dst[kPeerMaxRanks];
  int32_t* flags[kPeerMaxRanks];  // flag area of each rank's arena
  int32_t* counter;               // local: CTAs that have finished their stores
  int32_t rank, size, seq;
};
// Starts collective ++seq of `s` whose planes lie at dst_off + source_rank * plane_step in every arena (peer.cu).
int32_t symm_peer_planes(eb_symm* s, int64_t dst_off, int64_t plane_step, int64_t plane_bytes, PeerPlanes* out, int32_t* seq);

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
// Called by every thread of a CTA after its last store into the peers' arenas: the stores are fenced, and the CTA of
// the grid that arrives last writes the collective's sequence number into this rank's flag word on every
// peer (the protocol of the push kernels).
__device__ __forceinline__ void peer_arrive_cta(const PeerPlanes& a) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(a.counter, 1);
    if (prev == (int)(gridDim.x * gridDim.y * gridDim.z) - 1) {
      *a.counter = 0;  // every other CTA has arrived: the counter is free for the next collective
      __threadfence_system();
      for (int p = 0; p < a.size; ++p) {
        if (p == a.rank) continue;
        int32_t* f = a.flags[p] + (a.seq % kPeerFlagSlots) * kPeerMaxRanks + a.rank;
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(f), "r"(a.seq) : "memory");
      }
    }
  }
}
// Called by every thread of a CTA before it reads what its peers pushed: thread p polls the word rank p writes, with
// a bound (EB_DEV_WAIT_TIMEOUT when it runs out; the CTA then goes on and the step's results are void), then the CTA
// meets at a barrier.  The rows were not read by this kernel before, so no stale line can sit in L1.
__device__ __forceinline__ void peer_wait_cta(const PeerWait& w) {
  if (!w.flags) return;
  const int p = threadIdx.x;
  if (p < w.size && p != w.rank) {
    const int32_t* f = w.flags + (w.seq % kPeerFlagSlots) * kPeerMaxRanks + p;
    bool seen = false;
    for (uint32_t i = 0; i < w.tries && !seen; ++i) {
      int32_t v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      seen = v - w.seq >= 0;
      if (!seen && i > 16) __nanosleep(i < 4096 ? 32 : 256);
    }
    if (!seen) atomicOr(w.status, EB_DEV_WAIT_TIMEOUT);
  }
  __syncthreads();
}
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

// Symmetric peer memory and the small-message collectives of the tensor-/expert-parallel engine.
//
// One process per GPU.  Every rank allocates one arena of the same size and maps the arenas of its peers (CUDA IPC
// handles, exchanged once through the NCCL communicator), so a kernel of rank r can STORE into rank p's arena over
// NVLink / NVSwitch.  A decode step exchanges a few megabytes per layer: that is latency, not bandwidth, and a
// library collective costs tens of microseconds per call.  Here a collective is two small kernels:
//
//   push : every rank copies its rows straight into the place they belong in each peer's arena (plain 16-byte
//          stores to peer addresses), fences, and -- the last CTA to finish -- writes the collective's sequence
//          number into its flag word on every peer;
//   wait : one warp polls, with a bound, the flag words its peers write in ITS OWN arena, then returns; the consumer
//          kernels that follow in the stream read only local memory.
//
// No reduction happens in flight: the partial rows of a reduce-scatter land side by side as planes and the consumer
// (residual + RMSNorm) adds them in a fixed order in fp32, so the sum is rounded once and is the same on every run.
// Nothing here loads from a peer: no TMA, no multicast, no library kernel ever sees a peer address.
//
// Waiting on a peer is the one place where a kernel of one rank depends on another rank.  The wait is bounded
// (eb_wait_limit_set): when it runs out the kernel raises EB_DEV_WAIT_TIMEOUT and returns, the step's results are
// then meaningless and the host, which reads the status word after every step, treats the group as lost.
//
// The reference project has no collective communication (HTTP only).
#include <string.h>

#include <algorithm>
#include <new>
#include <vector>

#include "common.h"

namespace {

constexpr int kMaxRanks = eb::kPeerMaxRanks;
constexpr int kFlagSlots = eb::kPeerFlagSlots;  // collectives in flight never span more than two sequence numbers
constexpr int kMaxSegs = 4;
constexpr size_t kFlagBytes = 4096;  // flags + the push kernel's completion counter, at the end of the arena

struct PushSeg {
  int64_t src_off;         // byte offset in the local arena of the data for peer 0 (or for every peer when src_step == 0)
  int64_t src_step;        // added per destination rank
  int64_t dst_off;         // byte offset in the destination arena for source rank 0
  int64_t dst_step;        // added per SOURCE rank (this rank)
  int64_t bytes;           // per destination; 16-byte aligned segments move as 16-byte words, others as 4-byte words
  int64_t src_valid;       // bytes that exist from src_off on: destination p gets min(bytes, src_valid - p * src_step)
};

struct PushArgs {
  uint8_t* arena[kMaxRanks];
  int32_t* flags[kMaxRanks];  // flag area of each rank's arena
  int32_t* counter;           // local: CTAs that have finished their stores
  PushSeg seg[kMaxSegs];
  int32_t n_segs, rank, size, seq;
  int32_t self_copy;          // also copy to the own arena (a reduce-scatter keeps its own plane beside the peers')
};

__global__ void __launch_bounds__(256) symm_push_kernel(const PushArgs a) {
  eb::pdl_wait();  // the producer of the rows has completed
  eb::pdl_trigger();
  for (int s = 0; s < a.n_segs; ++s) {
    const PushSeg sg = a.seg[s];
    for (int p = 0; p < a.size; ++p) {
      if (p == a.rank && !a.self_copy) continue;
      const int64_t nb = max((int64_t)0, min(sg.bytes, sg.src_valid - (int64_t)p * sg.src_step));
      const uint8_t* src8 = a.arena[a.rank] + sg.src_off + (int64_t)p * sg.src_step;
      uint8_t* dst8 = a.arena[p] + sg.dst_off + (int64_t)a.rank * sg.dst_step;
      if (src8 == dst8) continue;
      const int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
      if ((((uintptr_t)src8 | (uintptr_t)dst8 | (uintptr_t)nb) & 15) == 0) {
        const uint4* src = reinterpret_cast<const uint4*>(src8);
        uint4* dst = reinterpret_cast<uint4*>(dst8);
        for (int64_t i = i0; i < (nb >> 4); i += stride) dst[i] = src[i];
      } else {  // small tables (block scales) whose slices are only 4-byte aligned
        const uint32_t* src = reinterpret_cast<const uint32_t*>(src8);
        uint32_t* dst = reinterpret_cast<uint32_t*>(dst8);
        for (int64_t i = i0; i < (nb >> 2); i += stride) dst[i] = src[i];
      }
    }
  }
  // every store of this CTA is ordered before its arrival; the last CTA to arrive publishes the sequence number
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(a.counter, 1);
    if (prev == (int)gridDim.x - 1) {
      *a.counter = 0;  // every other CTA has arrived: the counter is free for the next push
      __threadfence_system();
      const int slot = a.seq % kFlagSlots;
      for (int p = 0; p < a.size; ++p) {
        if (p == a.rank) continue;
        int32_t* f = a.flags[p] + slot * kMaxRanks + a.rank;
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(f), "r"(a.seq) : "memory");
      }
    }
  }
}

// Expert-parallel dispatch and return: whole rows to (rank, row) destinations computed from the routing, which every rank
// holds.  Row numbering is global (position in the expert-major order over all experts), so a row has the same offset
// in every rank's arena and neither direction needs a count exchange.
//   mode 0 (dispatch): row r of the grid is slot j = r % top_k of token t = t0 + r / top_k of this rank's token slice;
//                      it goes to the rank that holds expert idx[t][j], at row perm[t][j].
//   mode 1 (return)  : row i = seg[lo_e] + r of this rank's experts' range goes back to the owner of its token
//                      (rank row_token[i] / chunk), at the same row i.
struct RowsArgs {
  uint8_t* arena[kMaxRanks];
  int32_t* flags[kMaxRanks];
  int32_t* counter;
  int64_t src_off, dst_off;
  int32_t row_bytes, rank, size, seq, mode;
  const int32_t* idx;
  const int32_t* perm;
  int32_t t0, nt, top_k, e_l, n_experts;
  const int32_t* row_token;
  const int32_t* seg;
  int32_t lo_e, hi_e, chunk, n_rows;
  int32_t* status;
};

__global__ void __launch_bounds__(128) symm_rows_kernel(const RowsArgs a) {
  eb::pdl_wait();
  eb::pdl_trigger();
  const int r = blockIdx.x;
  int p = -1;
  int64_t srow = 0, drow = 0;
  if (a.mode == 0) {
    const int t = a.t0 + r / a.top_k, j = r % a.top_k;
    if (r < a.nt * a.top_k) {
      const int e = a.idx[(int64_t)t * a.top_k + j];
      const int d = a.perm[(int64_t)t * a.top_k + j];
      if (e < 0 || e >= a.n_experts || d < 0 || d >= a.n_rows) {
        if (threadIdx.x == 0) atomicOr(a.status, EB_DEV_BAD_INDEX);
      } else {
        p = e / a.e_l;
        srow = t;
        drow = d;
      }
    }
  } else {
    const int i = a.seg[a.lo_e] + r;
    if (i < a.seg[a.hi_e] && i >= 0 && i < a.n_rows) {
      const int t = a.row_token[i];
      if (t < 0) {
        if (threadIdx.x == 0) atomicOr(a.status, EB_DEV_BAD_INDEX);
      } else {
        p = min(t / a.chunk, a.size - 1);
        srow = drow = i;
      }
    }
  }
  if (p >= 0) {
    const uint4* src = reinterpret_cast<const uint4*>(a.arena[a.rank] + a.src_off + srow * a.row_bytes);
    uint4* dst = reinterpret_cast<uint4*>(a.arena[p] + a.dst_off + drow * a.row_bytes);
    if (src != dst)
      for (int c = threadIdx.x; c < (a.row_bytes >> 4); c += blockDim.x) dst[c] = src[c];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(a.counter, 1);
    if (prev == (int)gridDim.x - 1) {
      *a.counter = 0;
      __threadfence_system();
      const int slot = a.seq % kFlagSlots;
      for (int q = 0; q < a.size; ++q) {
        if (q == a.rank) continue;
        int32_t* f = a.flags[q] + slot * kMaxRanks + a.rank;
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(f), "r"(a.seq) : "memory");
      }
    }
  }
}

// One warp: lane p polls the word rank p writes.  Bounded; raises the status word when it gives up.
__global__ void symm_wait_kernel(const int32_t* flags, int rank, int size, int seq, uint32_t tries, int32_t* status) {
  eb::pdl_wait();
  eb::pdl_trigger();
  const int p = threadIdx.x;
  if (p >= size || p == rank) return;
  const int32_t* f = flags + (seq % kFlagSlots) * kMaxRanks + p;
  for (uint32_t i = 0; i < tries; ++i) {
    int32_t v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    if (v - seq >= 0) return;
    if (i > 16) __nanosleep(i < 4096 ? 32 : 256);
  }
  atomicOr(status, EB_DEV_WAIT_TIMEOUT);
}

}  // namespace

struct eb_symm {
  eb_comm* comm = nullptr;
  int rank = 0, size = 1;
  size_t bytes = 0;              // usable bytes (the flag area lies behind them)
  uint8_t* arena[kMaxRanks] = {nullptr};
  bool opened[kMaxRanks] = {false};
  int32_t seq = 0;               // sequence number of the last collective pushed
  int32_t waited = 0;
  int sms = 148;
};

namespace eb {
int32_t symm_peer_wait(eb_symm* s, int32_t seq, int32_t patience, PeerWait* out) {
  EB_REQUIRE(s && out && patience >= 1 && patience <= 64, EB_ERR_ARG, "peer wait: bad argument (patience 1..64)");
  *out = PeerWait{nullptr, s->rank, s->size, seq, 0, nullptr};
  if (s->size == 1) return EB_OK;
  out->status = eb::status_word();
  EB_REQUIRE(out->status, EB_ERR_NODEVICE, "peer wait: no device");
  out->flags = reinterpret_cast<const int32_t*>(s->arena[s->rank] + s->bytes);
  out->tries = (uint32_t)std::min<uint64_t>((uint64_t)eb::wait_tries() * (uint64_t)patience, 0x7fffffffull);
  s->waited = seq;
  return EB_OK;
}
int32_t symm_peer_planes(eb_symm* s, int64_t dst_off, int64_t plane_step, int64_t plane_bytes, PeerPlanes* out, int32_t* seq) {
  EB_REQUIRE(s && out && seq, EB_ERR_ARG, "peer planes: null argument");
  EB_REQUIRE(dst_off >= 0 && dst_off % 16 == 0 && plane_step >= plane_bytes && plane_step % 16 == 0 && plane_bytes >= 0 &&
                 dst_off + (int64_t)(s->size - 1) * plane_step + plane_bytes <= (int64_t)s->bytes,
             EB_ERR_ARG, "peer planes: %d planes of %lld bytes at %lld leave the arena of %zu bytes", s->size, (long long)plane_bytes,
             (long long)dst_off, s->bytes);
  *out = PeerPlanes{};
  out->rank = s->rank;
  out->size = s->size;
  out->seq = ++s->seq;
  *seq = out->seq;
  for (int p = 0; p < s->size; ++p) {
    out->dst[p] = s->arena[p] + dst_off + (int64_t)s->rank * plane_step;
    out->flags[p] = reinterpret_cast<int32_t*>(s->arena[p] + s->bytes);
  }
  out->counter = reinterpret_cast<int32_t*>(s->arena[s->rank] + s->bytes) + kFlagSlots * kMaxRanks;
  return EB_OK;
}
}  // namespace eb

extern "C" {

int32_t eb_symm_create(eb_comm* c, size_t bytes, eb_symm** out) {
  EB_REQUIRE(c && out && bytes > 0, EB_ERR_ARG, "eb_symm_create: bad argument");
  int32_t rank = 0, size = 1;
  int32_t rc = eb_comm_info(c, &rank, &size);
  if (rc != EB_OK) return rc;
  EB_REQUIRE(size >= 1 && size <= kMaxRanks, EB_ERR_UNSUPPORTED, "eb_symm_create: %d ranks (at most %d)", size, kMaxRanks);
  eb_symm* s = new (std::nothrow) eb_symm;
  EB_REQUIRE(s, EB_ERR_NOMEM, "eb_symm_create: host allocation failed");
  s->comm = c;
  s->rank = rank;
  s->size = size;
  s->bytes = (bytes + 255) & ~(size_t)255;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&s->sms, cudaDevAttrMultiProcessorCount, dev);
  const size_t total = s->bytes + kFlagBytes;
  cudaIpcMemHandle_t* d_handles = nullptr;
  auto fail = [&](int32_t code, const char* what, cudaError_t e) {
    if (d_handles) cudaFree(d_handles);
    eb_symm_destroy(s);
    return eb::fail(code, "eb_symm_create: %s: %s", what, cudaGetErrorString(e));
  };
  cudaError_t e = cudaMalloc((void**)&s->arena[rank], total);
  if (e != cudaSuccess) return fail((int32_t)e, "cudaMalloc", e);
  s->opened[rank] = false;
  if ((e = cudaMemset(s->arena[rank], 0, total)) != cudaSuccess) return fail((int32_t)e, "cudaMemset", e);
  if (size > 1) {
    // exchange the IPC handles through the communicator: every rank's 64 bytes, gathered in place on the device
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "CUDA IPC handle is 64 bytes");
    cudaIpcMemHandle_t mine;
    if ((e = cudaIpcGetMemHandle(&mine, s->arena[rank])) != cudaSuccess) return fail((int32_t)e, "cudaIpcGetMemHandle", e);
    if ((e = cudaMalloc((void**)&d_handles, sizeof(mine) * size)) != cudaSuccess) return fail((int32_t)e, "cudaMalloc", e);
    if ((e = cudaMemcpy(d_handles + rank, &mine, sizeof(mine), cudaMemcpyHostToDevice)) != cudaSuccess)
      return fail((int32_t)e, "cudaMemcpy", e);
    void* bufs[1] = {d_handles};
    const int64_t per[1] = {(int64_t)sizeof(mine)};
    rc = eb_comm_allgather(c, 1, bufs, per, nullptr);
    if (rc == EB_OK && (e = cudaDeviceSynchronize()) != cudaSuccess) rc = (int32_t)e;
    if (rc != EB_OK) {
      cudaFree(d_handles);
      eb_symm_destroy(s);
      return rc;
    }
    std::vector<cudaIpcMemHandle_t> all((size_t)size);
    if ((e = cudaMemcpy(all.data(), d_handles, sizeof(mine) * size, cudaMemcpyDeviceToHost)) != cudaSuccess)
      return fail((int32_t)e, "cudaMemcpy", e);
    cudaFree(d_handles);
    d_handles = nullptr;
    for (int p = 0; p < size; ++p) {
      if (p == rank) continue;
      void* ptr = nullptr;
      if ((e = cudaIpcOpenMemHandle(&ptr, all[(size_t)p], cudaIpcMemLazyEnablePeerAccess)) != cudaSuccess)
        return fail((int32_t)e, "cudaIpcOpenMemHandle (peer memory over NVLink is not available to this process)", e);
      s->arena[p] = (uint8_t*)ptr;
      s->opened[p] = true;
    }
    // nobody may push before every rank has mapped and cleared its arena: one more trip through the communicator
    int32_t* d_tok = nullptr;
    if ((e = cudaMalloc((void**)&d_tok, sizeof(int32_t) * size)) != cudaSuccess) return fail((int32_t)e, "cudaMalloc", e);
    void* b2[1] = {d_tok};
    const int64_t p2[1] = {4};
    rc = eb_comm_allgather(c, 1, b2, p2, nullptr);
    if (rc == EB_OK && (e = cudaDeviceSynchronize()) != cudaSuccess) rc = (int32_t)e;
    cudaFree(d_tok);
    if (rc != EB_OK) {
      eb_symm_destroy(s);
      return rc;
    }
  }
  *out = s;
  return EB_OK;
}

int32_t eb_symm_destroy(eb_symm* s) {
  if (!s) return EB_OK;
  cudaDeviceSynchronize();
  for (int p = 0; p < s->size; ++p)
    if (p != s->rank && s->opened[p] && s->arena[p]) cudaIpcCloseMemHandle(s->arena[p]);
  if (s->arena[s->rank]) cudaFree(s->arena[s->rank]);
  delete s;
  return EB_OK;
}

int32_t eb_symm_ptr(const eb_symm* s, int32_t rank, void** ptr, size_t* bytes) {
  EB_REQUIRE(s && ptr && rank >= 0 && rank < s->size, EB_ERR_ARG, "eb_symm_ptr: bad argument");
  *ptr = s->arena[rank];
  if (bytes) *bytes = s->bytes;
  return EB_OK;
}

// n_segs segments; segment i copies, for every destination rank p, `bytes[i]` bytes from local offset
// src_off[i] + p * src_step[i] to offset dst_off[i] + my_rank * dst_step[i] of rank p's arena.
//   all-gather of a buffer at offset o with b bytes per rank:  src_off = o + my_rank * b, src_step = 0, dst_off = o, dst_step = b
//   reduce-scatter planes (slice p of my partial -> plane my_rank at rank p): src_off = partial, src_step = slice bytes,
//                                                                              dst_off = planes, dst_step = slice bytes
// src_valid[i] (NULL = everything): bytes that exist from src_off[i] on; a destination whose part lies beyond gets less
// or nothing (the ragged last slice of a token range).
// Returns the collective's sequence number through seq; eb_symm_wait(seq) makes the peers' rows visible.
int32_t eb_symm_push(eb_symm* s, int32_t n_segs, const int64_t* src_off, const int64_t* src_step, const int64_t* dst_off,
                     const int64_t* dst_step, const int64_t* bytes, const int64_t* src_valid, int32_t self_copy, int32_t* seq,
                     void* stream) {
  EB_REQUIRE(s && src_off && src_step && dst_off && dst_step && bytes && seq && n_segs >= 1 && n_segs <= kMaxSegs, EB_ERR_ARG,
             "eb_symm_push: bad argument");
  PushArgs a = {};
  int64_t most = 0;
  for (int i = 0; i < n_segs; ++i) {
    EB_REQUIRE(bytes[i] >= 0 && bytes[i] % 4 == 0 && src_off[i] % 4 == 0 && dst_off[i] % 4 == 0 && src_step[i] % 4 == 0 &&
                   dst_step[i] % 4 == 0,
               EB_ERR_ARG, "eb_symm_push: segment %d is not 4-byte aligned", i);
    const int64_t src_end = src_off[i] + (int64_t)(s->size - 1) * src_step[i] + bytes[i];
    const int64_t dst_end = dst_off[i] + (int64_t)(s->size - 1) * dst_step[i] + bytes[i];
    EB_REQUIRE(src_off[i] >= 0 && dst_off[i] >= 0 && src_step[i] >= 0 && dst_step[i] >= 0 && src_end <= (int64_t)s->bytes &&
                   dst_end <= (int64_t)s->bytes,
               EB_ERR_ARG, "eb_symm_push: segment %d leaves the arena of %zu bytes", i, s->bytes);
    const int64_t valid = src_valid ? src_valid[i] : src_end - src_off[i];
    EB_REQUIRE(valid >= 0 && valid % 4 == 0, EB_ERR_ARG, "eb_symm_push: segment %d: valid bytes %lld", i, (long long)valid);
    a.seg[i] = PushSeg{src_off[i], src_step[i], dst_off[i], dst_step[i], bytes[i], valid};
    most = std::max(most, bytes[i]);
  }
  a.n_segs = n_segs;
  a.rank = s->rank;
  a.size = s->size;
  a.seq = ++s->seq;
  a.self_copy = self_copy;
  for (int p = 0; p < s->size; ++p) {
    a.arena[p] = s->arena[p];
    a.flags[p] = reinterpret_cast<int32_t*>(s->arena[p] + s->bytes);
  }
  a.counter = reinterpret_cast<int32_t*>(s->arena[s->rank] + s->bytes) + kFlagSlots * kMaxRanks;
  *seq = a.seq;
  if (s->size == 1) return EB_OK;
  // enough CTAs to keep the links busy, few enough that the last-arriver count stays cheap
  const int64_t per_cta = 16384;
  const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>((most * (s->size - 1) + per_cta - 1) / per_cta, s->sms));
  EB_CUDA(eb::launch(symm_push_kernel, dim3(grid), dim3(256), 0, eb::as_stream(stream), a));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

static int32_t rows_common(eb_symm* s, RowsArgs& a, int64_t src_off, int64_t dst_off, int32_t row_bytes, int32_t n_rows, int64_t grid,
                           int32_t* seq, void* stream) {
  EB_REQUIRE(row_bytes >= 16 && row_bytes % 16 == 0 && src_off >= 0 && dst_off >= 0 && src_off % 16 == 0 && dst_off % 16 == 0 &&
                 n_rows >= 0 && dst_off + (int64_t)n_rows * row_bytes <= (int64_t)s->bytes,
             EB_ERR_ARG, "eb_symm rows: %d rows of %d bytes at %lld leave the arena", n_rows, row_bytes, (long long)dst_off);
  int32_t* status = eb::status_word();
  EB_REQUIRE(status, EB_ERR_NODEVICE, "eb_symm rows: no device");
  a.src_off = src_off;
  a.dst_off = dst_off;
  a.row_bytes = row_bytes;
  a.rank = s->rank;
  a.size = s->size;
  a.seq = ++s->seq;
  a.n_rows = n_rows;
  a.status = status;
  for (int p = 0; p < s->size; ++p) {
    a.arena[p] = s->arena[p];
    a.flags[p] = reinterpret_cast<int32_t*>(s->arena[p] + s->bytes);
  }
  a.counter = reinterpret_cast<int32_t*>(s->arena[s->rank] + s->bytes) + kFlagSlots * kMaxRanks;
  *seq = a.seq;
  EB_CUDA(eb::launch(symm_rows_kernel, dim3((unsigned)std::max<int64_t>(1, grid)), dim3(128), 0, eb::as_stream(stream), a));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_symm_dispatch_rows(eb_symm* s, int64_t src_off, int64_t dst_off, int32_t row_bytes, const int32_t* d_idx,
                              const int32_t* d_perm, int32_t t0, int32_t nt, int32_t top_k, int32_t experts_per_rank,
                              int32_t n_experts, int32_t n_rows, int32_t* seq, void* stream) {
  EB_REQUIRE(s && d_idx && d_perm && seq && t0 >= 0 && nt >= 0 && top_k >= 1 && experts_per_rank >= 1 &&
                 n_experts == experts_per_rank * s->size,
             EB_ERR_ARG, "eb_symm_dispatch_rows: bad argument");
  RowsArgs a = {};
  a.mode = 0;
  a.idx = d_idx;
  a.perm = d_perm;
  a.t0 = t0;
  a.nt = nt;
  a.top_k = top_k;
  a.e_l = experts_per_rank;
  a.n_experts = n_experts;
  return rows_common(s, a, src_off, dst_off, row_bytes, n_rows, (int64_t)nt * top_k, seq, stream);
}

int32_t eb_symm_return_rows(eb_symm* s, int64_t src_off, int64_t dst_off, int32_t row_bytes, const int32_t* d_row_token,
                            const int32_t* d_seg_off, int32_t first_expert, int32_t experts_per_rank, int32_t chunk_tokens,
                            int32_t n_rows, int32_t* seq, void* stream) {
  EB_REQUIRE(s && d_row_token && d_seg_off && seq && first_expert >= 0 && experts_per_rank >= 1 && chunk_tokens >= 1, EB_ERR_ARG,
             "eb_symm_return_rows: bad argument");
  RowsArgs a = {};
  a.mode = 1;
  a.row_token = d_row_token;
  a.seg = d_seg_off;
  a.lo_e = first_expert;
  a.hi_e = first_expert + experts_per_rank;
  a.chunk = chunk_tokens;
  return rows_common(s, a, src_off, dst_off, row_bytes, n_rows, n_rows, seq, stream);
}

int32_t eb_symm_wait(eb_symm* s, int32_t seq, int32_t patience, void* stream) {
  EB_REQUIRE(s && patience >= 1 && patience <= 64, EB_ERR_ARG, "eb_symm_wait: bad argument (patience 1..64)");
  if (s->size == 1) return EB_OK;
  int32_t* status = eb::status_word();
  EB_REQUIRE(status, EB_ERR_NODEVICE, "eb_symm_wait: no device");
  const int32_t* flags = reinterpret_cast<const int32_t*>(s->arena[s->rank] + s->bytes);
  EB_CUDA(eb::launch(symm_wait_kernel, dim3(1), dim3(32), 0, eb::as_stream(stream), flags, s->rank, s->size, seq,
                     (uint32_t)std::min<uint64_t>((uint64_t)eb::wait_tries() * (uint64_t)patience, 0x7fffffffull), status));
  EB_LAUNCH_CHECK();
  s->waited = seq;
  return EB_OK;
}

}  // extern "C"

// Device-memory plumbing, the status word, and the seeded tensor generators of libeidola_b200.
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <string>

#include "../../include/eb_synth.h"
#include "common.h"

namespace eb {

static thread_local std::string g_last_error;

int32_t fail(int32_t code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

bool pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("EIDOLA_B200_NO_PDL");
    return !(v && v[0] == '1');
  }();
  return on;
}

static std::atomic<uint32_t> g_wait_tries{0};

uint32_t wait_tries() {
  uint32_t v = g_wait_tries.load(std::memory_order_relaxed);
  if (v == 0) {
    v = 1u << 22;
    if (const char* e = getenv("EIDOLA_B200_WAIT_TRIES")) {
      const long long x = atoll(e);
      if (x >= 1 && x <= 0x7fffffffll) v = (uint32_t)x;
    }
    g_wait_tries.store(v, std::memory_order_relaxed);
  }
  return v;
}

static std::mutex g_status_mu;
static int32_t* g_status_ptr[64] = {nullptr};

int32_t* status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_status_mu);
  if (!g_status_ptr[dev]) {
    int32_t* p = nullptr;
    if (cudaMalloc(&p, sizeof(int32_t)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, sizeof(int32_t));
    g_status_ptr[dev] = p;
  }
  return g_status_ptr[dev];
}

}  // namespace eb

using eb::as_stream;

extern "C" {

int32_t eb_version(int32_t* abi) {
  if (abi) *abi = EB_ABI_VERSION;
  return EB_OK;
}

int32_t eb_last_error(char* buf, size_t n) {
  if (!buf || n == 0) return EB_ERR_ARG;
  strncpy(buf, eb::g_last_error.c_str(), n - 1);
  buf[n - 1] = 0;
  return EB_OK;
}

int32_t eb_device_count(int32_t* n) {
  EB_REQUIRE(n, EB_ERR_ARG, "eb_device_count: null");
  int c = 0;
  cudaError_t e = cudaGetDeviceCount(&c);
  if (e != cudaSuccess) {
    *n = 0;
    return eb::fail(EB_ERR_NODEVICE, "cudaGetDeviceCount: %s", cudaGetErrorString(e));
  }
  *n = c;
  return EB_OK;
}

int32_t eb_device_set(int32_t device) {
  EB_CUDA(cudaSetDevice(device));
  return EB_OK;
}

int32_t eb_device_info(int32_t device, int32_t* sm_count, int64_t* l2_bytes, int64_t* hbm_bytes, int32_t* cc_major,
                       int32_t* cc_minor) {
  cudaDeviceProp p;
  EB_CUDA(cudaGetDeviceProperties(&p, device));
  if (sm_count) *sm_count = p.multiProcessorCount;
  if (l2_bytes) *l2_bytes = p.l2CacheSize;
  if (hbm_bytes) *hbm_bytes = (int64_t)p.totalGlobalMem;
  if (cc_major) *cc_major = p.major;
  if (cc_minor) *cc_minor = p.minor;
  return EB_OK;
}

int32_t eb_device_mem_info(int64_t* free_bytes, int64_t* total_bytes) {
  size_t f = 0, t = 0;
  EB_CUDA(cudaMemGetInfo(&f, &t));
  if (free_bytes) *free_bytes = (int64_t)f;
  if (total_bytes) *total_bytes = (int64_t)t;
  return EB_OK;
}

int32_t eb_malloc(void** d_ptr, size_t bytes) {
  EB_REQUIRE(d_ptr, EB_ERR_ARG, "eb_malloc: null");
  EB_CUDA(cudaMalloc(d_ptr, bytes ? bytes : 1));
  return EB_OK;
}
int32_t eb_free(void* d_ptr) {
  EB_CUDA(cudaFree(d_ptr));
  return EB_OK;
}
int32_t eb_host_alloc(void** h_ptr, size_t bytes) {
  EB_REQUIRE(h_ptr, EB_ERR_ARG, "eb_host_alloc: null");
  EB_CUDA(cudaMallocHost(h_ptr, bytes ? bytes : 1));
  return EB_OK;
}
int32_t eb_host_free(void* h_ptr) {
  EB_CUDA(cudaFreeHost(h_ptr));
  return EB_OK;
}
int32_t eb_memset(void* d_ptr, int32_t value, size_t bytes, void* stream) {
  EB_CUDA(cudaMemsetAsync(d_ptr, value, bytes, as_stream(stream)));
  return EB_OK;
}
int32_t eb_copy_h2d(void* d_dst, const void* h_src, size_t bytes, void* stream) {
  EB_CUDA(cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
  return EB_OK;
}
int32_t eb_copy_d2h(void* h_dst, const void* d_src, size_t bytes, void* stream) {
  EB_CUDA(cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
  return EB_OK;
}
int32_t eb_copy_d2d(void* d_dst, const void* d_src, size_t bytes, void* stream) {
  EB_CUDA(cudaMemcpyAsync(d_dst, d_src, bytes, cudaMemcpyDeviceToDevice, as_stream(stream)));
  return EB_OK;
}
int32_t eb_stream_create(void** stream) {
  EB_REQUIRE(stream, EB_ERR_ARG, "eb_stream_create: null");
  cudaStream_t s;
  EB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *stream = s;
  return EB_OK;
}
int32_t eb_stream_destroy(void* stream) {
  EB_CUDA(cudaStreamDestroy(as_stream(stream)));
  return EB_OK;
}
int32_t eb_stream_sync(void* stream) {
  EB_CUDA(cudaStreamSynchronize(as_stream(stream)));
  return EB_OK;
}
int32_t eb_device_sync(void) {
  EB_CUDA(cudaDeviceSynchronize());
  return EB_OK;
}
int32_t eb_event_create(void** ev) {
  EB_REQUIRE(ev, EB_ERR_ARG, "eb_event_create: null");
  cudaEvent_t e;
  EB_CUDA(cudaEventCreate(&e));
  *ev = e;
  return EB_OK;
}
int32_t eb_event_destroy(void* ev) {
  EB_CUDA(cudaEventDestroy((cudaEvent_t)ev));
  return EB_OK;
}
int32_t eb_event_record(void* ev, void* stream) {
  EB_CUDA(cudaEventRecord((cudaEvent_t)ev, as_stream(stream)));
  return EB_OK;
}
int32_t eb_event_elapsed_ms(void* ev_start, void* ev_stop, float* ms) {
  EB_REQUIRE(ms, EB_ERR_ARG, "eb_event_elapsed_ms: null");
  EB_CUDA(cudaEventSynchronize((cudaEvent_t)ev_stop));
  EB_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)ev_start, (cudaEvent_t)ev_stop));
  return EB_OK;
}

int32_t eb_wait_limit_set(uint32_t tries) {
  EB_REQUIRE(tries >= 1 && tries <= 0x7fffffffu, EB_ERR_ARG, "eb_wait_limit_set: %u polls outside 1..2^31-1", tries);
  eb::g_wait_tries.store(tries, std::memory_order_relaxed);
  return EB_OK;
}

int32_t eb_wait_limit_get(uint32_t* tries) {
  EB_REQUIRE(tries, EB_ERR_ARG, "eb_wait_limit_get: null");
  *tries = eb::wait_tries();
  return EB_OK;
}

int32_t eb_status_read(int32_t* status) {
  EB_REQUIRE(status, EB_ERR_ARG, "eb_status_read: null");
  int32_t* p = eb::status_word();
  EB_REQUIRE(p, EB_ERR_NODEVICE, "eb_status_read: no device status word");
  EB_CUDA(cudaMemcpy(status, p, sizeof(int32_t), cudaMemcpyDeviceToHost));
  EB_CUDA(cudaMemset(p, 0, sizeof(int32_t)));
  // bits raised by eb_attn_paged_sink_static calls that passed no status word of their own
  if (int32_t* q = eb::static_status_word_if_ready()) {
    int32_t extra = 0;
    EB_CUDA(cudaMemcpy(&extra, q, sizeof(int32_t), cudaMemcpyDeviceToHost));
    EB_CUDA(cudaMemset(q, 0, sizeof(int32_t)));
    *status |= extra;
  }
  return EB_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// kernels

namespace {

// One CTA waits, with the library's bounded-wait discipline, on a shared-memory barrier that nothing will ever
// complete: the wait runs out after `tries` polls, the status word gets EB_DEV_WAIT_TIMEOUT and the kernel returns.
__global__ void wait_expires_kernel(uint32_t tries, int32_t* status, uint32_t* polls_out) {
  __shared__ uint64_t bar;
  const uint32_t b = (uint32_t)__cvta_generic_to_shared(&bar);
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(b), "r"(1u));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t i = 0;
    bool done = false;
    for (; i < tries && !done; ++i) {
      uint32_t ok;
      asm volatile(
          "{\n\t.reg .pred p;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(ok)
          : "r"(b), "r"(0u)
          : "memory");
      done = ok != 0;
      if (!done && i > 64) __nanosleep(64);
    }
    if (!done) atomicOr(status, EB_DEV_WAIT_TIMEOUT);
    *polls_out = i;
  }
}

__global__ void l2_flush_kernel(uint4* p, size_t n16, uint32_t v) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n16; i += stride) p[i] = make_uint4(v, v, v, v);
}

template <int KIND>  // 0 bf16 normal, 1 f32 normal, 2 e4m3 normal, 3 f32 uniform
__global__ void synth_kernel(void* out, int64_t n, uint64_t seed, uint64_t sid, uint64_t idx0, float a, float b) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    if (KIND == 3) {
      ((float*)out)[i] = eb_uniform(seed, sid, idx0 + (uint64_t)i, a, b);
    } else {
      const float v = __fmul_rn(eb_normal(seed, sid, idx0 + (uint64_t)i), a);
      if (KIND == 0) ((uint16_t*)out)[i] = eb_bf16_from_f32(v);
      if (KIND == 1) ((float*)out)[i] = v;
      if (KIND == 2) ((uint8_t*)out)[i] = eb_f32_to_e4m3(v);
    }
  }
}

// One CTA per 128x128 block: generate, block amax, scale, quantise.  256 threads, thread t owns column
// pair-of-bytes positions; values are regenerated for the second pass instead of being held.
// `cols` columns starting at col0 of a tensor with cols_total columns; element index = row * cols_total + column.
__global__ void synth_weight_fp8_kernel(uint8_t* codes, float* scales, int64_t cols, int64_t row0, int64_t nrows,
                                        uint64_t seed, uint64_t sid, float std, int64_t cols_total, int64_t col0) {
  const int64_t cb = (cols + 127) / 128;
  const int64_t br = blockIdx.x / cb, bc = blockIdx.x % cb;
  const int64_t r_lo = br * 128, c_lo = bc * 128;
  const int r_n = (int)min((int64_t)128, nrows - r_lo), c_n = (int)min((int64_t)128, cols - c_lo);
  __shared__ float red[8];
  float amax = 0.f;
  for (int e = threadIdx.x; e < r_n * c_n; e += blockDim.x) {
    const int r = e / c_n, c = e % c_n;
    const float v = __fmul_rn(eb_normal(seed, sid, (uint64_t)((row0 + r_lo + r) * cols_total + col0 + c_lo + c)), std);
    amax = fmaxf(amax, fabsf(v));
  }
  for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
  for (int w = 1; w < (int)(blockDim.x >> 5); ++w) amax = fmaxf(amax, red[w]);
  const float s = amax > 0.f ? __fdiv_rn(amax, 448.0f) : 1.0f;
  if (threadIdx.x == 0) scales[br * cb + bc] = s;
  for (int e = threadIdx.x; e < r_n * c_n; e += blockDim.x) {
    const int r = e / c_n, c = e % c_n;
    const float v = __fmul_rn(eb_normal(seed, sid, (uint64_t)((row0 + r_lo + r) * cols_total + col0 + c_lo + c)), std);
    codes[(r_lo + r) * cols + c_lo + c] = eb_f32_to_e4m3(__fdiv_rn(v, s));
  }
}

// The same quantiser on values read from memory: fp32 weights [nrows][ld] (cols used) -> e4m3 codes [nrows][cols] and one
// scale per 128x128 block.  One CTA per block, the arithmetic of synth_weight_fp8_kernel operation for operation.
__global__ void quant_weight_f32_kernel(const float* w, int64_t ld, int64_t nrows, int64_t cols, uint8_t* codes, float* scales) {
  const int64_t cb = (cols + 127) / 128;
  const int64_t br = blockIdx.x / cb, bc = blockIdx.x % cb;
  const int64_t r_lo = br * 128, c_lo = bc * 128;
  const int r_n = (int)min((int64_t)128, nrows - r_lo), c_n = (int)min((int64_t)128, cols - c_lo);
  __shared__ float red[8];
  float amax = 0.f;
  for (int e = threadIdx.x; e < r_n * c_n; e += blockDim.x) {
    const int r = e / c_n, c = e % c_n;
    amax = fmaxf(amax, fabsf(w[(r_lo + r) * ld + c_lo + c]));
  }
  for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
  for (int x = 1; x < (int)(blockDim.x >> 5); ++x) amax = fmaxf(amax, red[x]);
  const float s = amax > 0.f ? __fdiv_rn(amax, 448.0f) : 1.0f;
  if (threadIdx.x == 0) scales[br * cb + bc] = s;
  for (int e = threadIdx.x; e < r_n * c_n; e += blockDim.x) {
    const int r = e / c_n, c = e % c_n;
    codes[(r_lo + r) * cols + c_lo + c] = eb_f32_to_e4m3(__fdiv_rn(w[(r_lo + r) * ld + c_lo + c], s));
  }
}

__global__ void f32_to_bf16_kernel(const float* in, uint16_t* out, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) out[i] = eb_bf16_from_f32(in[i]);
}

// Local KV heads [head0, head0 + n_local) of a cache whose global layout is [pages][2][n_total][page][dim]:
// element i of the local cache takes the value of its global index, so every rank fills the same global tensor.
__global__ void synth_kv_heads_kernel(uint16_t* out, int64_t n, int n_total, int head0, int n_local, int head_elems,
                                      uint64_t seed, uint64_t sid) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    const int64_t e = i % head_elems;
    const int64_t h = (i / head_elems) % n_local;
    const int64_t pk = i / ((int64_t)head_elems * n_local);  // page * 2 + (K or V)
    const uint64_t g = (uint64_t)((pk * n_total + head0 + h) * head_elems + e);
    out[i] = eb_bf16_from_f32(eb_normal(seed, sid, g));
  }
}

template <int KIND>
int32_t launch_synth(void* d_out, int64_t n, uint64_t seed, uint64_t sid, uint64_t idx0, float a, float b, void* st) {
  EB_REQUIRE(d_out && n >= 0, EB_ERR_ARG, "eb_synth: null or negative size");
  if (n == 0) return EB_OK;
  const int threads = 256;
  const int64_t blocks = std::min<int64_t>(eb::cdiv(n, threads), 148 * 32);
  synth_kernel<KIND><<<(unsigned)blocks, threads, 0, as_stream(st)>>>(d_out, n, seed, sid, idx0, a, b);
  EB_LAUNCH_CHECK();
  return EB_OK;
}

}  // namespace

extern "C" {

int32_t eb_selftest_wait_expires(uint32_t tries, uint32_t* h_polls) {
  EB_REQUIRE(tries >= 1 && tries <= (1u << 20), EB_ERR_ARG, "eb_selftest_wait_expires: %u polls outside 1..2^20", tries);
  int32_t* status = eb::status_word();
  EB_REQUIRE(status, EB_ERR_NODEVICE, "eb_selftest_wait_expires: no device");
  uint32_t* d_polls = nullptr;
  EB_CUDA(cudaMalloc(&d_polls, sizeof(uint32_t)));
  wait_expires_kernel<<<1, 32>>>(tries, status, d_polls);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  uint32_t polls = 0;
  if (e == cudaSuccess) e = cudaMemcpy(&polls, d_polls, sizeof(uint32_t), cudaMemcpyDeviceToHost);
  cudaFree(d_polls);
  if (e != cudaSuccess) return eb::fail((int32_t)e, "eb_selftest_wait_expires: %s", cudaGetErrorString(e));
  if (h_polls) *h_polls = polls;
  return EB_OK;
}

int32_t eb_l2_flush(void* d_scratch, size_t bytes, void* stream) {
  EB_REQUIRE(d_scratch && bytes >= 16, EB_ERR_ARG, "eb_l2_flush: null or too small");
  static uint32_t v = 0;
  l2_flush_kernel<<<148 * 8, 256, 0, as_stream(stream)>>>((uint4*)d_scratch, bytes / 16, ++v);
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_synth_normal_bf16(void* d_out, int64_t n, uint64_t seed, uint64_t sid, uint64_t idx0, float scale,
                             void* stream) {
  return launch_synth<0>(d_out, n, seed, sid, idx0, scale, 0.f, stream);
}
int32_t eb_synth_normal_f32(void* d_out, int64_t n, uint64_t seed, uint64_t sid, uint64_t idx0, float scale,
                            void* stream) {
  return launch_synth<1>(d_out, n, seed, sid, idx0, scale, 0.f, stream);
}
int32_t eb_synth_normal_e4m3(void* d_out, int64_t n, uint64_t seed, uint64_t sid, uint64_t idx0, float scale,
                             void* stream) {
  return launch_synth<2>(d_out, n, seed, sid, idx0, scale, 0.f, stream);
}
int32_t eb_synth_uniform_f32(void* d_out, int64_t n, uint64_t seed, uint64_t sid, uint64_t idx0, float lo, float hi,
                             void* stream) {
  return launch_synth<3>(d_out, n, seed, sid, idx0, lo, hi, stream);
}

int32_t eb_synth_weight_fp8(void* d_codes, void* d_scales, int64_t rows_total, int64_t cols, int64_t row0,
                            int64_t nrows, uint64_t seed, uint64_t sid, float std, void* stream) {
  EB_REQUIRE(d_codes && d_scales, EB_ERR_ARG, "eb_synth_weight_fp8: null");
  EB_REQUIRE(rows_total > 0 && cols > 0 && nrows > 0 && row0 >= 0 && row0 + nrows <= rows_total, EB_ERR_ARG,
             "eb_synth_weight_fp8: band [%lld,+%lld) outside %lld rows", (long long)row0, (long long)nrows,
             (long long)rows_total);
  EB_REQUIRE(row0 % 128 == 0, EB_ERR_ARG, "eb_synth_weight_fp8: row0 %lld not a multiple of 128", (long long)row0);
  const int64_t blocks = eb::cdiv(nrows, 128) * eb::cdiv(cols, 128);
  EB_REQUIRE(blocks < (1ll << 31), EB_ERR_ARG, "eb_synth_weight_fp8: too many blocks");
  synth_weight_fp8_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>((uint8_t*)d_codes, (float*)d_scales, cols,
                                                                           row0, nrows, seed, sid, std, cols, 0);
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_synth_weight_fp8_slice(void* d_codes, void* d_scales, int64_t rows_total, int64_t cols_total, int64_t row0,
                                  int64_t nrows, int64_t col0, int64_t ncols, uint64_t seed, uint64_t sid, float std,
                                  void* stream) {
  EB_REQUIRE(d_codes && d_scales, EB_ERR_ARG, "eb_synth_weight_fp8_slice: null");
  EB_REQUIRE(rows_total > 0 && cols_total > 0 && nrows > 0 && ncols > 0 && row0 >= 0 && col0 >= 0 &&
                 row0 + nrows <= rows_total && col0 + ncols <= cols_total,
             EB_ERR_ARG, "eb_synth_weight_fp8_slice: slice outside the tensor");
  EB_REQUIRE(row0 % 128 == 0 && col0 % 128 == 0, EB_ERR_ARG, "eb_synth_weight_fp8_slice: row0 and col0 must be multiples of 128");
  const int64_t blocks = eb::cdiv(nrows, 128) * eb::cdiv(ncols, 128);
  EB_REQUIRE(blocks < (1ll << 31), EB_ERR_ARG, "eb_synth_weight_fp8_slice: too many blocks");
  synth_weight_fp8_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>((uint8_t*)d_codes, (float*)d_scales, ncols,
                                                                           row0, nrows, seed, sid, std, cols_total, col0);
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_quant_weight_f32(const float* d_w, int64_t ld, int64_t nrows, int64_t cols, void* d_codes, void* d_scales, void* stream) {
  EB_REQUIRE(d_w && d_codes && d_scales && nrows > 0 && cols > 0 && ld >= cols, EB_ERR_ARG, "eb_quant_weight_f32: bad argument");
  const int64_t blocks = eb::cdiv(nrows, 128) * eb::cdiv(cols, 128);
  EB_REQUIRE(blocks < (1ll << 31), EB_ERR_ARG, "eb_quant_weight_f32: too many blocks");
  quant_weight_f32_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(d_w, ld, nrows, cols, (uint8_t*)d_codes, (float*)d_scales);
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_f32_to_bf16(const float* d_in, void* d_out, int64_t n, void* stream) {
  EB_REQUIRE(d_in && d_out && n >= 0, EB_ERR_ARG, "eb_f32_to_bf16: bad argument");
  if (n == 0) return EB_OK;
  const int64_t blocks = std::min<int64_t>(eb::cdiv(n, 256), 148 * 32);
  f32_to_bf16_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(d_in, (uint16_t*)d_out, n);
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_synth_kv_heads_bf16(void* d_cache, int64_t num_pages, int32_t n_kv_total, int32_t head0, int32_t n_kv_local,
                               int32_t page_size, int32_t head_dim, uint64_t seed, uint64_t sid, void* stream) {
  EB_REQUIRE(d_cache && num_pages >= 0 && n_kv_total >= 1 && head0 >= 0 && n_kv_local >= 1 &&
                 head0 + n_kv_local <= n_kv_total && page_size >= 1 && head_dim >= 1,
             EB_ERR_ARG, "eb_synth_kv_heads_bf16: bad argument");
  const int64_t n = num_pages * 2 * n_kv_local * page_size * head_dim;
  if (n == 0) return EB_OK;
  const int64_t blocks = std::min<int64_t>(eb::cdiv(n, 256), 148 * 32);
  synth_kv_heads_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>((uint16_t*)d_cache, n, n_kv_total, head0, n_kv_local,
                                                                         page_size * head_dim, seed, sid);
  EB_LAUNCH_CHECK();
  return EB_OK;
}

}  // extern "C"

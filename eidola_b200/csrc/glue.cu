// Per-token glue of the decode step: embedding gather, RMSNorm, rotary embedding, residual add, greedy argmax.
// All of it is [tokens x hidden] bf16 traffic, far below the weight and KV streams; the kernels are written for
// coalesced 16-byte accesses and few launches, not for arithmetic.
//
// The reference project has none of this (inference is delegated to `llama-server`,
// crates/eidola-app-core/src/local_models.rs:1612-1626).
#include <cuda_runtime.h>
#include <math.h>

#include <algorithm>

#include "common.h"

namespace {

__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Sum over a 256-thread CTA in a fixed order (an xor butterfly inside each warp, then the warps in ascending order), so
// that the CPU restatement can add the same numbers in the same order and RMSNorm is reproducible bit for bit.
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
  __syncthreads();
  return t;
}

// r = 1 / sqrt(ss / H + eps) with every operation rounded once (no contraction, no approximate reciprocal).
__device__ __forceinline__ float rms_scale(float ss, int H, float eps) {
  return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)H), eps)));
}
__device__ __forceinline__ float rms_apply(float x, float r, float g) { return __fmul_rn(__fmul_rn(x, r), g); }

// One CTA per token row: y = bf16(x * rsqrt(mean(x^2) + eps) * g).  H is a multiple of 8.
// Summation order of the squares (shared with the fused kernels below and restated by the CPU checker): thread t of
// 256 owns the 8-column chunks t, t + 256, ... and adds their squares in ascending column order with fused
// multiply-adds; the 256 partial sums are combined by block_sum.
__global__ void __launch_bounds__(256) rmsnorm_kernel(const uint16_t* x, const float* g, int H, float eps, uint16_t* y) {
  eb::pdl_wait();  // programmatic dependent launch: the predecessor in the stream has completed
  eb::pdl_trigger();
  __shared__ float red[8];
  const uint16_t* xr = x + (int64_t)blockIdx.x * H;
  uint16_t* yr = y + (int64_t)blockIdx.x * H;
  float ss = 0.f;
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + c);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      ss = __fmaf_rn(bf_lo(w[k]), bf_lo(w[k]), ss);
      ss = __fmaf_rn(bf_hi(w[k]), bf_hi(w[k]), ss);
    }
  }
  ss = block_sum(ss, red);
  const float r = rms_scale(ss, H, eps);
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + c);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    const float4 g0 = *reinterpret_cast<const float4*>(g + c), g1 = *reinterpret_cast<const float4*>(g + c + 4);
    uint4 o;
    o.x = pack_bf16(rms_apply(bf_lo(w[0]), r, g0.x), rms_apply(bf_hi(w[0]), r, g0.y));
    o.y = pack_bf16(rms_apply(bf_lo(w[1]), r, g0.z), rms_apply(bf_hi(w[1]), r, g0.w));
    o.z = pack_bf16(rms_apply(bf_lo(w[2]), r, g1.x), rms_apply(bf_hi(w[2]), r, g1.y));
    o.w = pack_bf16(rms_apply(bf_lo(w[3]), r, g1.z), rms_apply(bf_hi(w[3]), r, g1.w));
    *reinterpret_cast<uint4*>(yr + c) = o;
  }
}

// Rotate-half rotary embedding in place: one thread per (token, head, pair i < D/2).
__global__ void rope_kernel(uint16_t* x, int64_t row_stride, int n_heads, int head_dim, const int32_t* positions, int T,
                            const float* cos_t, const float* sin_t, int max_pos, int32_t* status) {
  eb::pdl_wait();  // programmatic dependent launch: the predecessor in the stream has completed
  eb::pdl_trigger();
  const int half = head_dim >> 1;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)T * n_heads * half) return;
  const int i = (int)(idx % half);
  const int h = (int)((idx / half) % n_heads);
  const int t = (int)(idx / ((int64_t)half * n_heads));
  const int pos = positions[t];
  if (pos < 0 || pos >= max_pos) {
    atomicOr(status, EB_DEV_BAD_INDEX);
    return;
  }
  const float c = cos_t[(int64_t)pos * half + i], s = sin_t[(int64_t)pos * half + i];
  uint16_t* r = x + (int64_t)t * row_stride + (int64_t)h * head_dim;
  const float a = __uint_as_float((uint32_t)r[i] << 16), b = __uint_as_float((uint32_t)r[i + half] << 16);
  // the products are rounded separately (no contraction) so the result matches a host evaluation of a*c - b*s
  const float ra = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
  const float rb = __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s));
  r[i] = (uint16_t)(pack_bf16(ra, 0.f) & 0xFFFFu);
  r[i + half] = (uint16_t)(pack_bf16(rb, 0.f) & 0xFFFFu);
}

// x = bf16(x + y), 8 elements per thread.
__global__ void residual_add_kernel(uint4* x, const uint4* y, int64_t n8) {
  eb::pdl_wait();  // programmatic dependent launch: the predecessor in the stream has completed
  eb::pdl_trigger();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  uint4 a = x[i];
  const uint4 b = y[i];
  a.x = pack_bf16(bf_lo(a.x) + bf_lo(b.x), bf_hi(a.x) + bf_hi(b.x));
  a.y = pack_bf16(bf_lo(a.y) + bf_lo(b.y), bf_hi(a.y) + bf_hi(b.y));
  a.z = pack_bf16(bf_lo(a.z) + bf_lo(b.z), bf_hi(a.z) + bf_hi(b.z));
  a.w = pack_bf16(bf_lo(a.w) + bf_lo(b.w), bf_hi(a.w) + bf_hi(b.w));
  x[i] = a;
}

__global__ void embed_kernel(const uint4* table, int V, int H8, const int32_t* tokens, uint4* x, int32_t* status) {
  eb::pdl_wait();  // programmatic dependent launch: the predecessor in the stream has completed
  eb::pdl_trigger();
  const int t = blockIdx.x;
  int tok = tokens[t];
  if (tok < 0 || tok >= V) {
    if (threadIdx.x == 0) atomicOr(status, EB_DEV_BAD_INDEX);
    tok = 0;
  }
  for (int c = threadIdx.x; c < H8; c += blockDim.x) x[(int64_t)t * H8 + c] = table[(int64_t)tok * H8 + c];
}

// Greedy argmax over bf16 logits, one CTA per token; ties go to the lower id.  Also the top-1 minus top-2 margin.
// NaN logits are never chosen.  A row without any value above -inf (all NaN or -inf) yields token 0, inside the
// vocabulary, and raises EB_DEV_BAD_INDEX.
__global__ void __launch_bounds__(1024) argmax_kernel(const uint16_t* logits, int64_t V, int64_t ld, int32_t* tok, float* margin,
                                                      float* cand, int32_t v_off, int32_t* status) {
  eb::pdl_wait();  // programmatic dependent launch: the predecessor in the stream has completed
  eb::pdl_trigger();
  const uint16_t* r = logits + (int64_t)blockIdx.x * ld;
  float b1 = -INFINITY, b2 = -INFINITY;
  int64_t i1 = V;
  auto take = [&](float x, int64_t v) {  // ascending v within a thread: strict > keeps the lower id
    if (x > b1) {
      b2 = b1;
      b1 = x;
      i1 = v;
    } else if (x > b2) {
      b2 = x;
    }
  };
  if ((((uintptr_t)r) & 15) == 0) {
    const int64_t V8 = V >> 3;
    for (int64_t c = threadIdx.x; c < V8; c += blockDim.x) {
      const uint4 q = *reinterpret_cast<const uint4*>(r + c * 8);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        take(bf_lo(w[k]), c * 8 + 2 * k);
        take(bf_hi(w[k]), c * 8 + 2 * k + 1);
      }
    }
    for (int64_t v = V8 * 8 + threadIdx.x; v < V; v += blockDim.x) take(__uint_as_float((uint32_t)r[v] << 16), v);
  } else {
    for (int64_t v = threadIdx.x; v < V; v += blockDim.x) take(__uint_as_float((uint32_t)r[v] << 16), v);
  }
  __shared__ float s1[1024], s2[1024];
  __shared__ int64_t si[1024];
  s1[threadIdx.x] = b1;
  s2[threadIdx.x] = b2;
  si[threadIdx.x] = i1;
  __syncthreads();
  for (int o = blockDim.x >> 1; o; o >>= 1) {
    if ((int)threadIdx.x < o) {
      const float a1 = s1[threadIdx.x], a2 = s2[threadIdx.x], c1 = s1[threadIdx.x + o], c2 = s2[threadIdx.x + o];
      const int64_t ai = si[threadIdx.x], ci = si[threadIdx.x + o];
      if (c1 > a1 || (c1 == a1 && ci < ai)) {
        s1[threadIdx.x] = c1;
        si[threadIdx.x] = ci;
        s2[threadIdx.x] = fmaxf(a1, c2);
      } else {
        s2[threadIdx.x] = fmaxf(a2, c1);
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const bool none = si[0] >= V;  // no value above -inf in this row (or slice)
    const int32_t best = none ? 0 : (int32_t)si[0];
    if (cand) {  // a vocabulary slice: leave the candidate for the merge, which decides whether the whole row is empty
      float* c = cand + (int64_t)blockIdx.x * 4;
      c[0] = s1[0];
      c[1] = s2[0];
      c[2] = __int_as_float(best + v_off);
      c[3] = 0.f;
    } else {
      if (none) atomicOr(status, EB_DEV_BAD_INDEX);
      tok[blockIdx.x] = best;
      if (margin) margin[blockIdx.x] = s1[0] - s2[0];
    }
  }
}

// One thread per row: fold the slices' candidates in ascending id order.
__global__ void argmax_merge_kernel(const float* cand, int n_parts, int64_t part_stride, int T, int32_t* tok, float* margin,
                                    int32_t* status) {
  eb::pdl_wait();  // programmatic dependent launch: the predecessor in the stream has completed
  eb::pdl_trigger();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  float a1 = -INFINITY, a2 = -INFINITY;
  int32_t ai = 0x7fffffff;
  for (int r = 0; r < n_parts; ++r) {
    const float* c = cand + ((int64_t)r * part_stride + t) * 4;
    const float c1 = c[0], c2 = c[1];
    const int32_t ci = __float_as_int(c[2]);
    if (c1 > a1 || (c1 == a1 && ci < ai)) {
      a2 = fmaxf(a1, c2);
      a1 = c1;
      ai = ci;
    } else {
      a2 = fmaxf(a2, c1);
    }
  }
  if (!(a1 > -INFINITY)) {  // every slice was empty (all NaN or -inf): token 0, flagged, as eb_argmax does
    atomicOr(status, EB_DEV_BAD_INDEX);
    ai = 0;
  }
  tok[t] = ai;
  if (margin) margin[t] = a1 - a2;
}

}  // namespace

extern "C" {

int32_t eb_rmsnorm(const void* d_x, const float* d_g, int32_t T, int32_t H, float eps, void* d_y, void* stream) {
  EB_REQUIRE(d_x && d_g && d_y, EB_ERR_ARG, "eb_rmsnorm: null pointer");
  EB_REQUIRE(T >= 0 && H >= 8 && H % 8 == 0, EB_ERR_ARG, "eb_rmsnorm: H %d must be a positive multiple of 8", H);
  EB_REQUIRE(((uintptr_t)d_x % 16 == 0) && ((uintptr_t)d_y % 16 == 0) && ((uintptr_t)d_g % 16 == 0), EB_ERR_ARG,
             "eb_rmsnorm: 16-byte alignment");
  if (T == 0) return EB_OK;
  EB_CUDA(eb::launch(rmsnorm_kernel, dim3(T), dim3(256), 0, eb::as_stream(stream), (const uint16_t*)d_x, d_g, H, eps, (uint16_t*)d_y));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_rope_table(int32_t max_pos, int32_t head_dim, double theta, float* h_cos, float* h_sin) {
  EB_REQUIRE(h_cos && h_sin && max_pos >= 1 && head_dim >= 2 && head_dim % 2 == 0 && theta > 0, EB_ERR_ARG,
             "eb_rope_table: bad argument");
  const int half = head_dim / 2;
  for (int i = 0; i < half; ++i) {
    const double inv = pow(theta, -2.0 * (double)i / (double)head_dim);
    for (int p = 0; p < max_pos; ++p) {
      const double a = (double)p * inv;
      h_cos[(int64_t)p * half + i] = (float)cos(a);
      h_sin[(int64_t)p * half + i] = (float)sin(a);
    }
  }
  return EB_OK;
}

int32_t eb_rope(void* d_x, int64_t row_stride, int32_t n_heads, int32_t head_dim, const int32_t* d_positions, int32_t T,
                const float* d_cos, const float* d_sin, int32_t max_pos, void* stream) {
  EB_REQUIRE(d_x && d_positions && d_cos && d_sin, EB_ERR_ARG, "eb_rope: null pointer");
  EB_REQUIRE(T >= 0 && n_heads >= 1 && head_dim >= 2 && head_dim % 2 == 0 && max_pos >= 1 &&
                 row_stride >= (int64_t)n_heads * head_dim,
             EB_ERR_ARG, "eb_rope: bad size");
  if (T == 0) return EB_OK;
  int32_t* status = eb::status_word();
  EB_REQUIRE(status, EB_ERR_NODEVICE, "eb_rope: no device");
  const int64_t n = (int64_t)T * n_heads * (head_dim / 2);
  EB_CUDA(eb::launch(rope_kernel, dim3((unsigned)eb::cdiv(n, 256)), dim3(256), 0, eb::as_stream(stream), (uint16_t*)d_x, row_stride, n_heads, head_dim,
                                                                             d_positions, T, d_cos, d_sin, max_pos, status));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_residual_add(void* d_x, const void* d_y, int64_t n, void* stream) {
  EB_REQUIRE(d_x && d_y && n >= 0 && n % 8 == 0, EB_ERR_ARG, "eb_residual_add: n %lld must be a multiple of 8", (long long)n);
  EB_REQUIRE(((uintptr_t)d_x % 16 == 0) && ((uintptr_t)d_y % 16 == 0), EB_ERR_ARG, "eb_residual_add: 16-byte alignment");
  if (n == 0) return EB_OK;
  EB_CUDA(eb::launch(residual_add_kernel, dim3((unsigned)eb::cdiv(n / 8, 256)), dim3(256), 0, eb::as_stream(stream), (uint4*)d_x, (const uint4*)d_y, n / 8));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_embed(const void* d_table, int32_t V, int32_t H, const int32_t* d_tokens, int32_t T, void* d_x, void* stream) {
  EB_REQUIRE(d_table && d_tokens && d_x, EB_ERR_ARG, "eb_embed: null pointer");
  EB_REQUIRE(V >= 1 && H >= 8 && H % 8 == 0 && T >= 0, EB_ERR_ARG, "eb_embed: bad size");
  if (T == 0) return EB_OK;
  int32_t* status = eb::status_word();
  EB_REQUIRE(status, EB_ERR_NODEVICE, "eb_embed: no device");
  EB_CUDA(eb::launch(embed_kernel, dim3(T), dim3(128), 0, eb::as_stream(stream), (const uint4*)d_table, V, H / 8, d_tokens, (uint4*)d_x, status));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_argmax(const void* d_logits, int32_t T, int64_t V, int64_t ld, int32_t* d_tok, float* d_margin, void* stream) {
  EB_REQUIRE(d_logits && d_tok, EB_ERR_ARG, "eb_argmax: null pointer");
  EB_REQUIRE(T >= 0 && V >= 1 && ld >= V, EB_ERR_ARG, "eb_argmax: bad size");
  if (T == 0) return EB_OK;
  int32_t* status = eb::status_word();
  EB_REQUIRE(status, EB_ERR_NODEVICE, "eb_argmax: no device");
  EB_CUDA(eb::launch(argmax_kernel, dim3(T), dim3(1024), 0, eb::as_stream(stream), (const uint16_t*)d_logits, V, ld, d_tok, d_margin,
                     (float*)nullptr, 0, status));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_argmax_partial(const void* d_logits, int32_t T, int64_t V, int64_t ld, int32_t v_off, float* d_cand, void* stream) {
  EB_REQUIRE(d_logits && d_cand, EB_ERR_ARG, "eb_argmax_partial: null pointer");
  EB_REQUIRE(T >= 0 && V >= 1 && ld >= V && v_off >= 0, EB_ERR_ARG, "eb_argmax_partial: bad size");
  if (T == 0) return EB_OK;
  EB_CUDA(eb::launch(argmax_kernel, dim3(T), dim3(1024), 0, eb::as_stream(stream), (const uint16_t*)d_logits, V, ld, (int32_t*)nullptr,
                     (float*)nullptr, d_cand, v_off, (int32_t*)nullptr));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_argmax_merge(const float* d_cand, int32_t n_parts, int64_t part_stride, int32_t T, int32_t* d_tok, float* d_margin,
                        void* stream) {
  EB_REQUIRE(d_cand && d_tok, EB_ERR_ARG, "eb_argmax_merge: null pointer");
  EB_REQUIRE(n_parts >= 1 && T >= 0 && part_stride >= T, EB_ERR_ARG, "eb_argmax_merge: bad size");
  if (T == 0) return EB_OK;
  int32_t* status = eb::status_word();
  EB_REQUIRE(status, EB_ERR_NODEVICE, "eb_argmax_merge: no device");
  EB_CUDA(eb::launch(argmax_merge_kernel, dim3((unsigned)eb::cdiv(T, 128)), dim3(128), 0, eb::as_stream(stream), d_cand, n_parts,
                     part_stride, T, d_tok, d_margin, status));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Fused consumers of the dense GEMMs and of the expert combine (fewer, fatter launches per layer).

namespace {

__device__ __forceinline__ float sum_partials(const float* part, int splits, int64_t plane, int64_t idx) {
  float a = 0.f;
  for (int s = 0; s < splits; ++s) a += part[(int64_t)s * plane + idx];
  return a;
}
__device__ __forceinline__ float round_bf16(float v) { return __uint_as_float(pack_bf16(v, 0.f) << 16); }

// One thread per (token, head, 8 consecutive i < D/2): elements [i, i+8) and [i + D/2, i + D/2 + 8) of a q, k or v
// head, moved with 16-byte accesses.
__global__ void qkv_rope_append_kernel(const float* part, int splits, uint16_t* qkv, int T, int n_q, int n_kv, int head_dim,
                                       const int32_t* positions, const float* cos_t, const float* sin_t, int max_pos,
                                       uint16_t* cache, int num_pages, int page_size, const int32_t* block_tables,
                                       int bt_stride, const int32_t* tok_slot, int32_t* status, int N, int k_col0,
                                       int v_col0) {
  eb::pdl_wait();  // programmatic dependent launch: the predecessor in the stream has completed
  eb::pdl_trigger();
  const int half = head_dim >> 1;
  const int groups = half >> 3;  // threads per head
  const int n_heads = n_q + 2 * n_kv;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)T * n_heads * groups) return;
  const int i = (int)(idx % groups) * 8;
  const int h = (int)((idx / groups) % n_heads);
  const int t = (int)(idx / ((int64_t)groups * n_heads));
  const int pos = positions[t];
  if (pos < 0 || pos >= max_pos) {
    atomicOr(status, EB_DEV_BAD_INDEX);
    return;
  }
  // column of this head in the row: q heads first, then the K band and the V band (under tensor parallelism a band
  // may start before this rank's first head, when 128-row scale blocks of the weight straddle ranks)
  const int col = h < n_q ? h * head_dim : h < n_q + n_kv ? k_col0 + (h - n_q) * head_dim : v_col0 + (h - n_q - n_kv) * head_dim;
  const int64_t e0 = (int64_t)t * N + col + i;
  float a[8], b[8];
  if (splits > 1) {
#pragma unroll
    for (int k = 0; k < 8; ++k) a[k] = b[k] = 0.f;
    const int64_t plane = (int64_t)T * N;
    for (int s = 0; s < splits; ++s) {
      const float4* pa = reinterpret_cast<const float4*>(part + s * plane + e0);
      const float4* pb = reinterpret_cast<const float4*>(part + s * plane + e0 + half);
      const float4 a0 = pa[0], a1 = pa[1], b0 = pb[0], b1 = pb[1];
      a[0] += a0.x; a[1] += a0.y; a[2] += a0.z; a[3] += a0.w; a[4] += a1.x; a[5] += a1.y; a[6] += a1.z; a[7] += a1.w;
      b[0] += b0.x; b[1] += b0.y; b[2] += b0.z; b[3] += b0.w; b[4] += b1.x; b[5] += b1.y; b[6] += b1.z; b[7] += b1.w;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      a[k] = round_bf16(a[k]);
      b[k] = round_bf16(b[k]);
    }
  } else {
    const uint4 va = *reinterpret_cast<const uint4*>(qkv + e0), vb = *reinterpret_cast<const uint4*>(qkv + e0 + half);
    const uint32_t wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      a[2 * k] = bf_lo(wa[k]);
      a[2 * k + 1] = bf_hi(wa[k]);
      b[2 * k] = bf_lo(wb[k]);
      b[2 * k + 1] = bf_hi(wb[k]);
    }
  }
  if (h < n_q + n_kv) {  // q and k heads rotate
    const float4* pc = reinterpret_cast<const float4*>(cos_t + (int64_t)pos * half + i);
    const float4* ps = reinterpret_cast<const float4*>(sin_t + (int64_t)pos * half + i);
    const float4 c0 = pc[0], c1 = pc[1], s0 = ps[0], s1 = ps[1];
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float ra = __fsub_rn(__fmul_rn(a[k], c[k]), __fmul_rn(b[k], sn[k]));
      const float rb = __fadd_rn(__fmul_rn(b[k], c[k]), __fmul_rn(a[k], sn[k]));
      a[k] = ra;
      b[k] = rb;
    }
  }
  const uint4 oa = make_uint4(pack_bf16(a[0], a[1]), pack_bf16(a[2], a[3]), pack_bf16(a[4], a[5]), pack_bf16(a[6], a[7]));
  const uint4 ob = make_uint4(pack_bf16(b[0], b[1]), pack_bf16(b[2], b[3]), pack_bf16(b[4], b[5]), pack_bf16(b[6], b[7]));
  if (h < n_q) {
    *reinterpret_cast<uint4*>(qkv + e0) = oa;
    *reinterpret_cast<uint4*>(qkv + e0 + half) = ob;
    return;
  }
  const int kv = (h >= n_q + n_kv) ? 1 : 0;
  const int hk = h - n_q - kv * n_kv;
  const int32_t page = block_tables[(int64_t)tok_slot[t] * bt_stride + pos / page_size];
  if (page < 0 || page >= num_pages) {
    atomicOr(status, EB_DEV_BAD_INDEX);
    return;
  }
  uint16_t* dst = cache + ((((int64_t)page * 2 + kv) * n_kv + hk) * page_size + pos % page_size) * head_dim;
  *reinterpret_cast<uint4*>(dst + i) = oa;
  *reinterpret_cast<uint4*>(dst + i + half) = ob;
}

// One CTA per token row; a thread owns chunks of 8 consecutive columns (16-byte accesses), at most two (H <= 4096):
//   MODE 0: v = bf16(sum of split-K partials) or the bf16 GEMM output    (O projection)
//   MODE 1: v = bf16(sum_j w_j * y[perm_row_j])                          (expert combine)
// then x = bf16(x + v), h = bf16(x * rsqrt(mean(x^2) + eps) * g).
template <int MODE>
__global__ void __launch_bounds__(256)
row_residual_rmsnorm_kernel(const float* part, int splits, const uint16_t* o_bf16, const uint16_t* y, const int32_t* perm_row,
                            const float* wts, int top_k, int64_t n_rows, uint16_t* x, const float* g, int T, int H, float eps,
                            uint16_t* hout, int64_t plane_stride, int planes_bf16, const eb::PeerWait pw) {
  eb::pdl_wait();  // programmatic dependent launch: the predecessor in the stream has completed
  eb::pdl_trigger();
  eb::peer_wait_cta(pw);  // planes pushed by the peers: wait for their flags here instead of behind a wait launch
  __shared__ float red[8];
  const int t = blockIdx.x;
  const int H8 = H >> 3;
  float xv[2][8];
  float ss = 0.f;
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    const int ch = threadIdx.x + 256 * q;
    if (ch >= H8) continue;
    const int64_t e = (int64_t)t * H + ch * 8;
    float v[8];
    if (MODE == 0) {
      if (planes_bf16) {  // `splits` bf16 planes (one per rank), added in plane order in fp32 and rounded once
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = 0.f;
        for (int s = 0; s < splits; ++s) {
          const uint4 pv = *reinterpret_cast<const uint4*>(o_bf16 + s * plane_stride + e);
          const uint32_t w[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            v[2 * k] += bf_lo(w[k]);
            v[2 * k + 1] += bf_hi(w[k]);
          }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = round_bf16(v[k]);
      } else if (part) {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = 0.f;
        const int64_t plane = plane_stride ? plane_stride : (int64_t)T * H;
        for (int s = 0; s < splits; ++s) {
          const float4* pp = reinterpret_cast<const float4*>(part + s * plane + e);
          const float4 p0 = pp[0], p1 = pp[1];
          v[0] += p0.x; v[1] += p0.y; v[2] += p0.z; v[3] += p0.w; v[4] += p1.x; v[5] += p1.y; v[6] += p1.z; v[7] += p1.w;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = round_bf16(v[k]);
      } else {
        const uint4 ov = *reinterpret_cast<const uint4*>(o_bf16 + e);
        const uint32_t w[4] = {ov.x, ov.y, ov.z, ov.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          v[2 * k] = bf_lo(w[k]);
          v[2 * k + 1] = bf_hi(w[k]);
        }
      }
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = 0.f;
      for (int j = 0; j < top_k; ++j) {
        const int r = perm_row[(int64_t)t * top_k + j];
        if (r < 0 || r >= n_rows) continue;
        const float wj = wts[(int64_t)t * top_k + j];
        const uint4 yv = *reinterpret_cast<const uint4*>(y + (int64_t)r * H + ch * 8);
        const uint32_t w[4] = {yv.x, yv.y, yv.z, yv.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          v[2 * k] = __fmaf_rn(wj, bf_lo(w[k]), v[2 * k]);
          v[2 * k + 1] = __fmaf_rn(wj, bf_hi(w[k]), v[2 * k + 1]);
        }
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = round_bf16(v[k]);
    }
    const uint4 xin = *reinterpret_cast<const uint4*>(x + e);
    const uint32_t xw[4] = {xin.x, xin.y, xin.z, xin.w};
    uint32_t xo[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      xo[k] = pack_bf16(__fadd_rn(bf_lo(xw[k]), v[2 * k]), __fadd_rn(bf_hi(xw[k]), v[2 * k + 1]));
      xv[q][2 * k] = bf_lo(xo[k]);
      xv[q][2 * k + 1] = bf_hi(xo[k]);
      ss = __fmaf_rn(xv[q][2 * k], xv[q][2 * k], ss);
      ss = __fmaf_rn(xv[q][2 * k + 1], xv[q][2 * k + 1], ss);
    }
    *reinterpret_cast<uint4*>(x + e) = make_uint4(xo[0], xo[1], xo[2], xo[3]);
  }
  ss = block_sum(ss, red);
  const float r = rms_scale(ss, H, eps);
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    const int ch = threadIdx.x + 256 * q;
    if (ch >= H8) continue;
    const float4 g0 = *reinterpret_cast<const float4*>(g + ch * 8), g1 = *reinterpret_cast<const float4*>(g + ch * 8 + 4);
    uint4 o;
    o.x = pack_bf16(rms_apply(xv[q][0], r, g0.x), rms_apply(xv[q][1], r, g0.y));
    o.y = pack_bf16(rms_apply(xv[q][2], r, g0.z), rms_apply(xv[q][3], r, g0.w));
    o.z = pack_bf16(rms_apply(xv[q][4], r, g1.x), rms_apply(xv[q][5], r, g1.y));
    o.w = pack_bf16(rms_apply(xv[q][6], r, g1.z), rms_apply(xv[q][7], r, g1.w));
    *reinterpret_cast<uint4*>(hout + (int64_t)t * H + ch * 8) = o;
  }
}

}  // namespace

extern "C" {

int32_t eb_qkv_rope_append(const float* d_part, int32_t splits, void* d_qkv, int32_t T, int32_t n_q, int32_t n_kv,
                           int32_t head_dim, const int32_t* d_positions, const float* d_cos, const float* d_sin,
                           int32_t max_pos, void* d_cache, int32_t num_pages, int32_t page_size,
                           const int32_t* d_block_tables, int32_t bt_stride, const int32_t* d_tok_slot, void* stream) {
  EB_REQUIRE(d_qkv && d_positions && d_cos && d_sin && d_cache && d_block_tables && d_tok_slot, EB_ERR_ARG,
             "eb_qkv_rope_append: null pointer");
  EB_REQUIRE(splits >= 1 && (splits == 1 || d_part), EB_ERR_ARG, "eb_qkv_rope_append: splits %d without partials", splits);
  EB_REQUIRE(T >= 0 && n_q >= 1 && n_kv >= 1 && head_dim >= 16 && head_dim % 16 == 0 && max_pos >= 1 && num_pages >= 1 &&
                 page_size >= 1 && bt_stride >= 1,
             EB_ERR_ARG, "eb_qkv_rope_append: bad size (head_dim must be a multiple of 16)");
  EB_REQUIRE(((uintptr_t)d_qkv % 16 == 0) && ((uintptr_t)d_cache % 16 == 0) && ((uintptr_t)d_cos % 16 == 0) &&
                 ((uintptr_t)d_sin % 16 == 0) && ((uintptr_t)d_part % 16 == 0),
             EB_ERR_ARG, "eb_qkv_rope_append: 16-byte alignment");
  if (T == 0) return EB_OK;
  int32_t* status = eb::status_word();
  EB_REQUIRE(status, EB_ERR_NODEVICE, "eb_qkv_rope_append: no device");
  const int64_t n = (int64_t)T * (n_q + 2 * n_kv) * (head_dim / 16);
  EB_CUDA(eb::launch(qkv_rope_append_kernel, dim3((unsigned)eb::cdiv(n, 256)), dim3(256), 0, eb::as_stream(stream), 
      d_part, splits, (uint16_t*)d_qkv, T, n_q, n_kv, head_dim, d_positions, d_cos, d_sin, max_pos, (uint16_t*)d_cache,
      num_pages, page_size, d_block_tables, bt_stride, d_tok_slot, status, (n_q + 2 * n_kv) * head_dim, n_q * head_dim,
      (n_q + n_kv) * head_dim));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_oproj_residual_rmsnorm(const float* d_part, int32_t splits, const void* d_o_bf16, void* d_x, const float* d_g,
                                  int32_t T, int32_t H, float eps, void* d_h, void* stream) {
  EB_REQUIRE(d_x && d_g && d_h, EB_ERR_ARG, "eb_oproj_residual_rmsnorm: null pointer");
  EB_REQUIRE(splits >= 1 && (d_part || (splits == 1 && d_o_bf16)), EB_ERR_ARG,
             "eb_oproj_residual_rmsnorm: splits %d without its input", splits);
  EB_REQUIRE(T >= 0 && H >= 8 && H % 8 == 0 && H <= 4096, EB_ERR_UNSUPPORTED, "eb_oproj_residual_rmsnorm: H %d (multiple of 8, <= 4096)", H);
  if (T == 0) return EB_OK;
  if (splits > 1 && !d_part) return eb::fail(EB_ERR_ARG, "eb_oproj_residual_rmsnorm: partials missing");
  EB_CUDA(eb::launch(row_residual_rmsnorm_kernel<0>, dim3(T), dim3(256), 0, eb::as_stream(stream), d_part, splits, (const uint16_t*)d_o_bf16, nullptr,
                                                                       nullptr, nullptr, 0, 0, (uint16_t*)d_x, d_g, T, H, eps,
                                                                       (uint16_t*)d_h, (int64_t)0, 0, eb::PeerWait{}));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_planes_residual_rmsnorm(const void* d_planes, int32_t planes_are_bf16, int32_t n_planes, int64_t plane_stride, void* d_x,
                                   const float* d_g, int32_t T, int32_t H, float eps, void* d_h, void* stream) {
  return eb_planes_residual_rmsnorm_after(nullptr, 0, 1, d_planes, planes_are_bf16, n_planes, plane_stride, d_x, d_g, T, H, eps, d_h,
                                          stream);
}

int32_t eb_planes_residual_rmsnorm_after(eb_symm* s, int32_t seq, int32_t patience, const void* d_planes, int32_t planes_are_bf16,
                                         int32_t n_planes, int64_t plane_stride, void* d_x, const float* d_g, int32_t T, int32_t H,
                                         float eps, void* d_h, void* stream) {
  eb::PeerWait pw = {};
  if (s) {
    const int32_t rc = eb::symm_peer_wait(s, seq, patience, &pw);
    if (rc != EB_OK) return rc;
  }
  EB_REQUIRE(d_planes && d_x && d_g && d_h, EB_ERR_ARG, "eb_planes_residual_rmsnorm: null pointer");
  EB_REQUIRE(n_planes >= 1 && n_planes <= 64 && plane_stride >= (int64_t)T * H && plane_stride % 8 == 0, EB_ERR_ARG,
             "eb_planes_residual_rmsnorm: %d planes, stride %lld", n_planes, (long long)plane_stride);
  EB_REQUIRE(T >= 0 && H >= 8 && H % 8 == 0 && H <= 4096, EB_ERR_UNSUPPORTED, "eb_planes_residual_rmsnorm: H %d (multiple of 8, <= 4096)", H);
  if (T == 0) return EB_OK;
  EB_CUDA(eb::launch(row_residual_rmsnorm_kernel<0>, dim3(T), dim3(256), 0, eb::as_stream(stream),
                     planes_are_bf16 ? (const float*)nullptr : (const float*)d_planes, n_planes,
                     planes_are_bf16 ? (const uint16_t*)d_planes : (const uint16_t*)nullptr, (const uint16_t*)nullptr, (const int32_t*)nullptr,
                     (const float*)nullptr, 0, (int64_t)0, (uint16_t*)d_x, d_g, T, H, eps, (uint16_t*)d_h, plane_stride,
                     planes_are_bf16 ? 1 : 0, pw));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_moe_combine_rmsnorm(const void* d_y, const int32_t* d_perm_row, const float* d_wts, int32_t T, int32_t top_k,
                               int32_t H, void* d_x, const float* d_g, float eps, void* d_h, void* stream) {
  return eb_moe_combine_rmsnorm_ex(d_y, d_perm_row, d_wts, T, top_k, H, (int64_t)T * top_k, d_x, d_g, eps, d_h, stream);
}

int32_t eb_moe_combine_rmsnorm_ex(const void* d_y, const int32_t* d_perm_row, const float* d_wts, int32_t T, int32_t top_k,
                                  int32_t H, int64_t n_rows, void* d_x, const float* d_g, float eps, void* d_h, void* stream) {
  EB_REQUIRE(d_y && d_perm_row && d_wts && d_x && d_g && d_h && n_rows >= 0, EB_ERR_ARG, "eb_moe_combine_rmsnorm: null pointer");
  EB_REQUIRE(T >= 0 && top_k >= 1 && H >= 8 && H % 8 == 0 && H <= 4096, EB_ERR_UNSUPPORTED, "eb_moe_combine_rmsnorm: H %d (multiple of 8, <= 4096)", H);
  if (T == 0) return EB_OK;
  EB_CUDA(eb::launch(row_residual_rmsnorm_kernel<1>, dim3(T), dim3(256), 0, eb::as_stream(stream), nullptr, 1, nullptr, (const uint16_t*)d_y, d_perm_row,
                                                                       d_wts, top_k, n_rows, (uint16_t*)d_x, d_g, T,
                                                                       H, eps, (uint16_t*)d_h, (int64_t)0, 0, eb::PeerWait{}));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Tensor-/expert-parallel helpers: fp32 buffers that an all-reduce sums across ranks.

namespace {

// out == nullptr: the sum goes straight into every rank's plane of a whole-batch exchange (pp), and the launch raises the
// collective's flags itself.
__global__ void sum_planes_kernel(const float4* part, int splits, int64_t n4, float4* out, const eb::PeerPlanes pp) {
  eb::pdl_wait();
  eb::pdl_trigger();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n4) {
    float4 a = part[i];
    for (int s = 1; s < splits; ++s) {
      const float4 b = part[(int64_t)s * n4 + i];
      a.x += b.x;
      a.y += b.y;
      a.z += b.z;
      a.w += b.w;
    }
    if (out) {
      out[i] = a;
    } else {
      for (int p = 0; p < pp.size; ++p) reinterpret_cast<float4*>(pp.dst[p])[i] = a;
    }
  }
  if (!out) eb::peer_arrive_cta(pp);
}

__global__ void bf16_to_f32_kernel(const uint16_t* in, int64_t n, float* out) {
  eb::pdl_wait();
  eb::pdl_trigger();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __uint_as_float((uint32_t)in[i] << 16);
}

}  // namespace

extern "C" {

int32_t eb_qkv_rope_append_ex(const float* d_part, int32_t splits, void* d_qkv, int32_t row_elems, int32_t k_col0,
                              int32_t v_col0, int32_t T, int32_t n_q, int32_t n_kv, int32_t head_dim,
                              const int32_t* d_positions, const float* d_cos, const float* d_sin, int32_t max_pos,
                              void* d_cache, int32_t num_pages, int32_t page_size, const int32_t* d_block_tables,
                              int32_t bt_stride, const int32_t* d_tok_slot, void* stream) {
  EB_REQUIRE(d_qkv && d_positions && d_cos && d_sin && d_cache && d_block_tables && d_tok_slot, EB_ERR_ARG,
             "eb_qkv_rope_append_ex: null pointer");
  EB_REQUIRE(splits >= 1 && (splits == 1 || d_part), EB_ERR_ARG, "eb_qkv_rope_append_ex: splits %d without partials", splits);
  EB_REQUIRE(T >= 0 && n_q >= 1 && n_kv >= 1 && head_dim >= 16 && head_dim % 16 == 0 && max_pos >= 1 && num_pages >= 1 &&
                 page_size >= 1 && bt_stride >= 1,
             EB_ERR_ARG, "eb_qkv_rope_append_ex: bad size (head_dim must be a multiple of 16)");
  EB_REQUIRE(k_col0 >= n_q * head_dim && v_col0 >= k_col0 + n_kv * head_dim && v_col0 + n_kv * head_dim <= row_elems &&
                 k_col0 % 8 == 0 && v_col0 % 8 == 0 && row_elems % 8 == 0,
             EB_ERR_ARG, "eb_qkv_rope_append_ex: K/V bands at %d/%d do not fit a row of %d", k_col0, v_col0, row_elems);
  EB_REQUIRE(((uintptr_t)d_qkv % 16 == 0) && ((uintptr_t)d_cache % 16 == 0) && ((uintptr_t)d_cos % 16 == 0) &&
                 ((uintptr_t)d_sin % 16 == 0) && ((uintptr_t)d_part % 16 == 0),
             EB_ERR_ARG, "eb_qkv_rope_append_ex: 16-byte alignment");
  if (T == 0) return EB_OK;
  int32_t* status = eb::status_word();
  EB_REQUIRE(status, EB_ERR_NODEVICE, "eb_qkv_rope_append_ex: no device");
  const int64_t n = (int64_t)T * (n_q + 2 * n_kv) * (head_dim / 16);
  EB_CUDA(eb::launch(qkv_rope_append_kernel, dim3((unsigned)eb::cdiv(n, 256)), dim3(256), 0, eb::as_stream(stream), d_part,
                     splits, (uint16_t*)d_qkv, T, n_q, n_kv, head_dim, d_positions, d_cos, d_sin, max_pos, (uint16_t*)d_cache,
                     num_pages, page_size, d_block_tables, bt_stride, d_tok_slot, status, row_elems, k_col0, v_col0));
  return EB_OK;
}

int32_t eb_sum_planes_f32(const float* d_part, int32_t splits, const void* d_bf16, int64_t n, float* d_out, void* stream) {
  EB_REQUIRE(d_out && n >= 0 && n % 4 == 0 && splits >= 1 && (d_part || (splits == 1 && d_bf16)), EB_ERR_ARG,
             "eb_sum_planes_f32: bad argument");
  if (n == 0) return EB_OK;
  if (d_part)
    EB_CUDA(eb::launch(sum_planes_kernel, dim3((unsigned)eb::cdiv(n / 4, 256)), dim3(256), 0, eb::as_stream(stream),
                       (const float4*)d_part, splits, n / 4, (float4*)d_out, eb::PeerPlanes{}));
  else
    EB_CUDA(eb::launch(bf16_to_f32_kernel, dim3((unsigned)eb::cdiv(n, 256)), dim3(256), 0, eb::as_stream(stream),
                       (const uint16_t*)d_bf16, n, d_out));
  return EB_OK;
}


int32_t eb_sum_planes_f32_to_peers(eb_symm* s, int64_t dst_off, int64_t plane_step, const float* d_part, int32_t splits, int64_t n,
                                   int32_t* seq, void* stream) {
  EB_REQUIRE(s && d_part && seq && splits >= 1 && n >= 0 && n % 4 == 0 && ((uintptr_t)d_part % 16 == 0), EB_ERR_ARG,
             "eb_sum_planes_f32_to_peers: bad argument");
  eb::PeerPlanes pp;
  const int32_t rc = eb::symm_peer_planes(s, dst_off, plane_step, n * (int64_t)sizeof(float), &pp, seq);
  if (rc != EB_OK) return rc;
  const unsigned grid = (unsigned)std::max<int64_t>(1, eb::cdiv(n / 4, 256));
  EB_CUDA(eb::launch(sum_planes_kernel, dim3(grid), dim3(256), 0, eb::as_stream(stream), (const float4*)d_part, splits, n / 4,
                     (float4*)nullptr, pp));
  return EB_OK;
}

}  // extern "C"

// Per-token glue of the decode step: embedding gather, RMSNorm, rotary embedding, residual add, greedy argmax.
// All of it is [tokens x hidden] bf16 traffic, far below the weight and KV streams; the kernels are written for
// coalesced 16-byte accesses and few launches, not for arithmetic.
//
// The reference project has none of this (inference is delegated to `llama-server`,
// crates/eidola-app-core/src/local_models.rs:1612-1626).
#include <cuda_runtime.h>
#include <math.h>

#include "common.h"

namespace {

__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

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

// One CTA per token row: y = bf16(x * rsqrt(mean(x^2) + eps) * g).  H is a multiple of 8.
__global__ void __launch_bounds__(256) rmsnorm_kernel(const uint16_t* x, const float* g, int H, float eps, uint16_t* y) {
  __shared__ float red[8];
  const uint16_t* xr = x + (int64_t)blockIdx.x * H;
  uint16_t* yr = y + (int64_t)blockIdx.x * H;
  float ss = 0.f;
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + c);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) ss += bf_lo(w[k]) * bf_lo(w[k]) + bf_hi(w[k]) * bf_hi(w[k]);
  }
  ss = block_sum(ss, red);
  const float r = 1.0f / sqrtf(ss / (float)H + eps);
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + c);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    const float4 g0 = *reinterpret_cast<const float4*>(g + c), g1 = *reinterpret_cast<const float4*>(g + c + 4);
    uint4 o;
    o.x = pack_bf16(bf_lo(w[0]) * r * g0.x, bf_hi(w[0]) * r * g0.y);
    o.y = pack_bf16(bf_lo(w[1]) * r * g0.z, bf_hi(w[1]) * r * g0.w);
    o.z = pack_bf16(bf_lo(w[2]) * r * g1.x, bf_hi(w[2]) * r * g1.y);
    o.w = pack_bf16(bf_lo(w[3]) * r * g1.z, bf_hi(w[3]) * r * g1.w);
    *reinterpret_cast<uint4*>(yr + c) = o;
  }
}

// Rotate-half rotary embedding in place: one thread per (token, head, pair i < D/2).
__global__ void rope_kernel(uint16_t* x, int64_t row_stride, int n_heads, int head_dim, const int32_t* positions, int T,
                            const float* cos_t, const float* sin_t, int max_pos, int32_t* status) {
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
  const int t = blockIdx.x;
  int tok = tokens[t];
  if (tok < 0 || tok >= V) {
    if (threadIdx.x == 0) atomicOr(status, EB_DEV_BAD_INDEX);
    tok = 0;
  }
  for (int c = threadIdx.x; c < H8; c += blockDim.x) x[(int64_t)t * H8 + c] = table[(int64_t)tok * H8 + c];
}

// Greedy argmax over bf16 logits, one CTA per token; ties go to the lower id.  Also the top-1 minus top-2 margin.
__global__ void __launch_bounds__(1024) argmax_kernel(const uint16_t* logits, int64_t V, int64_t ld, int32_t* tok, float* margin) {
  const uint16_t* r = logits + (int64_t)blockIdx.x * ld;
  float b1 = -INFINITY, b2 = -INFINITY;
  int64_t i1 = V;
  for (int64_t v = threadIdx.x; v < V; v += blockDim.x) {
    const float x = __uint_as_float((uint32_t)r[v] << 16);
    if (x > b1) {  // ascending v within a thread: strict > keeps the lower id
      b2 = b1;
      b1 = x;
      i1 = v;
    } else if (x > b2) {
      b2 = x;
    }
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
    tok[blockIdx.x] = (int32_t)si[0];
    if (margin) margin[blockIdx.x] = s1[0] - s2[0];
  }
}

}  // namespace

extern "C" {

int32_t eb_rmsnorm(const void* d_x, const float* d_g, int32_t T, int32_t H, float eps, void* d_y, void* stream) {
  EB_REQUIRE(d_x && d_g && d_y, EB_ERR_ARG, "eb_rmsnorm: null pointer");
  EB_REQUIRE(T >= 0 && H >= 8 && H % 8 == 0, EB_ERR_ARG, "eb_rmsnorm: H %d must be a positive multiple of 8", H);
  EB_REQUIRE(((uintptr_t)d_x % 16 == 0) && ((uintptr_t)d_y % 16 == 0) && ((uintptr_t)d_g % 16 == 0), EB_ERR_ARG,
             "eb_rmsnorm: 16-byte alignment");
  if (T == 0) return EB_OK;
  rmsnorm_kernel<<<T, 256, 0, eb::as_stream(stream)>>>((const uint16_t*)d_x, d_g, H, eps, (uint16_t*)d_y);
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
  rope_kernel<<<(unsigned)eb::cdiv(n, 256), 256, 0, eb::as_stream(stream)>>>((uint16_t*)d_x, row_stride, n_heads, head_dim,
                                                                             d_positions, T, d_cos, d_sin, max_pos, status);
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_residual_add(void* d_x, const void* d_y, int64_t n, void* stream) {
  EB_REQUIRE(d_x && d_y && n >= 0 && n % 8 == 0, EB_ERR_ARG, "eb_residual_add: n %lld must be a multiple of 8", (long long)n);
  EB_REQUIRE(((uintptr_t)d_x % 16 == 0) && ((uintptr_t)d_y % 16 == 0), EB_ERR_ARG, "eb_residual_add: 16-byte alignment");
  if (n == 0) return EB_OK;
  residual_add_kernel<<<(unsigned)eb::cdiv(n / 8, 256), 256, 0, eb::as_stream(stream)>>>((uint4*)d_x, (const uint4*)d_y, n / 8);
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_embed(const void* d_table, int32_t V, int32_t H, const int32_t* d_tokens, int32_t T, void* d_x, void* stream) {
  EB_REQUIRE(d_table && d_tokens && d_x, EB_ERR_ARG, "eb_embed: null pointer");
  EB_REQUIRE(V >= 1 && H >= 8 && H % 8 == 0 && T >= 0, EB_ERR_ARG, "eb_embed: bad size");
  if (T == 0) return EB_OK;
  int32_t* status = eb::status_word();
  EB_REQUIRE(status, EB_ERR_NODEVICE, "eb_embed: no device");
  embed_kernel<<<T, 128, 0, eb::as_stream(stream)>>>((const uint4*)d_table, V, H / 8, d_tokens, (uint4*)d_x, status);
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_argmax(const void* d_logits, int32_t T, int64_t V, int64_t ld, int32_t* d_tok, float* d_margin, void* stream) {
  EB_REQUIRE(d_logits && d_tok, EB_ERR_ARG, "eb_argmax: null pointer");
  EB_REQUIRE(T >= 0 && V >= 1 && ld >= V, EB_ERR_ARG, "eb_argmax: bad size");
  if (T == 0) return EB_OK;
  argmax_kernel<<<T, 1024, 0, eb::as_stream(stream)>>>((const uint16_t*)d_logits, V, ld, d_tok, d_margin);
  EB_LAUNCH_CHECK();
  return EB_OK;
}

}  // extern "C"

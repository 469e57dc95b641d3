// Temperature / nucleus (top-p) sampling over bf16 logits: the step after the LM head for requests that carry
// `temperature` and `top_p` (the reference server's request type has both: crates/eidola-server/src/types.rs:24-30;
// the reference itself forwards them to a remote engine and holds no sampler).
//
// The result is a pure function of (logits row, scale, top_p, one 32-bit random number): everything after the
// per-token weight is integer arithmetic, so the order in which threads add things up cannot change the token, and a
// CPU restatement (oracle/sampler.py) reproduces it bit for bit.
//
//   weight     W_v = trunc(2^31 * 2^t), t = (x_v - max_x) * scale, scale = log2(e) / temperature (fp32, given by the
//              caller); 2^t = 2^floor(t) * P(t - floor(t)) with P the degree-8 Taylor polynomial of 2^f evaluated by
//              Horner in separately rounded fp32 multiplies and adds (no fused multiply-add: numpy has none);
//              t < -32 and NaN logits weigh nothing.  W_v is the softmax numerator to 2e-7 relative, cut off where a
//              token is 2^-31 times less likely than the likeliest.
//   nucleus    bf16 logits have 65536 possible values: key(x) orders them, and all logits with one key weigh the same.
//              Z = sum W; target = max(1, Z * top_p_q24 >> 24); thr = the largest key whose tail mass
//              sum{W_v : key_v >= thr} reaches target; the nucleus is every token with key >= thr (ties at the
//              threshold all belong), mass M.  The kernel COUNTS the row's logits per key in shared memory (the lower
//              and the upper half of the key space in turn, 32768 counters each) and multiplies count by weight once
//              per key that occurs; a scan over 32-key groups from the top finds thr.
//   draw       r = (M * rand32) >> 32; the token is the first v, in index order, whose running nucleus mass exceeds r.
//
// One CTA of 1024 threads per row; four passes over the row (max, the two counting passes, draw; a fifth when the
// threshold lies among the negative logits), which stays in L2 between them.  Rows whose scale is <= 0 are left alone (greedy rows keep the argmax token).
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/eidola_b200.h"
#include "common.h"

namespace {

constexpr int kThreads = 1024;

__device__ __forceinline__ uint32_t key_of(uint32_t bits) {  // ascending in the value the bf16 bits stand for
  return (bits & 0x8000u) ? (~bits & 0xFFFFu) : (bits | 0x8000u);
}
__device__ __forceinline__ bool is_nan_bf16(uint32_t bits) { return (bits & 0x7FFFu) > 0x7F80u; }

// trunc(2^31 * 2^t) for t <= 0, by separately rounded fp32 operations
__device__ __forceinline__ uint32_t weight_of(float x, float mx, float scale) {
  const float t = __fmul_rn(__fsub_rn(x, mx), scale);
  if (!(t >= -32.f)) return 0u;  // also NaN
  const float n = floorf(t);
  const float f = __fsub_rn(t, n);  // exact, in [0, 1)
  // ln2^k / k!, k = 8 .. 0
  float p = 1.3215486790e-6f;
  p = __fadd_rn(__fmul_rn(p, f), 1.5252733804e-5f);
  p = __fadd_rn(__fmul_rn(p, f), 1.5403530393e-4f);
  p = __fadd_rn(__fmul_rn(p, f), 1.3333558146e-3f);
  p = __fadd_rn(__fmul_rn(p, f), 9.6181291076e-3f);
  p = __fadd_rn(__fmul_rn(p, f), 5.5504108665e-2f);
  p = __fadd_rn(__fmul_rn(p, f), 2.4022650696e-1f);
  p = __fadd_rn(__fmul_rn(p, f), 6.9314718056e-1f);
  p = __fadd_rn(__fmul_rn(p, f), 1.0f);
  return (uint32_t)ldexpf(p, (int)n + 31);  // exact scaling, then truncation; at most 2^31
}

// Visits every element of the row once, the whole warp together (so that fn may use warp collectives):
// fn(index, bf16 bits, live).  Lane l of warp w takes the 8-element chunks w * 32 + l, + 1024, ...
template <typename F>
__device__ __forceinline__ void for_row(const uint16_t* r, int64_t V, bool vec, F fn) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (vec) {
    const int64_t V8 = V >> 3;
    for (int64_t c0 = (int64_t)warp * 32; c0 < V8; c0 += kThreads) {
      const int64_t c = c0 + lane;
      const bool live = c < V8;
      uint4 q = make_uint4(0, 0, 0, 0);
      if (live) q = *reinterpret_cast<const uint4*>(r + c * 8);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        fn(c * 8 + 2 * k, w[k] & 0xFFFFu, live);
        fn(c * 8 + 2 * k + 1, w[k] >> 16, live);
      }
    }
    for (int64_t v0 = V8 * 8 + (int64_t)warp * 32; v0 < V; v0 += kThreads) {
      const int64_t v = v0 + lane;
      fn(v, v < V ? (uint32_t)r[v] : 0u, v < V);
    }
  } else {
    for (int64_t v0 = (int64_t)warp * 32; v0 < V; v0 += kThreads) {
      const int64_t v = v0 + lane;
      fn(v, v < V ? (uint32_t)r[v] : 0u, v < V);
    }
  }
}

__device__ __forceinline__ uint32_t bits_of_key(uint32_t key) {  // inverse of key_of
  return (key & 0x8000u) ? (key & 0x7FFFu) : (~key & 0xFFFFu);
}

// One half of the key space (the 32768 keys with key >> 15 == half): count the row's logits per key with shared-memory
// adds of 1, then let thread t turn the counts of its 32 keys [32 t, 32 t + 32) into integer mass, count x W(key): a
// weight is computed once per KEY that occurs, not once per logit.  Returns the thread's mass.
__device__ __forceinline__ unsigned long long count_half(const uint16_t* r, int64_t V, bool vec, uint32_t half, uint32_t* cnt, float mx,
                                                         float sc) {
  for (int i = threadIdx.x; i < 32768; i += kThreads) cnt[i] = 0u;
  __syncthreads();
  for_row(r, V, vec, [&](int64_t, uint32_t b, bool live) {
    const uint32_t k = key_of(b);
    if (live && !is_nan_bf16(b) && (k >> 15) == half) atomicAdd(&cnt[k & 0x7FFFu], 1u);
  });
  __syncthreads();
  unsigned long long mass = 0;
#pragma unroll 4
  for (int i = 0; i < 32; ++i) {
    const uint32_t kk = threadIdx.x * 32 + i, c = cnt[kk];
    if (c) mass += (unsigned long long)c * weight_of(__uint_as_float(bits_of_key((half << 15) | kk) << 16), mx, sc);
  }
  return mass;
}

__global__ void __launch_bounds__(kThreads) sample_top_p_kernel(const uint16_t* logits, int64_t V, int64_t ld, const float* scale,
                                                                const uint32_t* top_p_q24, const uint32_t* rand32, int32_t* tok,
                                                                int32_t* status) {
  eb::pdl_wait();  // programmatic dependent launch: the predecessor in the stream has completed
  eb::pdl_trigger();
  const int row = blockIdx.x;
  const float sc = scale[row];
  if (!(sc > 0.f)) return;  // a greedy row
  const uint16_t* r = logits + (int64_t)row * ld;
  const bool vec = (((uintptr_t)r) & 15) == 0;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  extern __shared__ uint32_t s_cnt[];  // [32768] logits per key of the half being counted
  __shared__ float s_max[32];
  __shared__ unsigned long long s_gm[2 * kThreads];  // mass of 32-key groups, from the largest keys down; then the runs of the draw
  __shared__ unsigned long long s_above, s_target, s_r;
  __shared__ uint32_t s_thr;
  __shared__ int s_group;
  __shared__ float s_mx;

  // ---- pass 1: the row maximum (NaN never wins)
  float mx = -INFINITY;
  for_row(r, V, vec, [&](int64_t, uint32_t b, bool live) {
    if (live && !is_nan_bf16(b)) mx = fmaxf(mx, __uint_as_float(b << 16));
  });
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) s_max[warp] = mx;
  __syncthreads();
  if (warp == 0) {
    float m = s_max[lane];
#pragma unroll
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) s_mx = m;
  }
  __syncthreads();
  mx = s_mx;
  if (!(mx > -INFINITY) || mx == INFINITY) return;  // nothing to weigh (all -inf / NaN) or an infinite logit: the argmax token stays

  // ---- passes 2 and 3: integer mass per group of 32 keys; the lower half of the key space (negative logits) first,
  // so that the counts left in shared memory are those of the upper half, where the threshold usually lies.
  // Group g (0 = the largest keys) is thread 1023 - g of the upper half, then thread 2047 - g of the lower half.
  s_gm[2 * kThreads - 1 - tid] = count_half(r, V, vec, 0u, s_cnt, mx, sc);
  __syncthreads();
  s_gm[kThreads - 1 - tid] = count_half(r, V, vec, 1u, s_cnt, mx, sc);
  __syncthreads();
  // the total, the target, and the group in which the tail mass reaches it (warp 0: 64 groups per lane)
  if (warp == 0) {
    unsigned long long run = 0;
    for (int i = 0; i < 64; ++i) run += s_gm[lane * 64 + i];
    unsigned long long incl = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    const unsigned long long Z = __shfl_sync(0xffffffffu, incl, 31);
    const uint32_t q = top_p_q24[row];
    unsigned long long target = q >= (1u << 24) ? Z : __umul64hi(Z, (unsigned long long)q << 40);
    if (target < 1ull) target = 1ull;
    const unsigned long long before = incl - run;
    if (before < target && incl >= target) {  // exactly one lane (Z >= target >= 1)
      unsigned long long cum = before;
      int g = lane * 64;
      for (; g < lane * 64 + 63; ++g) {
        if (cum + s_gm[g] >= target) break;
        cum += s_gm[g];
      }
      s_group = g;
      s_above = cum;  // mass of the groups above the chosen one
      s_target = target;
    }
  }
  __syncthreads();
  const int group = s_group;
  if (group >= kThreads) {  // the threshold lies among the negative logits: their counts again
    (void)count_half(r, V, vec, 0u, s_cnt, mx, sc);
    __syncthreads();
  }
  if (tid == 0) {
    const uint32_t half = group < kThreads ? 1u : 0u;
    const uint32_t t_owner = (uint32_t)(group < kThreads ? kThreads - 1 - group : 2 * kThreads - 1 - group);
    unsigned long long cum = s_above;
    int i = 31;
    for (; i >= 0; --i) {
      const uint32_t kk = t_owner * 32 + (uint32_t)i, c = s_cnt[kk];
      if (c) cum += (unsigned long long)c * weight_of(__uint_as_float(bits_of_key((half << 15) | kk) << 16), mx, sc);
      if (cum >= s_target) break;
    }
    if (i < 0) i = 0;  // (cannot happen: the group's mass reaches the target)
    s_thr = (half << 15) | (t_owner * 32 + (uint32_t)i);  // the nucleus: every key >= thr, mass cum
    s_r = __umul64hi(cum, (unsigned long long)rand32[row] << 32);  // (M * rand32) >> 32 < M
  }
  __syncthreads();
  const uint32_t thr = s_thr;
  unsigned long long* s_part = s_gm;

  // ---- pass 4: the draw, in index order.  Thread t owns the contiguous run [t * per, (t + 1) * per).
  const int64_t per = ((V + kThreads - 1) / kThreads + 7) / 8 * 8;
  const int64_t v0 = (int64_t)tid * per, v1 = min(V, v0 + per);
  // (v0 is a multiple of 8: whole 16-byte chunks while they last, then the row's tail)
  auto for_run = [&](auto fn) {  // fn(index, bits) -> true to stop
    int64_t v = v0;
    if (vec) {
      for (; v + 8 <= v1; v += 8) {
        const uint4 q = *reinterpret_cast<const uint4*>(r + v);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (fn(v + 2 * k, w[k] & 0xFFFFu)) return;
          if (fn(v + 2 * k + 1, w[k] >> 16)) return;
        }
      }
    }
    for (; v < v1; ++v)
      if (fn(v, (uint32_t)r[v])) return;
  };
  unsigned long long mine = 0;
  for_run([&](int64_t, uint32_t b) {
    if (!is_nan_bf16(b) && key_of(b) >= thr) mine += weight_of(__uint_as_float(b << 16), mx, sc);
    return false;
  });
  s_part[tid] = mine;
  __syncthreads();
  if (warp == 0) {  // exclusive scan of the 1024 run sums: 32 per lane, then across the lanes
    unsigned long long run = 0;
    for (int i = 0; i < 32; ++i) run += s_part[lane * 32 + i];
    unsigned long long incl = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    unsigned long long base = incl - run;
    for (int i = 0; i < 32; ++i) {
      const unsigned long long p = s_part[lane * 32 + i];
      s_part[lane * 32 + i] = base;
      base += p;
    }
  }
  __syncthreads();
  const unsigned long long before = s_part[tid], want = s_r;
  if (mine > 0 && want >= before && want < before + mine) {  // exactly one thread
    unsigned long long cum = before;
    int64_t pick = -1;
    for_run([&](int64_t v, uint32_t b) {
      if (is_nan_bf16(b) || key_of(b) < thr) return false;
      cum += weight_of(__uint_as_float(b << 16), mx, sc);
      if (cum > want) {
        pick = v;
        return true;
      }
      return false;
    });
    if (pick < 0 || pick >= V) {
      atomicOr(status, EB_DEV_BAD_INDEX);
      pick = 0;
    }
    tok[row] = (int32_t)pick;
  }
}

constexpr size_t kSampleSmem = 32768 * sizeof(uint32_t);

}  // namespace

extern "C" {

uint32_t eb_sample_rand32(uint64_t seed, uint64_t counter) {
  uint64_t z = seed + 0x9E3779B97F4A7C15ull * (counter + 1);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return (uint32_t)(z >> 32);
}

int32_t eb_sample_top_p(const void* d_logits, int32_t T, int64_t V, int64_t ld, const float* d_scale, const uint32_t* d_top_p_q24,
                        const uint32_t* d_rand32, int32_t* d_tok, void* stream) {
  EB_REQUIRE(d_logits && d_scale && d_top_p_q24 && d_rand32 && d_tok, EB_ERR_ARG, "eb_sample_top_p: null pointer");
  EB_REQUIRE(T >= 0 && V >= 1 && ld >= V, EB_ERR_ARG, "eb_sample_top_p: T %d, V %lld, ld %lld", T, (long long)V, (long long)ld);
  EB_REQUIRE(V <= (int64_t)kThreads * 65536, EB_ERR_UNSUPPORTED, "eb_sample_top_p: vocabulary %lld", (long long)V);
  if (T == 0) return EB_OK;
  int32_t* status = eb::status_word();
  EB_REQUIRE(status, EB_ERR_NODEVICE, "eb_sample_top_p: no device");
  static std::mutex attr_mu;
  static bool attr_set[64] = {};  // the attribute is per device
  int dev = 0;
  EB_CUDA(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lk(attr_mu);
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
      EB_CUDA(cudaFuncSetAttribute(sample_top_p_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSampleSmem));
      if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
  }
  EB_CUDA(eb::launch(sample_top_p_kernel, dim3((unsigned)T), dim3(kThreads), kSampleSmem, eb::as_stream(stream), (const uint16_t*)d_logits, V, ld,
                     d_scale, d_top_p_q24, d_rand32, d_tok, status));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

}  // extern "C"

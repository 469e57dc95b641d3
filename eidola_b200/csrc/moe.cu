// Mixture-of-experts routing for the decode step: router logits + top-k, token -> expert permutation, and the
// weighted combine of expert outputs.  The expert matrices themselves run in the grouped FP8 GEMM (gemm.cu).
//
// Routing decisions must be bit-exact against the CPU restatement, so the router logit is summed in one fixed
// order: the row is cut in groups of 8 consecutive elements, lane l of a warp owns groups l, l+32, ... and adds
// their exact bf16 x bf16 products in ascending k with fmaf, then the 32 lane sums are combined by an xor
// butterfly (offsets 16, 8, 4, 2, 1).  Ties go to the lower expert.
//
// The reference project has no router (inference is delegated, crates/eidola-server/src/backend.rs:421-433).
#include <cuda_runtime.h>

#include <stdlib.h>

#include "common.h"

namespace {

constexpr int kMaxExperts = 256;
constexpr int kMaxTopK = 8;

__device__ __forceinline__ float bf(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }

// Top-k selection and softmax weights of one token, run by one warp: lane l holds the logits of experts l + 32 q.
template <int EPL>
__device__ __forceinline__ void router_select(float (&lg)[EPL], int lane, int E, int top_k, int64_t t, int32_t* idx, float* wts) {
  float sel[kMaxTopK];
  for (int j = 0; j < top_k; ++j) {
    // local best (lowest index on ties: ascending scan with strict >)
    float bv = -INFINITY;
    int bi = 0x7FFFFFFF;
#pragma unroll
    for (int q = 0; q < EPL; ++q) {
      const int e = lane + 32 * q;
      if (e < E && lg[q] > bv) {
        bv = lg[q];
        bi = e;
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    sel[j] = bv;
    if (lane == 0) idx[(int64_t)t * top_k + j] = bi;
    if ((bi & 31) == lane) {
#pragma unroll
      for (int q = 0; q < EPL; ++q)
        if (q == (bi >> 5)) lg[q] = -INFINITY;  // taken
    }
  }
  if (lane == 0) {
    float ex[kMaxTopK], den = 0.f;
    for (int j = 0; j < top_k; ++j) {
      ex[j] = expf(sel[j] - sel[0]);
      den += ex[j];
    }
    for (int j = 0; j < top_k; ++j) wts[(int64_t)t * top_k + j] = ex[j] / den;
  }
}

// Up to a few thousand tokens: one CTA per TPC tokens (1, 2, 4 or 8), the experts dealt to its eight warps, router rows
// read straight from L2 (every lane's loads are issued before any is used, so a pass over two experts costs about one
// memory round trip, and a row fetched once serves all the CTA's tokens: the router matrix crosses the L2 -> SM path
// T / TPC times, which is what bounds the kernel once T is in the hundreds).  With more than one token per CTA the
// token rows live in shared memory instead of registers.
// The dot products use exactly the order of router_topk_kernel (lane l owns 8-element groups l, l + 32, ...,
// ascending k, xor butterfly), so all router kernels produce the same bits.
template <int EPL, int GPL, int TPC>
__global__ void __launch_bounds__(256)
router_direct_kernel(const uint16_t* x, const uint16_t* wr, int T, int E, int H, int top_k, int32_t* idx, float* wts,
                     float* logits_out) {
  eb::pdl_wait();  // programmatic dependent launch: the predecessor in the stream has completed
  eb::pdl_trigger();
  __shared__ float s_lg[TPC][kMaxExperts];
  extern __shared__ __align__(16) uint16_t xs[];  // TPC > 1: the CTA's token rows, [TPC][H]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * TPC;
  const int H8 = H >> 3;
  constexpr bool XS = TPC > 1;  // several tokens per CTA keep their rows in shared memory, not in registers
  uint4 xp[XS ? 1 : TPC][GPL];  // the tokens' rows as packed bf16 pairs
  if (XS) {
    for (int i = threadIdx.x; i < TPC * H8; i += 256) {
      const int k = i / H8, g = i - k * H8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (t0 + k < T) v = *reinterpret_cast<const uint4*>(x + (int64_t)(t0 + k) * H + 8 * g);
      *reinterpret_cast<uint4*>(xs + (size_t)k * H + 8 * g) = v;
    }
    __syncthreads();
  } else {
#pragma unroll
    for (int k = 0; k < (XS ? 1 : TPC); ++k)
#pragma unroll
      for (int j = 0; j < GPL; ++j) {
        const int g = lane + 32 * j;
        xp[k][j] = make_uint4(0, 0, 0, 0);
        if (g < H8 && t0 + k < T) xp[k][j] = *reinterpret_cast<const uint4*>(x + (int64_t)(t0 + k) * H + 8 * g);
      }
  }
  for (int e = warp; e < E; e += 16) {  // two experts per pass: e and e + 8
    const bool two = e + 8 < E;
    const uint4* w0 = reinterpret_cast<const uint4*>(wr + (int64_t)e * H);
    const uint4* w1 = reinterpret_cast<const uint4*>(wr + (int64_t)(two ? e + 8 : e) * H);
    uint4 u0[GPL], u1[GPL];
#pragma unroll
    for (int j = 0; j < GPL; ++j) {
      const int g = lane + 32 * j;
      u0[j] = u1[j] = make_uint4(0, 0, 0, 0);
      if (g < H8) {
        u0[j] = w0[g];
        u1[j] = w1[g];
      }
    }
    float a0[TPC], a1[TPC];
#pragma unroll
    for (int k = 0; k < TPC; ++k) a0[k] = a1[k] = 0.f;
#pragma unroll
    for (int j = 0; j < GPL; ++j) {
      const int g = lane + 32 * j;
      if (g < H8) {
        const uint32_t p0[4] = {u0[j].x, u0[j].y, u0[j].z, u0[j].w}, p1[4] = {u1[j].x, u1[j].y, u1[j].z, u1[j].w};
#pragma unroll
        for (int k = 0; k < TPC; ++k) {
          const uint4 xv = XS ? *reinterpret_cast<const uint4*>(xs + (size_t)k * H + 8 * g) : xp[XS ? 0 : k][j];
          const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float xl = __uint_as_float(xw[q] << 16), xh = __uint_as_float(xw[q] & 0xFFFF0000u);
            a0[k] = __fmaf_rn(xl, __uint_as_float(p0[q] << 16), a0[k]);
            a0[k] = __fmaf_rn(xh, __uint_as_float(p0[q] & 0xFFFF0000u), a0[k]);
            a1[k] = __fmaf_rn(xl, __uint_as_float(p1[q] << 16), a1[k]);
            a1[k] = __fmaf_rn(xh, __uint_as_float(p1[q] & 0xFFFF0000u), a1[k]);
          }
        }
      }
    }
#pragma unroll
    for (int k = 0; k < TPC; ++k) {
#pragma unroll
      for (int o = 16; o; o >>= 1) {
        a0[k] = __fadd_rn(a0[k], __shfl_xor_sync(0xffffffffu, a0[k], o));
        a1[k] = __fadd_rn(a1[k], __shfl_xor_sync(0xffffffffu, a1[k], o));
      }
      if (lane == 0 && t0 + k < T) {
        s_lg[k][e] = a0[k];
        if (two) s_lg[k][e + 8] = a1[k];
        if (logits_out) {
          logits_out[(int64_t)(t0 + k) * E + e] = a0[k];
          if (two) logits_out[(int64_t)(t0 + k) * E + e + 8] = a1[k];
        }
      }
    }
  }
  __syncthreads();
  if (warp >= TPC || t0 + warp >= T) return;  // warp k finishes token t0 + k
  float lg[EPL];
#pragma unroll
  for (int q = 0; q < EPL; ++q) lg[q] = (lane + 32 * q < E) ? s_lg[warp][lane + 32 * q] : -INFINITY;
  router_select<EPL>(lg, lane, E, top_k, t0 + warp, idx, wts);
}

// One warp per token, eight tokens per CTA.  Lane l keeps its slice of the token row (x[k], k = l mod 32) in
// registers; the CTA streams the router matrix through shared memory eight expert rows at a time (double
// buffered: the next chunk's 16-byte loads are in flight while the current chunk is reduced), so every row is
// fetched once per CTA and the inner loop reads only shared memory.  Lane l keeps the logits of experts
// e = l + 32*j.
constexpr int kRouterChunk = 8;

template <int EPL, int GPL>  // experts per lane = ceil(E / 32), 8-element groups per lane = ceil(H / 256)
__global__ void __launch_bounds__(256, 2)
router_topk_kernel(const uint16_t* x, const uint16_t* wr, int T, int E, int H, int top_k, int32_t* idx, float* wts,
                   float* logits_out) {
  eb::pdl_wait();  // programmatic dependent launch: the predecessor in the stream has completed
  eb::pdl_trigger();
  extern __shared__ __align__(16) uint16_t wrow[];  // [2][kRouterChunk][H]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + warp;
  const bool on = t < T;
  const int H8 = H >> 3;  // groups of 8 elements = 16-byte words per row
  float xr[GPL][8];
#pragma unroll
  for (int j = 0; j < GPL; ++j) {
    const int g = lane + 32 * j;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (on && g < H8) v = *reinterpret_cast<const uint4*>(x + (int64_t)t * H + 8 * g);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      xr[j][2 * q] = __uint_as_float(w[q] << 16);
      xr[j][2 * q + 1] = __uint_as_float(w[q] & 0xFFFF0000u);
    }
  }
  // Rows [e0, e0 + chunk) are contiguous in the router matrix: copy them with 16-byte cp.async, no registers held.
  auto stage = [&](int e0, int buf) {
    const int n16 = min(kRouterChunk, E - e0) * H8;
    const uint4* src = reinterpret_cast<const uint4*>(wr + (int64_t)e0 * H);
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(wrow + (size_t)buf * kRouterChunk * H);
    for (int c = threadIdx.x; c < n16; c += 256)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + c * 16), "l"(src + c) : "memory");
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  stage(0, 0);
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();

  float lg[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) lg[j] = -INFINITY;
  for (int e0 = 0, buf = 0; e0 < E; e0 += kRouterChunk, buf ^= 1) {
    const bool more = e0 + kRouterChunk < E;
    if (more) stage(e0 + kRouterChunk, buf ^ 1);  // that buffer was last read one iteration ago, before a barrier
    const int ne = min(kRouterChunk, E - e0);
    for (int r0 = 0; r0 < ne; r0 += 2) {
      // two experts at a time (two independent fmaf chains); one 16-byte shared-memory load feeds eight fmaf
      const uint4* w0 = reinterpret_cast<const uint4*>(wrow + ((size_t)buf * kRouterChunk + r0) * H);
      const uint4* w1 = w0 + (r0 + 1 < ne ? H8 : 0);
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int j = 0; j < GPL; ++j) {
        const int g = lane + 32 * j;
        if (g < H8) {
          const uint4 u0 = w0[g], u1 = w1[g];
          const uint32_t p0[4] = {u0.x, u0.y, u0.z, u0.w}, p1[4] = {u1.x, u1.y, u1.z, u1.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            a0 = __fmaf_rn(xr[j][2 * q], __uint_as_float(p0[q] << 16), a0);
            a0 = __fmaf_rn(xr[j][2 * q + 1], __uint_as_float(p0[q] & 0xFFFF0000u), a0);
            a1 = __fmaf_rn(xr[j][2 * q], __uint_as_float(p1[q] << 16), a1);
            a1 = __fmaf_rn(xr[j][2 * q + 1], __uint_as_float(p1[q] & 0xFFFF0000u), a1);
          }
        }
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) {
        a0 = __fadd_rn(a0, __shfl_xor_sync(0xffffffffu, a0, o));
        a1 = __fadd_rn(a1, __shfl_xor_sync(0xffffffffu, a1, o));
      }
      const float av[2] = {a0, a1};
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int e = e0 + r0 + q;
        if (r0 + q >= ne) break;
        if ((e & 31) == lane) {
#pragma unroll
          for (int j = 0; j < EPL; ++j)
            if (j == (e >> 5)) lg[j] = av[q];
        }
        if (logits_out && on && lane == 0) logits_out[(int64_t)t * E + e] = av[q];
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
  }
  if (!on) return;

  router_select<EPL>(lg, lane, E, top_k, t, idx, wts);
}

// Stable counting sort of the T*top_k routed slots by expert, one CTA per expert (512 threads):
//   seg_off[E+1]  : expert segment bounds in the permuted row space
//   perm_row[i]   : permuted row of slot i = t*top_k + j   (order: expert, then slot index)
//   row_token[r]  : token whose activations permuted row r carries
// Every CTA counts all slots per expert (shared-memory histogram, then a prefix sum over the experts, so it knows where
// every segment starts without talking to the others) and then places the slots of ITS expert in slot order (ballot +
// prefix over the CTA, 512 slots per round).  CTA 0 also writes the segment bounds and the tile table.  The result is
// the one a sequential stable sort gives, whatever the number of CTAs.
constexpr int kPermThreads = 512;

__global__ void __launch_bounds__(kPermThreads)
moe_permute_kernel(const int32_t* idx, int n_slots, int top_k, int E, int32_t* seg_off, int32_t* perm_row,
                   int32_t* row_token, int tn, int max_tiles, int32_t* tile_ws, int32_t* status, int skip_foreign) {
  eb::pdl_wait();  // programmatic dependent launch: the predecessor in the stream has completed
  eb::pdl_trigger();
  __shared__ int32_t base[kMaxExperts + 1];  // counts, then exclusive prefix sums: start of each expert's segment
  __shared__ int32_t t_off[kMaxExperts + 1];
  __shared__ int32_t wsum[kPermThreads / 32];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int me = blockIdx.x;
  for (int e = tid; e <= E; e += kPermThreads) base[e] = 0;
  __syncthreads();
  // a slot whose expert is out of range: another rank's under expert parallelism (skipped, perm_row = -1), else a bad
  // index (flagged, counted as expert 0)
  auto expert_of = [&](int i) -> int {
    int e = idx[i];
    if (e < 0 || e >= E) e = skip_foreign ? -1 : 0;
    return e;
  };
  for (int i = tid; i < n_slots; i += kPermThreads) {
    const int raw = idx[i];
    if (raw < 0 || raw >= E) {
      if (skip_foreign) continue;
      if (me == 0) atomicOr(status, EB_DEV_BAD_INDEX);
    }
    atomicAdd(&base[expert_of(i) + 1], 1);
  }
  __syncthreads();
  if (warp == 0) {  // inclusive prefix over base[1..E], 32 experts per step
    int carry = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane;
      int v = e < E ? base[e + 1] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
      }
      if (e < E) base[e + 1] = carry + v;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
  }
  __syncthreads();
  if (me == 0) {
    for (int e = tid; e <= E; e += kPermThreads) seg_off[e] = base[e];
    if (tile_ws) {
      // token-tile table of the grouped GEMMs over these segments (layout of eb_gemm_group_tiles):
      // blk_off[E+1], n_tiles, tile_group[max_tiles], tile_row0[max_tiles]
      int32_t* blk_off = tile_ws;
      int32_t* n_tiles = tile_ws + (E + 1);
      int32_t* tile_group = n_tiles + 1;
      int32_t* tile_row0 = tile_group + max_tiles;
      if (tid == 0) {
        int tt = 0, bb = 0;
        for (int e = 0; e < E; ++e) {
          const int len = base[e + 1] - base[e];
          t_off[e] = tt;
          blk_off[e] = bb;
          tt += (len + tn - 1) / tn;
          bb += (len + 127) / 128;
        }
        t_off[E] = tt;
        blk_off[E] = bb;
        if (tt > max_tiles) {
          atomicOr(status, EB_DEV_BAD_INDEX);
          tt = max_tiles;
        }
        *n_tiles = tt;
      }
      __syncthreads();
      for (int e = tid; e < E; e += kPermThreads)
        for (int t = t_off[e]; t < t_off[e + 1] && t < max_tiles; ++t) {
          tile_group[t] = e;
          tile_row0[t] = base[e] + (t - t_off[e]) * tn;
        }
    }
  }
  // the slots of expert `me`, in slot order
  int placed = base[me];
  for (int i0 = 0; i0 < n_slots; i0 += kPermThreads) {
    const int i = i0 + tid;
    const int e = i < n_slots ? expert_of(i) : -2;
    const bool mine = e == me;
    const unsigned votes = __ballot_sync(0xffffffffu, mine);
    if (lane == 0) wsum[warp] = __popc(votes);
    __syncthreads();
    int before = 0, total = 0;
#pragma unroll
    for (int w = 0; w < kPermThreads / 32; ++w) {
      const int c = wsum[w];
      if (w < warp) before += c;
      total += c;
    }
    if (mine) {
      const int r = placed + before + __popc(votes & ((1u << lane) - 1u));
      perm_row[i] = r;
      row_token[r] = i / top_k;
    } else if (me == 0 && e == -1) {
      perm_row[i] = -1;  // another rank's expert
    }
    placed += total;
    __syncthreads();
  }
}

// x[t] = bf16( x[t] + bf16( sum_j w[t][j] * y[perm_row[t*top_k+j]] ) ), j ascending, fmaf.  8 columns per thread.
__global__ void moe_combine_kernel(const uint16_t* y, const int32_t* perm_row, const float* wts, int T, int top_k,
                                   int H, uint16_t* x, int64_t n_rows) {
  eb::pdl_wait();  // programmatic dependent launch: the predecessor in the stream has completed
  eb::pdl_trigger();
  const int h8 = H >> 3;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)T * h8) return;
  const int t = (int)(idx / h8), c = (int)(idx % h8) * 8;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int j = 0; j < top_k; ++j) {
    const int r = perm_row[(int64_t)t * top_k + j];
    if (r < 0 || r >= n_rows) continue;
    const float w = wts[(int64_t)t * top_k + j];
    const uint4 v = *reinterpret_cast<const uint4*>(y + (int64_t)r * H + c);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      acc[2 * k] = __fmaf_rn(w, __uint_as_float(u[k] << 16), acc[2 * k]);
      acc[2 * k + 1] = __fmaf_rn(w, __uint_as_float(u[k] & 0xFFFF0000u), acc[2 * k + 1]);
    }
  }
  uint4 xv = *reinterpret_cast<const uint4*>(x + (int64_t)t * H + c);
  uint32_t xu[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    uint32_t m;  // the expert mix is rounded to bf16 before the residual add
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(m) : "f"(acc[2 * k + 1]), "f"(acc[2 * k]));
    const float lo = __fadd_rn(__uint_as_float(xu[k] << 16), __uint_as_float(m << 16));
    const float hi = __fadd_rn(__uint_as_float(xu[k] & 0xFFFF0000u), __uint_as_float(m & 0xFFFF0000u));
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(xu[k]) : "f"(hi), "f"(lo));
  }
  *reinterpret_cast<uint4*>(x + (int64_t)t * H + c) = make_uint4(xu[0], xu[1], xu[2], xu[3]);
}

template <int EPL, int HPL>
int32_t launch_router2(unsigned grid, size_t smem, cudaStream_t st, const uint16_t* x, const uint16_t* wr, int T, int E, int H,
                    int top_k, int32_t* idx, float* wts, float* logits) {
  // The one-CTA-per-few-tokens kernel up to 4096 tokens; tokens per CTA: the fewest of 1, 2, 4, 8 that give at most one
  // CTA per SM (the kernel's registers allow one CTA per SM), 8 beyond that.  (The staged pipeline below costs at least
  // ~5 us per 8 experts however few tokens there are: 85 us at 320 tokens x 128 experts, 21 us at 256 x 32.)
  if (T <= 4096) {
    int sms = 148, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const size_t xs_bytes = (size_t)H * sizeof(uint16_t);
    if (T <= sms) {
      EB_CUDA(eb::launch(router_direct_kernel<EPL, HPL, 1>, dim3((unsigned)T), dim3(256), 0, st, x, wr, T, E, H, top_k, idx, wts, logits));
    } else if (T <= 2 * sms) {
      EB_CUDA(eb::launch(router_direct_kernel<EPL, HPL, 2>, dim3((unsigned)((T + 1) / 2)), dim3(256), 2 * xs_bytes, st, x, wr, T, E, H,
                         top_k, idx, wts, logits));
    } else if (T <= 4 * sms) {
      auto k4 = router_direct_kernel<EPL, HPL, 4>;
      EB_CUDA(cudaFuncSetAttribute(k4, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(4 * xs_bytes)));
      EB_CUDA(eb::launch(k4, dim3((unsigned)((T + 3) / 4)), dim3(256), 4 * xs_bytes, st, x, wr, T, E, H, top_k, idx, wts, logits));
    } else {
      auto k8 = router_direct_kernel<EPL, HPL, 8>;
      EB_CUDA(cudaFuncSetAttribute(k8, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(8 * xs_bytes)));
      EB_CUDA(eb::launch(k8, dim3((unsigned)((T + 7) / 8)), dim3(256), 8 * xs_bytes, st, x, wr, T, E, H, top_k, idx, wts, logits));
    }
    return EB_OK;
  }
  auto kfn = router_topk_kernel<EPL, HPL>;
  static bool configured[64] = {false};  // the attribute is per device
  int dev = 0;
  EB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    EB_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 2 * kRouterChunk * HPL * 256 * (int)sizeof(uint16_t)));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  EB_CUDA(eb::launch(kfn, dim3(grid), dim3(256), smem, st, x, wr, T, E, H, top_k, idx, wts, logits));
  return EB_OK;
}

template <int HPL>
int32_t launch_router(int epl, unsigned grid, size_t smem, cudaStream_t st, const uint16_t* x, const uint16_t* wr, int T,
                   int E, int H, int top_k, int32_t* idx, float* wts, float* logits) {
  if (epl <= 1)
    return launch_router2<1, HPL>(grid, smem, st, x, wr, T, E, H, top_k, idx, wts, logits);
  else if (epl <= 2)
    return launch_router2<2, HPL>(grid, smem, st, x, wr, T, E, H, top_k, idx, wts, logits);
  else if (epl <= 4)
    return launch_router2<4, HPL>(grid, smem, st, x, wr, T, E, H, top_k, idx, wts, logits);
  else
    return launch_router2<8, HPL>(grid, smem, st, x, wr, T, E, H, top_k, idx, wts, logits);
}

}  // namespace

extern "C" {

int32_t eb_moe_route(const void* d_x, const void* d_wr, int32_t T, int32_t E, int32_t H, int32_t top_k, int32_t* d_idx,
                     float* d_wts, float* d_logits, void* stream) {
  EB_REQUIRE(d_x && d_wr && d_idx && d_wts, EB_ERR_ARG, "eb_moe_route: null pointer");
  EB_REQUIRE(T >= 0 && E >= 1 && E <= kMaxExperts && top_k >= 1 && top_k <= kMaxTopK && top_k <= E, EB_ERR_UNSUPPORTED,
             "eb_moe_route: E %d (<= %d), top_k %d (<= %d)", E, kMaxExperts, top_k, kMaxTopK);
  EB_REQUIRE(H >= 8 && H % 8 == 0 && H <= 4096, EB_ERR_UNSUPPORTED, "eb_moe_route: hidden size %d (multiple of 8, <= 4096)", H);
  EB_REQUIRE((uintptr_t)d_wr % 16 == 0, EB_ERR_ARG, "eb_moe_route: router matrix must be 16-byte aligned");
  EB_REQUIRE((uintptr_t)d_wr % 16 == 0, EB_ERR_ARG, "eb_moe_route: router matrix must be 16-byte aligned");
  if (T == 0) return EB_OK;
  const size_t smem = 2 * (size_t)kRouterChunk * H * sizeof(uint16_t);
  const unsigned grid = (unsigned)((T + 7) / 8);
  cudaStream_t st = eb::as_stream(stream);
  const uint16_t* x = (const uint16_t*)d_x;
  const uint16_t* wr = (const uint16_t*)d_wr;
  const int epl = (E + 31) / 32, hpl = (H + 255) / 256;  // 8-element groups per lane
  if (hpl <= 2)
    return launch_router<2>(epl, grid, smem, st, x, wr, T, E, H, top_k, d_idx, d_wts, d_logits);
  else if (hpl <= 4)
    return launch_router<4>(epl, grid, smem, st, x, wr, T, E, H, top_k, d_idx, d_wts, d_logits);
  else if (hpl <= 8)
    return launch_router<8>(epl, grid, smem, st, x, wr, T, E, H, top_k, d_idx, d_wts, d_logits);
  else if (hpl <= 12)
    return launch_router<12>(epl, grid, smem, st, x, wr, T, E, H, top_k, d_idx, d_wts, d_logits);
  else
    return launch_router<16>(epl, grid, smem, st, x, wr, T, E, H, top_k, d_idx, d_wts, d_logits);
}

int32_t eb_moe_permute(const int32_t* d_idx, int32_t T, int32_t top_k, int32_t E, int32_t* d_seg_off,
                       int32_t* d_perm_row, int32_t* d_row_token, void* stream) {
  EB_REQUIRE(d_idx && d_seg_off && d_perm_row && d_row_token, EB_ERR_ARG, "eb_moe_permute: null pointer");
  EB_REQUIRE(T >= 0 && top_k >= 1 && E >= 1 && E <= kMaxExperts, EB_ERR_UNSUPPORTED, "eb_moe_permute: E %d (<= %d)", E,
             kMaxExperts);
  int32_t* status = eb::status_word();
  EB_REQUIRE(status, EB_ERR_NODEVICE, "eb_moe_permute: no device");
  EB_CUDA(eb::launch(moe_permute_kernel, dim3((unsigned)E), dim3(kPermThreads), 0, eb::as_stream(stream), d_idx, T * top_k, top_k, E,
                     d_seg_off, d_perm_row, d_row_token, 0, 0, nullptr, status, 0));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

static int32_t permute_tiles(const int32_t* d_idx, int32_t T, int32_t top_k, int32_t E, int32_t* d_seg_off,
                             int32_t* d_perm_row, int32_t* d_row_token, int32_t tile_tokens, void* d_group_work,
                             void* stream, int skip_foreign);

int32_t eb_moe_permute_tiles(const int32_t* d_idx, int32_t T, int32_t top_k, int32_t E, int32_t* d_seg_off,
                             int32_t* d_perm_row, int32_t* d_row_token, int32_t tile_tokens, void* d_group_work,
                             void* stream) {
  return permute_tiles(d_idx, T, top_k, E, d_seg_off, d_perm_row, d_row_token, tile_tokens, d_group_work, stream, 0);
}

static int32_t permute_tiles(const int32_t* d_idx, int32_t T, int32_t top_k, int32_t E, int32_t* d_seg_off,
                             int32_t* d_perm_row, int32_t* d_row_token, int32_t tile_tokens, void* d_group_work,
                             void* stream, int skip_foreign) {
  EB_REQUIRE(d_idx && d_seg_off && d_perm_row && d_row_token && d_group_work, EB_ERR_ARG, "eb_moe_permute_tiles: null pointer");
  EB_REQUIRE(T >= 0 && top_k >= 1 && E >= 1 && E <= kMaxExperts, EB_ERR_UNSUPPORTED, "eb_moe_permute_tiles: E %d (<= %d)",
             E, kMaxExperts);
  EB_REQUIRE(tile_tokens == 16 || tile_tokens == 32 || tile_tokens == 64 || tile_tokens == 128, EB_ERR_ARG,
             "eb_moe_permute_tiles: tile_tokens %d not in {16,32,64,128}", tile_tokens);
  int32_t* status = eb::status_word();
  EB_REQUIRE(status, EB_ERR_NODEVICE, "eb_moe_permute_tiles: no device");
  const int max_tiles = (T * top_k) / tile_tokens + E;
  EB_CUDA(eb::launch(moe_permute_kernel, dim3((unsigned)E), dim3(kPermThreads), 0, eb::as_stream(stream), d_idx, T * top_k, top_k, E,
                     d_seg_off, d_perm_row, d_row_token, tile_tokens, max_tiles, (int32_t*)d_group_work, status, skip_foreign));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_moe_combine(const void* d_y, const int32_t* d_perm_row, const float* d_wts, int32_t T, int32_t top_k,
                       int32_t H, void* d_x, void* stream) {
  EB_REQUIRE(d_y && d_perm_row && d_wts && d_x, EB_ERR_ARG, "eb_moe_combine: null pointer");
  EB_REQUIRE(T >= 0 && top_k >= 1 && H >= 8 && H % 8 == 0, EB_ERR_ARG, "eb_moe_combine: H %d must be a multiple of 8", H);
  EB_REQUIRE(((uintptr_t)d_y % 16 == 0) && ((uintptr_t)d_x % 16 == 0), EB_ERR_ARG, "eb_moe_combine: 16-byte alignment");
  if (T == 0) return EB_OK;
  const int64_t n = (int64_t)T * (H / 8);
  EB_CUDA(eb::launch(moe_combine_kernel, dim3((unsigned)eb::cdiv(n, 256)), dim3(256), 0, eb::as_stream(stream), 
      (const uint16_t*)d_y, d_perm_row, d_wts, T, top_k, H, (uint16_t*)d_x, (int64_t)T * top_k));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Expert parallelism: a rank owns experts [e0, e0 + E_local).  Routing is replicated (every rank sees the same
// activations after the tensor-parallel all-reduce), so no index exchange is needed: each rank keeps the slots of
// its own experts, and the per-rank partial mixes are summed by an all-reduce.

namespace {

__global__ void localize_experts_kernel(const int32_t* idx, int n, int e0, int e_local, int32_t* out) {
  eb::pdl_wait();
  eb::pdl_trigger();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int e = idx[i] - e0;
  out[i] = (e >= 0 && e < e_local) ? e : -1;
}

// out[t] = sum over this rank's slots j of w[t][j] * y[perm_row[t][j]]  (fp32, slots in ascending j)
// out == nullptr (bf16 only): the mix goes straight into every rank's plane of a whole-batch exchange (pp), and the launch
// raises the collective's flags itself.
template <int BF16_OUT>
__global__ void moe_combine_f32_kernel(const uint16_t* y, const int32_t* perm_row, const float* wts, int T, int top_k, int H,
                                       float* out, int64_t n_rows, const eb::PeerPlanes pp) {
  eb::pdl_wait();
  eb::pdl_trigger();
  const int h8 = H >> 3;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < (int64_t)T * h8) {
    const int t = (int)(idx / h8), c = (int)(idx % h8) * 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < top_k; ++j) {
      const int r = perm_row[(int64_t)t * top_k + j];
      if (r < 0 || r >= n_rows) continue;
      const float w = wts[(int64_t)t * top_k + j];
      const uint4 v = *reinterpret_cast<const uint4*>(y + (int64_t)r * H + c);
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        acc[2 * k] = __fmaf_rn(w, __uint_as_float(u[k] << 16), acc[2 * k]);
        acc[2 * k + 1] = __fmaf_rn(w, __uint_as_float(u[k] & 0xFFFF0000u), acc[2 * k + 1]);
      }
    }
    if (BF16_OUT) {
      uint32_t h[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(h[k]) : "f"(acc[2 * k + 1]), "f"(acc[2 * k]));
      const uint4 hv = make_uint4(h[0], h[1], h[2], h[3]);
      if (out) {
        *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(out) + (int64_t)t * H + c) = hv;
      } else {
        for (int p = 0; p < pp.size; ++p) *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(pp.dst[p]) + (int64_t)t * H + c) = hv;
      }
    } else {
      float4* o = reinterpret_cast<float4*>(out + (int64_t)t * H + c);
      o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
  }
  if (BF16_OUT && !out) eb::peer_arrive_cta(pp);  // reached by every thread of the CTA
}

}  // namespace

extern "C" {

int32_t eb_moe_localize(const int32_t* d_idx, int32_t n, int32_t e0, int32_t e_local, int32_t* d_out, void* stream) {
  EB_REQUIRE(d_idx && d_out && n >= 0 && e0 >= 0 && e_local >= 1, EB_ERR_ARG, "eb_moe_localize: bad argument");
  if (n == 0) return EB_OK;
  EB_CUDA(eb::launch(localize_experts_kernel, dim3((unsigned)eb::cdiv(n, 256)), dim3(256), 0, eb::as_stream(stream), d_idx, n, e0,
                     e_local, d_out));
  return EB_OK;
}

int32_t eb_moe_permute_tiles_local(const int32_t* d_idx_local, int32_t T, int32_t top_k, int32_t e_local, int32_t* d_seg_off,
                                   int32_t* d_perm_row, int32_t* d_row_token, int32_t tile_tokens, void* d_group_work,
                                   void* stream) {
  return permute_tiles(d_idx_local, T, top_k, e_local, d_seg_off, d_perm_row, d_row_token, tile_tokens, d_group_work, stream, 1);
}

int32_t eb_moe_combine_f32(const void* d_y, const int32_t* d_perm_row, const float* d_wts, int32_t T, int32_t top_k, int32_t H,
                           float* d_out, void* stream) {
  EB_REQUIRE(d_y && d_perm_row && d_wts && d_out, EB_ERR_ARG, "eb_moe_combine_f32: null pointer");
  EB_REQUIRE(T >= 0 && top_k >= 1 && H >= 8 && H % 8 == 0, EB_ERR_ARG, "eb_moe_combine_f32: H %d must be a multiple of 8", H);
  if (T == 0) return EB_OK;
  const int64_t n = (int64_t)T * (H / 8);
  EB_CUDA(eb::launch(moe_combine_f32_kernel<0>, dim3((unsigned)eb::cdiv(n, 256)), dim3(256), 0, eb::as_stream(stream),
                     (const uint16_t*)d_y, d_perm_row, d_wts, T, top_k, H, d_out, (int64_t)T * top_k, eb::PeerPlanes{}));
  return EB_OK;
}

int32_t eb_moe_combine_bf16(const void* d_y, const int32_t* d_perm_row, const float* d_wts, int32_t T, int32_t top_k, int32_t H,
                            void* d_out, void* stream) {
  EB_REQUIRE(d_y && d_perm_row && d_wts && d_out, EB_ERR_ARG, "eb_moe_combine_bf16: null pointer");
  EB_REQUIRE(T >= 0 && top_k >= 1 && H >= 8 && H % 8 == 0, EB_ERR_ARG, "eb_moe_combine_bf16: H %d must be a multiple of 8", H);
  EB_REQUIRE((uintptr_t)d_out % 16 == 0, EB_ERR_ARG, "eb_moe_combine_bf16: output must be 16-byte aligned");
  if (T == 0) return EB_OK;
  const int64_t n = (int64_t)T * (H / 8);
  EB_CUDA(eb::launch(moe_combine_f32_kernel<1>, dim3((unsigned)eb::cdiv(n, 256)), dim3(256), 0, eb::as_stream(stream),
                     (const uint16_t*)d_y, d_perm_row, d_wts, T, top_k, H, (float*)d_out, (int64_t)T * top_k, eb::PeerPlanes{}));
  return EB_OK;
}

int32_t eb_moe_combine_bf16_to_peers(eb_symm* s, int64_t dst_off, int64_t plane_step, const void* d_y, const int32_t* d_perm_row,
                                     const float* d_wts, int32_t T, int32_t top_k, int32_t H, int32_t* seq, void* stream) {
  EB_REQUIRE(s && d_y && d_perm_row && d_wts && seq, EB_ERR_ARG, "eb_moe_combine_bf16_to_peers: null pointer");
  EB_REQUIRE(T >= 1 && top_k >= 1 && H >= 8 && H % 8 == 0, EB_ERR_ARG, "eb_moe_combine_bf16_to_peers: T %d, H %d (a multiple of 8)", T, H);
  eb::PeerPlanes pp;
  const int32_t rc = eb::symm_peer_planes(s, dst_off, plane_step, (int64_t)T * H * 2, &pp, seq);
  if (rc != EB_OK) return rc;
  const int64_t n = (int64_t)T * (H / 8);
  EB_CUDA(eb::launch(moe_combine_f32_kernel<1>, dim3((unsigned)eb::cdiv(n, 256)), dim3(256), 0, eb::as_stream(stream),
                     (const uint16_t*)d_y, d_perm_row, d_wts, T, top_k, H, (float*)nullptr, (int64_t)T * top_k, pp));
  return EB_OK;
}

}  // extern "C"

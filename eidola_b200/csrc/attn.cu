// Paged KV-cache append and paged sink attention (decode / speculative verify) for sm_100a.
//
// Cache layout of one layer: [num_pages][2 (K,V)][n_kv][16 tokens][64 dims] bf16.  Seen as a 2-D tensor of
// 128-byte rows, a page is 32*n_kv consecutive rows, so one tiled TMA copy (128-byte swizzle) brings a whole
// page -- every KV head of 16 tokens, K and V -- into shared memory, and ldmatrix reads it without bank
// conflicts.
//
// attn_kernel: one CTA per work item (a run of logical pages of one sequence, planned on the host by
// eb_attn_plan).  Eight compute warps per 16 query rows (one set for decode, two or three sets for speculative
// verification) and one producer warp.  A pipeline stage holds 256 rows (32 KiB): one page when the rank holds 8 KV
// heads, 8/n_kv pages otherwise.  Compute warp w of a set owns KV head w % n_kv of page w / n_kv of each stage:
// S = Q K^T and O += P V on mma.sync m16n8k16 (bf16 in, fp32 accumulate), rows of the M tile = (query position,
// query head of the GQA group), online softmax in base 2 with quad shuffles.
// P is fed to the second MMA as a bf16 head plus a bf16 remainder (two MMAs), so the result carries about 16
// bits of the softmax weights.  The kernel is HBM-bound: per 2 KiB of K and 2 KiB of V a warp issues 24 MMAs.
//
// The sink logit enters the softmax denominator exactly once: in the kernel epilogue when a sequence has a
// single partial, otherwise in attn_merge_kernel, which combines split-K partials (m, l, acc) by log-sum-exp.
//
// The reference project has no attention code (its inference runs in a `llama-server` child process,
// crates/eidola-app-core/src/local_models.rs:1612-1626).
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdlib.h>

#include <algorithm>
#include <mutex>

#include "common.h"

namespace {

constexpr int kHeadDim = 64;
constexpr int kPage = 16;
constexpr int kComputeWarps = 8;
constexpr int kStageBytes = 32768;   // 256 rows of 128 bytes
constexpr int kMaxItemPages = 512;
constexpr uint32_t kWaitTries = 1u << 22;
constexpr float kNegBig = -1.0e30f;

struct AttnParams {
  const uint16_t* q;
  int64_t q_stride;
  uint16_t* out;
  int64_t out_stride;
  const int32_t* block_tables;
  int32_t bt_stride;
  const int32_t* seq_slots;
  const int32_t* q_off;
  const int32_t* ctx_lens;
  const float* sinks;
  int32_t window, n_q, max_q_len, num_pages;
  float scale_log2;
  const eb_attn_item* items;
  const int32_t* seq_part;
  float* part_acc;
  float* part_ml;
  uint32_t wait_tries;  // polls a bounded wait makes before it gives up (eb_wait_limit_set)
  int32_t part_slots;  // partial slots part_acc / part_ml hold; a slot index outside [0, part_slots) is skipped and flagged
  int32_t* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `tries` polls, raises the CTA's abort flag and the device status word.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status,
                                          uint32_t tries) {
  for (uint32_t i = 0; i < tries; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 64) {
      __nanosleep(64);
      if (*abort_flag) return false;
    }
  }
  *abort_flag = 1;
  atomicOr(status, EB_DEV_WAIT_TIMEOUT);
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int32_t x, int32_t y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x for x <= 0 (or -inf): one MUFU instruction, relative error about 2^-22.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// MT  : 16-row M tiles per warp
// WT  : warp sets; set w handles M tiles [w * MT, (w + 1) * MT) of every page, so ceil(max_q_len * G / 16) = MT * WT.
//       Verify shapes (40 query rows per KV head) run MT = 1, WT = 3: the same 72 MMAs per page and KV head as one
//       warp with three tiles, but on 24 warps whose dependent MMA chains overlap, at 80 registers instead of 168.
// HKV : KV heads held by this rank (8, 4, 2 or 1)
// G   : query heads per KV head (8 or 4); row r of the M tiles = (query position r / G, head r % G of the group)
template <int MT, int WT, int HKV, int STAGES, int G>
__global__ void __launch_bounds__((kComputeWarps * WT + 1) * 32, (MT == 1 && WT == 1) ? 2 : 1)
attn_kernel(const __grid_constant__ CUtensorMap tmap, const AttnParams p) {
  eb::pdl_wait();  // programmatic dependent launch: the predecessor in the stream has completed
  eb::pdl_trigger();
  constexpr int kCW = kComputeWarps * WT;        // compute warps of the CTA
  constexpr int kNT = (kCW + 1) * 32;            // threads of the CTA
  constexpr int PPS = kComputeWarps / HKV;       // pages per stage
  constexpr int kPageRows = 2 * HKV * kPage;     // 128-byte rows per page
  constexpr int kPageBytes = kPageRows * 128;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t stage0 = (raw + 1023u) & ~1023u;
  uint8_t* after = smem_raw + (stage0 - raw) + STAGES * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(after);  // full[STAGES], empty[STAGES]
  int32_t* page_ids = reinterpret_cast<int32_t*>(after + 2 * STAGES * sizeof(uint64_t));
  __shared__ int abort_flag;
  __shared__ int n_issued;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const eb_attn_item item = p.items[blockIdx.x];
  const int seq = item.seq;
  const int slot = p.seq_slots[seq];
  const int L = p.ctx_lens[seq];
  const int q0 = p.q_off[seq];
  const int ql = p.q_off[seq + 1] - q0;
  int n_pages = item.page_end - item.page_begin;
  if (n_pages > kMaxItemPages) {  // the planner never emits this; refuse instead of overrunning page_ids
    if (tid == 0) atomicOr(p.status, EB_DEV_BAD_INDEX);
    n_pages = kMaxItemPages;
  }

  for (int j = tid; j < n_pages; j += kNT) {
    int32_t id = p.block_tables[(int64_t)slot * p.bt_stride + item.page_begin + j];
    if (id < 0 || id >= p.num_pages) {
      atomicOr(p.status, EB_DEV_BAD_INDEX);
      id = 0;
    }
    page_ids[j] = id;
  }
  if (tid == 0) {
    abort_flag = 0;
    n_issued = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bars[s]), 1);
      mbar_init(smem_u32(&bars[STAGES + s]), kCW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  const int n_iters = (n_pages + PPS - 1) / PPS;

  if (warp == kCW) {
    // ---------------- producer: one thread feeds the stage ring with whole pages
    if (lane == 0) {
      for (int it = 0; it < n_iters; ++it) {
        const int s = it % STAGES;
        if (it >= STAGES) {
          if (!mbar_wait(smem_u32(&bars[STAGES + s]), ((it / STAGES) - 1) & 1, &abort_flag, p.status, p.wait_tries)) break;
        }
        const int np = min(PPS, n_pages - it * PPS);
        const uint32_t full = smem_u32(&bars[s]);
        mbar_arrive_expect_tx(full, (uint32_t)(np * kPageBytes));
        for (int j = 0; j < np; ++j)
          tma_load_2d(stage0 + s * kStageBytes + j * kPageBytes, &tmap, 0, page_ids[it * PPS + j] * kPageRows, full);
        n_issued = it + 1;
      }
    }
  } else {
    // ---------------- consumers
    const int set = warp / kComputeWarps;             // warp set = which M tiles
    const int hk = (warp % kComputeWarps) % HKV;      // KV head of this warp
    const int sub = (warp % kComputeWarps) / HKV;     // page of the stage this warp takes
    const int row_base = set * MT * 16;               // first query row of this warp's tiles
    const int tq = lane & 3;

    // Q fragments (A operand): rows = (query position, head of the group), kept in registers.
    uint32_t qf[MT][4][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int row = row_base + mt * 16 + half * 8 + (lane >> 2);
        const int qi = row / G;
        const uint16_t* qrow = p.q + (int64_t)(q0 + qi) * p.q_stride + (int64_t)(hk * G + row % G) * kHeadDim;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          uint32_t lo = 0, hi = 0;
          if (qi < ql) {
            lo = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + tq * 2);
            hi = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + tq * 2 + 8);
          }
          qf[mt][ks][half] = lo;       // a0 (row g) / a1 (row g+8)
          qf[mt][ks][2 + half] = hi;   // a2 / a3
        }
      }
    }

    float o[MT][8][4];
    float m_run[MT][2], l_run[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      m_run[mt][0] = m_run[mt][1] = kNegBig;
      l_run[mt][0] = l_run[mt][1] = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) o[mt][nt][0] = o[mt][nt][1] = o[mt][nt][2] = o[mt][nt][3] = 0.f;
    }

    // per-lane constant parts of the ldmatrix addresses
    const int mj = lane >> 3, mr = lane & 7;
    const int k_tok = (mj >> 1) * 8 + mr, k_chunk = mj & 1;  // K: matrices (tok 0-7 | 8-15) x (dims lo | hi)
    const int v_tok = (mj & 1) * 8 + mr, v_chunk = mj >> 1;  // V: matrices (dims lo | hi) x (tok 0-7 | 8-15)

    for (int it = 0; it < n_iters; ++it) {
      const int s = it % STAGES;
      if (!mbar_wait(smem_u32(&bars[s]), (it / STAGES) & 1, &abort_flag, p.status, p.wait_tries)) break;
      const int pl = it * PPS + sub;
      if (pl < n_pages) {
        const uint32_t page_base = stage0 + s * kStageBytes + sub * kPageBytes;
        const uint32_t kbase = page_base + hk * (kPage * 128);
        const uint32_t vbase = page_base + (HKV + hk) * (kPage * 128);
        const int t0 = (item.page_begin + pl) * kPage;

        float sc[MT][2][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int nt = 0; nt < 2; ++nt) sc[mt][nt][0] = sc[mt][nt][1] = sc[mt][nt][2] = sc[mt][nt][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          uint32_t b[4];
          ldsm_x4(b, kbase + k_tok * 128 + (((ks * 2 + k_chunk) ^ (k_tok & 7)) << 4));
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma_bf16(sc[mt][0], qf[mt][ks], b[0], b[1]);
            mma_bf16(sc[mt][1], qf[mt][ks], b[2], b[3]);
          }
        }

        // Only the pages at the ends of the visible range need the causal / window mask (warp-uniform test).
        const bool edge = (t0 + kPage - 1 > L - ql) || (p.window > 0 && t0 < L - p.window);
        uint32_t pa[MT][4], pb[MT][4];  // P = pa + pb: bf16 head and bf16 remainder, so P V keeps ~16 bits of P
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int pq = L - ql + (row_base + mt * 16 + half * 8 + (lane >> 2)) / G;  // absolute position of this row's query
            const int lo = p.window > 0 ? pq - p.window + 1 : 0;
            float v[2][2];
            float mx = kNegBig;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const int t = t0 + nt * 8 + tq * 2 + e;
                float x = sc[mt][nt][half * 2 + e];  // raw score; the positive scale is applied after the max
                if (edge && (t > pq || t < lo)) x = -INFINITY;
                v[nt][e] = x;
                mx = fmaxf(mx, x);
              }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run[mt][half], mx * p.scale_log2);
            float ps = 0.f;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                v[nt][e] = fast_exp2(fmaf(v[nt][e], p.scale_log2, -m_new));
                ps += v[nt][e];
              }
            // the running maximum of a quad's row rarely moves after the first pages: rescale only then
            if (m_new != m_run[mt][half]) {
              const float alpha = fast_exp2(m_run[mt][half] - m_new);
              m_run[mt][half] = m_new;
              l_run[mt][half] *= alpha;
#pragma unroll
              for (int nt = 0; nt < 8; ++nt) {
                o[mt][nt][half * 2 + 0] *= alpha;
                o[mt][nt][half * 2 + 1] *= alpha;
              }
            }
            l_run[mt][half] += ps;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {  // a0 / a1: tokens 0-7, a2 / a3: tokens 8-15
              const uint32_t hi = pack_bf16(v[nt][0], v[nt][1]);
              pa[mt][2 * nt + half] = hi;
              pb[mt][2 * nt + half] = pack_bf16(v[nt][0] - __uint_as_float(hi << 16), v[nt][1] - __uint_as_float(hi & 0xFFFF0000u));
            }
          }
        }

#pragma unroll
        for (int dp = 0; dp < 4; ++dp) {
          uint32_t b[4];
          ldsm_x4_t(b, vbase + v_tok * 128 + (((dp * 2 + v_chunk) ^ (v_tok & 7)) << 4));
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma_bf16(o[mt][dp * 2], pa[mt], b[0], b[1]);
            mma_bf16(o[mt][dp * 2 + 1], pa[mt], b[2], b[3]);
            mma_bf16(o[mt][dp * 2], pb[mt], b[0], b[1]);
            mma_bf16(o[mt][dp * 2 + 1], pb[mt], b[2], b[3]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars[STAGES + s]));
    }

    // ---------------- epilogue
    const int n_parts_seq = p.seq_part[seq + 1] - p.seq_part[seq];
    const bool direct = (n_parts_seq == 1);
    const int part = item.part + sub;
    // a plan that disagrees with the scratch the caller sized (stale items, an understated n_parts) is not followed
    const bool part_ok = direct || (part >= 0 && part < p.part_slots);
    if (!part_ok && lane == 0) atomicOr(p.status, EB_DEV_BAD_INDEX);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int row = row_base + mt * 16 + half * 8 + (lane >> 2);
        const int qi = row / G;
        float l = l_run[mt][half];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (qi >= ql || !part_ok) continue;
        const int head = hk * G + row % G;
        const float m = m_run[mt][half];
        if (direct) {
          const float sk = p.sinks[head] * 1.4426950408889634f;
          const float mf = fmaxf(m, sk);
          const float w = exp2f(m - mf);
          const float inv = w / (l * w + exp2f(sk - mf));
          uint16_t* orow = p.out + (int64_t)(q0 + qi) * p.out_stride + (int64_t)head * kHeadDim;
#pragma unroll
          for (int nt = 0; nt < 8; ++nt)
            *reinterpret_cast<uint32_t*>(orow + nt * 8 + tq * 2) =
                pack_bf16(o[mt][nt][half * 2] * inv, o[mt][nt][half * 2 + 1] * inv);
        } else {
          const int64_t row = ((int64_t)part * p.max_q_len + qi) * p.n_q + head;
          float* arow = p.part_acc + row * kHeadDim;
#pragma unroll
          for (int nt = 0; nt < 8; ++nt)
            *reinterpret_cast<float2*>(arow + nt * 8 + tq * 2) = make_float2(o[mt][nt][half * 2], o[mt][nt][half * 2 + 1]);
          if (tq == 0) *reinterpret_cast<float2*>(p.part_ml + row * 2) = make_float2(m, l);
        }
      }
    }
  }

  __syncthreads();
  if (abort_flag && tid == 0) {
    // A wait gave up.  Before the CTA releases its shared memory, wait (bounded) for the copies still in flight.
    const int issued = n_issued;
    for (int it = max(0, issued - STAGES); it < issued; ++it) {
      const uint32_t bar = smem_u32(&bars[it % STAGES]);
      for (uint32_t i = 0; i < kWaitTries; ++i) {
        if (mbar_try_wait(bar, (it / STAGES) & 1)) break;
        __nanosleep(64);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// tcgen05 helpers of the verify kernel below.
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint64_t tc_desc_sw128(uint32_t addr) {  // 128-byte rows, 8-row groups 1 KiB apart, 128-byte swizzle
  uint64_t d = (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(1024u >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// D[tmem] (+)= A[smem] x B[smem], bf16 -> fp32
__device__ __forceinline__ void tc_mma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
}
// D[tmem] (+)= A[tmem] x B[smem]
__device__ __forceinline__ void tc_mma_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d), "r"(a_tmem), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
}
#define EB_O8(a, o) "=r"(a[o]), "=r"(a[o + 1]), "=r"(a[o + 2]), "=r"(a[o + 3]), "=r"(a[o + 4]), "=r"(a[o + 5]), "=r"(a[o + 6]), "=r"(a[o + 7])
#define EB_I8(a, o) "r"(a[o]), "r"(a[o + 1]), "r"(a[o + 2]), "r"(a[o + 3]), "r"(a[o + 4]), "r"(a[o + 5]), "r"(a[o + 6]), "r"(a[o + 7])
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// Verify shapes on the sm_100a tensor cores (tcgen05).  With 17..48 query rows per KV head the mma.sync kernel above is
// bound by the legacy tensor pipe and by instruction issue (0.44 of the HBM rate at q_len 5); here S = Q K^T and
// O += P V run as tcgen05.mma with the accumulators in tensor memory.  One CTA = one work item x one KV head, two CTAs
// per SM.  A pipeline stage is 128 keys (8 pages), fetched per page as one 2 KiB TMA copy of the head's K rows and one
// of its V rows; it is worked on as two sub-blocks of 64 keys, which alternate between two 64-column buffers of tensor
// memory, so that the products of one sub-block run while the softmax warps work on the next.  Per sub-block:
//   S[64 x 64] = Q K^T       4 MMAs with M = 64: row r of the tile lives in tensor-memory lane 32 (r / 16) + r % 16,
//                            so rows 16 w .. 16 w + 15 belong to the lane quarter of warps w and w + 4
//   softmax                  warps w and w + 4 take keys 0..31 and 32..63 of those rows and read them with the 16x256b
//                            shape: a thread holds, per group of 8 keys, two adjacent keys of row lane / 4 and of row
//                            lane / 4 + 8, so all 32 lanes work whenever the warp has 16 rows.  The two warps exchange
//                            their maxima through shared memory.  The reference maximum of a row is only raised when a
//                            score exceeds it by 2^8 (then the row of O is rescaled in tensor memory), a thread keeps
//                            the sum of its own weights, and the row sums are formed once, at the end of the item.
//   P                        written over S with the 16x128b store shape, two keys per column, which lands exactly
//                            where the A operand of the second product is read: the bf16 heads in the rows' own lanes,
//                            the bf16 remainders 16 lanes up, in the lanes a 64-row product never touches
//   O[128 x 64] += P V       4 MMAs with M = 128 (V is the MN-major B operand): lanes 32 w .. 32 w + 15 accumulate
//                            P_head V, lanes 32 w + 16 .. 32 w + 31 P_remainder V; the two are added in the epilogue
// Measured on the way (256 ragged sequences, q_len 5, CUDA events): every MMA of these shapes occupies the issuing
// thread for about 64 clocks whatever its N (a 72-column product that also accumulated the row sums against a tile of
// ones cost as much as 128 columns), so the count of MMAs matters, not their size: 16 + 8 per 128 keys with head and
// remainder as separate 64-row products made the MMA thread the bottleneck (358 us), 8 + 8 as above do not (332 us).
// A bf16 A operand cannot be paired with an fp16 one (the instruction is rejected), so P stays head + remainder: P as a
// single bf16 passes the operator tests at 376 us of the earlier variant but fails the whole-decoder parity bounds.
constexpr int kV64Keys = 128;
constexpr int kV64Pages = kV64Keys / kPage;
constexpr int kV64Stage = 2 * kV64Keys * 128;  // K rows then V rows of one head
constexpr int kV64Stages = 3;
constexpr int kV64Threads = 320;               // 8 softmax warps, producer warp, MMA warp

#define EB_O16(a, o) EB_O8(a, o), EB_O8(a, o + 8)
#define EB_I16(a, o) EB_I8(a, o), EB_I8(a, o + 8)
// 16 lanes x 16 columns: registers 2 j, 2 j + 1 = (row lane/4, column 4 j + lane%4), (row lane/4 + 8, same column)
__device__ __forceinline__ void tc_st_16x128b_x4(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.16x128b.x4.b32 [%8], {%0,%1,%2,%3,%4,%5,%6,%7};" ::EB_I8(r, 0), "r"(taddr) : "memory");
}

// 16 lanes x 32 columns: registers 4 j .. 4 j + 3 = (row lane/4, columns 8 j + 2 (lane%4) + {0, 1}), (row lane/4 + 8, same)
__device__ __forceinline__ void tc_ld_16x256b_x4(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : EB_O16(r, 0)
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_st_16x256b_x4(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x256b.x4.b32 [%16], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};"
      ::EB_I16(r, 0), "r"(taddr)
      : "memory");
}

struct V64Params {
  int32_t n_kv;  // KV heads held by this rank
  int32_t ppi;   // partial slots the plan reserves per item (8 / n_kv)
};

template <int G>  // query heads per KV head
__global__ void __launch_bounds__(kV64Threads, 2)
attn_v64_kernel(const __grid_constant__ CUtensorMap tmap, const AttnParams p, const V64Params vp) {
  eb::pdl_wait();  // programmatic dependent launch: the predecessor in the stream has completed
  eb::pdl_trigger();
  constexpr int NS = kV64Stages;
  constexpr uint32_t kCols = 256;  // S / P of even sub-blocks: 0..63, of odd sub-blocks: 64..127, O: 128..191

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  const uint32_t q_addr = base;                                // 64 rows x 128 B
  const uint32_t stage0 = base + 8192;                         // NS stages
  uint8_t* after = sm + 8192 + NS * kV64Stage;
  uint64_t* bars = reinterpret_cast<uint64_t*>(after);         // full[NS], empty[NS], s_ready[2], p_ready[2], pv_done[2], o_ready
  int32_t* page_ids = reinterpret_cast<int32_t*>(after + (2 * NS + 7) * sizeof(uint64_t) + 8);
  __shared__ int abort_flag;
  __shared__ int n_issued;
  __shared__ uint32_t tmem_slot;
  __shared__ float s_mx[2][64];  // half-row maxima of the two warps that share a row set
  __shared__ float s_l[2][64];   // and, at the end, their shares of the row sums

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const eb_attn_item item = p.items[blockIdx.x];
  const int kvh = blockIdx.y;
  const int seq = item.seq;
  const int slot = p.seq_slots[seq];
  const int L = p.ctx_lens[seq];
  const int q0 = p.q_off[seq];
  const int ql = p.q_off[seq + 1] - q0;
  int n_pages = item.page_end - item.page_begin;
  if (n_pages > kMaxItemPages) {
    if (tid == 0) atomicOr(p.status, EB_DEV_BAD_INDEX);
    n_pages = kMaxItemPages;
  }
  for (int j = tid; j < n_pages; j += kV64Threads) {
    int32_t id = p.block_tables[(int64_t)slot * p.bt_stride + item.page_begin + j];
    if (id < 0 || id >= p.num_pages) {
      atomicOr(p.status, EB_DEV_BAD_INDEX);
      id = 0;
    }
    page_ids[j] = id;
  }
  const uint32_t bar_full = smem_u32(&bars[0]), bar_empty = smem_u32(&bars[NS]);
  const uint32_t bar_s = smem_u32(&bars[2 * NS]), bar_p = bar_s + 16, bar_pv = bar_s + 32, bar_o = bar_s + 48;  // [2] each
  const int q_rows = ql * G;                 // real query rows
  const int n_act = (q_rows + 15) / 16;      // row sets (16 rows, two softmax warps each) that hold real rows
  if (tid == 0) {
    abort_flag = 0;
    n_issued = 0;
    for (int i = 0; i < NS; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_s + 8 * i, 1);
      mbar_init(bar_p + 8 * i, (uint32_t)(2 * n_act));
      mbar_init(bar_pv + 8 * i, 1);
    }
    mbar_init(bar_o, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 8) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(kCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (warp < 8) {
    // the Q tile with the 128-byte swizzle a TMA copy would apply; rows past the real ones are zero
    for (int i = tid; i < 64 * 8; i += 256) {
      const int r = i >> 3, c = i & 7;
      const int qi = r / G, g = r - qi * G;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (qi < ql) {
        const uint32_t* src = reinterpret_cast<const uint32_t*>(p.q + (int64_t)(q0 + qi) * p.q_stride +
                                                                (int64_t)(kvh * G + g) * kHeadDim + c * 8);
        v = make_uint4(src[0], src[1], src[2], src[3]);
      }
      *reinterpret_cast<uint4*>(sm + r * 128 + ((c ^ (r & 7)) << 4)) = v;
    }
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t tO = tmem + 128;
  const int n_blk = (n_pages + kV64Pages - 1) / kV64Pages;   // stages of 128 keys
  const int n_sub = (n_pages + kV64Pages / 2 - 1) / (kV64Pages / 2);  // sub-blocks of 64 keys
  const int page_rows = 2 * vp.n_kv * kPage;

  if (warp == 8) {
    // ---------------- producer
    if (lane == 0) {
      for (int blk = 0; blk < n_blk; ++blk) {
        const int sidx = blk % NS;
        if (blk >= NS && !mbar_wait(bar_empty + 8 * sidx, ((blk / NS) - 1) & 1, &abort_flag, p.status, p.wait_tries)) break;
        const uint32_t full = bar_full + 8 * sidx;
        mbar_arrive_expect_tx(full, (uint32_t)kV64Stage);
        const uint32_t sb = stage0 + sidx * kV64Stage;
        for (int j = 0; j < kV64Pages; ++j) {
          const int pl = min(blk * kV64Pages + j, n_pages - 1);  // a block's missing pages repeat the last one (masked below)
          const int row = page_ids[pl] * page_rows;
          tma_load_2d(sb + j * 2048, &tmap, 0, row + kvh * kPage, full);
          tma_load_2d(sb + kV64Keys * 128 + j * 2048, &tmap, 0, row + (vp.n_kv + kvh) * kPage, full);
        }
        n_issued = blk + 1;
      }
    }
  } else if (warp == 9) {
    // ---------------- MMA issuer: S of sub-block i + 2 follows P V of sub-block i into the same 64 columns, so the
    // products of one sub-block run while the softmax warps work on the next
    if (lane == 0) {
      constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(64 >> 4) << 24);
      // P V as a 128-row product: lanes 32 w .. 32 w + 15 of P hold the heads, lanes 32 w + 16 .. 32 w + 31 the remainders
      constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(kHeadDim >> 3) << 17) |
                                   ((uint32_t)(128 >> 4) << 24);
      const uint64_t dq = tc_desc_sw128(q_addr);
      auto issue_s = [&](int i) -> bool {
        const int blk = i >> 1, sidx = blk % NS;
        if ((i & 1) == 0) {
          if (!mbar_wait(bar_full + 8 * sidx, (blk / NS) & 1, &abort_flag, p.status, p.wait_tries)) return false;
          tc_fence_after();
        }
        const uint64_t dk = tc_desc_sw128(stage0 + sidx * kV64Stage + (i & 1) * 8192);
#pragma unroll
        for (int k = 0; k < 4; ++k) tc_mma_ss(tmem + (i & 1) * 64, dq + 2 * k, dk + 2 * k, idesc_s, k > 0 ? 1u : 0u);
        tc_commit(bar_s + 8 * (i & 1));
        return true;
      };
      bool ok = issue_s(0);
      if (ok && n_sub > 1) ok = issue_s(1);
      for (int i = 0; i < n_sub && ok; ++i) {
        const int b = i & 1, blk = i >> 1, sidx = blk % NS;
        if (!mbar_wait(bar_p + 8 * b, (i >> 1) & 1, &abort_flag, p.status, p.wait_tries)) break;
        tc_fence_after();
        const uint32_t vb = stage0 + sidx * kV64Stage + kV64Keys * 128 + b * 8192;
        const uint32_t tP = tmem + b * 64;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)  // 16 keys per instruction
          tc_mma_ts(tO, tP + kk * 8, tc_desc_sw128(vb + kk * 2048), idesc_o, (i > 0 || kk > 0) ? 1u : 0u);
        if (i + 2 >= n_sub) tc_commit(bar_pv + 8 * b);  // otherwise S of sub-block i + 2, issued below, signals this product too
        if (b == 1 || i + 1 == n_sub) tc_commit(bar_empty + 8 * sidx);  // the stage's last sub-block has read its V rows
        if (i + 1 == n_sub) tc_commit(bar_o);
        if (i + 2 < n_sub) ok = issue_s(i + 2);
      }
    }
  } else if ((warp & 3) < n_act) {
    // ---------------- softmax of rows 16 w .. 16 w + 15, keys 32 kh .. 32 kh + 31 of every sub-block
    const int w = warp & 3, kh = warp >> 2;
    const int quad = lane >> 2, qc = lane & 3;
    const int r_lo = 16 * w + quad, r_hi = r_lo + 8;
    const bool hi_on = 16 * w + 8 < q_rows;  // warp-uniform: the upper eight rows hold real rows
    const bool ok_lo = r_lo < q_rows, ok_hi = r_hi < q_rows;
    const int qi_lo = ok_lo ? r_lo / G : 0, qi_hi = ok_hi ? r_hi / G : 0;
    const int pq_lo = L - ql + qi_lo, pq_hi = L - ql + qi_hi;  // absolute positions of the rows' queries
    const int lw_lo = p.window > 0 ? pq_lo - p.window + 1 : 0, lw_hi = p.window > 0 ? pq_hi - p.window + 1 : 0;
    const int t_end = item.page_end * kPage;
    const uint32_t t_lane = (uint32_t)(32 * w) << 16;
    float m_lo = kNegBig, m_hi = kNegBig;
    float l_lo = 0.f, l_hi = 0.f;  // this thread's share of the rows' sums (its keys of every sub-block)
    bool ok = true;
    for (int i = 0; i < n_sub; ++i) {
      const int b = i & 1;
      const uint32_t tS = tmem + b * 64;
      if (!mbar_wait(bar_s + 8 * b, (i >> 1) & 1, &abort_flag, p.status, p.wait_tries)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t sv[16];
      tc_ld_16x256b_x4(tS + t_lane + kh * 32, sv);
      const int t0 = (item.page_begin + i * (kV64Pages / 2)) * kPage;
      // only sub-blocks at the ends of the visible range need the causal / window / end-of-item mask (CTA-uniform test)
      const bool edge = (t0 + 63 > L - ql) || (p.window > 0 && t0 < L - p.window) || (t0 + 64 > t_end);
      if (edge) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int t = t0 + kh * 32 + 8 * j + 2 * qc + e;
            if (t > pq_lo || t < lw_lo || t >= t_end) sv[4 * j + e] = __float_as_uint(-INFINITY);
            if (t > pq_hi || t < lw_hi || t >= t_end) sv[4 * j + 2 + e] = __float_as_uint(-INFINITY);
          }
      }
      float mx_lo, mx_hi = -INFINITY;
      {
        float ta[2], tb[2];  // independent partial maxima, then a tree
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          ta[j] = fmaxf(fmaxf(__uint_as_float(sv[8 * j]), __uint_as_float(sv[8 * j + 1])),
                        fmaxf(__uint_as_float(sv[8 * j + 4]), __uint_as_float(sv[8 * j + 5])));
          tb[j] = fmaxf(fmaxf(__uint_as_float(sv[8 * j + 2]), __uint_as_float(sv[8 * j + 3])),
                        fmaxf(__uint_as_float(sv[8 * j + 6]), __uint_as_float(sv[8 * j + 7])));
        }
        mx_lo = fmaxf(ta[0], ta[1]);
        if (hi_on) mx_hi = fmaxf(tb[0], tb[1]);
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      // The other warp of the row set holds the other 32 keys: exchange the maxima so that both take the same decision.
      // The barrier also orders this warp's stores of P behind the partner's loads of S (P overwrites both warps' columns),
      // and the next write of these slots follows the partner's read: it comes two arrivals of both warps later.
      if (qc == 0) {
        s_mx[kh][r_lo] = mx_lo;
        s_mx[kh][r_hi] = mx_hi;
      }
      asm volatile("bar.sync %0, 64;" ::"r"(1 + w) : "memory");
      mx_lo = fmaxf(mx_lo, s_mx[kh ^ 1][r_lo]);
      mx_hi = fmaxf(mx_hi, s_mx[kh ^ 1][r_hi]);
      const float mb_lo = mx_lo * p.scale_log2, mb_hi = mx_hi * p.scale_log2;
      // raise a row's reference maximum only when a score exceeds it by 2^8 (always on the first finite one)
      const bool raise_lo = mb_lo > m_lo + 8.0f, raise_hi = mb_hi > m_hi + 8.0f;
      if (__any_sync(0xffffffffu, raise_lo || raise_hi)) {
        const float n_lo = raise_lo ? mb_lo : m_lo, n_hi = raise_hi ? mb_hi : m_hi;
        const float a_lo = fast_exp2(m_lo - n_lo), a_hi = fast_exp2(m_hi - n_hi);
        m_lo = n_lo;
        m_hi = n_hi;
        l_lo *= a_lo;
        l_hi *= a_hi;
        if (i > 0) {
          // O holds earlier sub-blocks; the product of the last one may still run: wait for it, then each warp rescales
          // its half of the columns
          // (S of sub-block i + 1 was issued after that product, so its arrival covers it; the last two products of an
          // item, which no S follows, arrive on a barrier of their own)
          const bool done = (i + 1 < n_sub) ? mbar_wait(bar_s + 8 * ((i + 1) & 1), ((i + 1) >> 1) & 1, &abort_flag, p.status, p.wait_tries)
                                            : mbar_wait(bar_pv + 8 * ((i - 1) & 1), 0, &abort_flag, p.status, p.wait_tries);
          if (!done) {
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int part = 0; part < 2; ++part) {  // the heads' product, then the remainders'
            const uint32_t ta = tO + t_lane + ((uint32_t)(16 * part) << 16) + kh * 32;
            uint32_t ov[16];
            tc_ld_16x256b_x4(ta, ov);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              ov[4 * j] = __float_as_uint(__uint_as_float(ov[4 * j]) * a_lo);
              ov[4 * j + 1] = __float_as_uint(__uint_as_float(ov[4 * j + 1]) * a_lo);
              ov[4 * j + 2] = __float_as_uint(__uint_as_float(ov[4 * j + 2]) * a_hi);
              ov[4 * j + 3] = __float_as_uint(__uint_as_float(ov[4 * j + 3]) * a_hi);
            }
            tc_st_16x256b_x4(ta, ov);
          }
          tc_wait_st();
        }
      }
      // P = 2^(s * scale - m), written over S, two keys per column (columns 0..31 of the buffer): the bf16 heads in the
      // rows' own lanes, the bf16 remainders 16 lanes up, which the 64-row product S never touches.  The steps are written as separate passes over the thread's 16 values so that independent instructions
      // follow each other (a warp has little else to hide an exponential's latency behind).
      float ev[16];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        ev[4 * j] = fmaf(__uint_as_float(sv[4 * j]), p.scale_log2, -m_lo);
        ev[4 * j + 1] = fmaf(__uint_as_float(sv[4 * j + 1]), p.scale_log2, -m_lo);
        ev[4 * j + 2] = fmaf(__uint_as_float(sv[4 * j + 2]), p.scale_log2, -m_hi);
        ev[4 * j + 3] = fmaf(__uint_as_float(sv[4 * j + 3]), p.scale_log2, -m_hi);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        ev[4 * j] = fast_exp2(ev[4 * j]);
        ev[4 * j + 1] = fast_exp2(ev[4 * j + 1]);
        if (hi_on) {
          ev[4 * j + 2] = fast_exp2(ev[4 * j + 2]);
          ev[4 * j + 3] = fast_exp2(ev[4 * j + 3]);
        }
      }
      uint32_t ph[8], pl[8];  // registers 2 j, 2 j + 1: rows lane/4 and lane/4 + 8 of key group j
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        ph[2 * j] = pack_bf16(ev[4 * j], ev[4 * j + 1]);
        ph[2 * j + 1] = hi_on ? pack_bf16(ev[4 * j + 2], ev[4 * j + 3]) : 0u;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        pl[2 * j] = pack_bf16(ev[4 * j] - __uint_as_float(ph[2 * j] << 16), ev[4 * j + 1] - __uint_as_float(ph[2 * j] & 0xFFFF0000u));
        pl[2 * j + 1] = hi_on ? pack_bf16(ev[4 * j + 2] - __uint_as_float(ph[2 * j + 1] << 16),
                                          ev[4 * j + 3] - __uint_as_float(ph[2 * j + 1] & 0xFFFF0000u))
                              : 0u;
      }
      l_lo += (ev[0] + ev[1]) + (ev[4] + ev[5]) + ((ev[8] + ev[9]) + (ev[12] + ev[13]));
      if (hi_on) l_hi += (ev[2] + ev[3]) + (ev[6] + ev[7]) + ((ev[10] + ev[11]) + (ev[14] + ev[15]));
      tc_st_16x128b_x4(tS + t_lane + kh * 16, ph);
      tc_st_16x128b_x4(tS + t_lane + (16u << 16) + kh * 16, pl);
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p + 8 * b);
    }
    // ---------------- epilogue: this warp's 32 columns of the rows of O; the row sums are added over the quad and the
    // two warps of the row set (both warps pass the barrier: a failed wait above has raised the abort flag for all)
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    if (qc == 0) {
      s_l[kh][r_lo] = l_lo;
      s_l[kh][r_hi] = l_hi;
    }
    asm volatile("bar.sync %0, 64;" ::"r"(1 + w) : "memory");
    l_lo = s_l[0][r_lo] + s_l[1][r_lo];
    l_hi = s_l[0][r_hi] + s_l[1][r_hi];
    if (ok && n_sub > 0 && mbar_wait(bar_o, 0, &abort_flag, p.status, p.wait_tries)) {
      tc_fence_after();
      const int n_parts_seq = p.seq_part[seq + 1] - p.seq_part[seq];
      const bool direct = (n_parts_seq == 1);
      // partial slots [item.part, item.part + ppi) must lie inside the scratch; otherwise skip and flag
      const bool part_ok = direct || (item.part >= 0 && item.part + vp.ppi <= p.part_slots);
      if (!part_ok && lane == 0 && kh == 0) atomicOr(p.status, EB_DEV_BAD_INDEX);
      uint32_t ov[16];
      tc_ld_16x256b_x4(tO + t_lane + kh * 32, ov);
      {  // O = P_head V + P_remainder V
        uint32_t o2[16];
        tc_ld_16x256b_x4(tO + t_lane + (16u << 16) + kh * 32, o2);
#pragma unroll
        for (int j = 0; j < 16; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) + __uint_as_float(o2[j]));
      }
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const bool row_ok = half ? ok_hi : ok_lo;
        if (!(row_ok && part_ok)) continue;
        const int r = half ? r_hi : r_lo, qi = half ? qi_hi : qi_lo;
        const int head = kvh * G + (r - qi * G);
        const float m_row = half ? m_hi : m_lo, l_row = half ? l_hi : l_lo;
        if (direct) {
          const float sk = p.sinks[head] * 1.4426950408889634f;
          const float mf = fmaxf(m_row, sk);
          const float wgt = exp2f(m_row - mf);
          const float inv = wgt / (l_row * wgt + exp2f(sk - mf));
          uint32_t* orow = reinterpret_cast<uint32_t*>(p.out + (int64_t)(q0 + qi) * p.out_stride + (int64_t)head * kHeadDim) + kh * 16;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            orow[4 * j + qc] = pack_bf16(__uint_as_float(ov[4 * j + 2 * half]) * inv, __uint_as_float(ov[4 * j + 2 * half + 1]) * inv);
        } else {
          const int64_t prow = ((int64_t)item.part * p.max_q_len + qi) * p.n_q + head;
          float2* arow = reinterpret_cast<float2*>(p.part_acc + prow * kHeadDim) + kh * 16;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            arow[4 * j + qc] = make_float2(__uint_as_float(ov[4 * j + 2 * half]), __uint_as_float(ov[4 * j + 2 * half + 1]));
          if (qc == 0 && kh == 0) *reinterpret_cast<float2*>(p.part_ml + prow * 2) = make_float2(m_row, l_row);
          // the plan reserves vp.ppi partial slots per item; this kernel fills one, the others are declared empty (a sum of
          // zero: the merge skips such a slot without reading its accumulator, which is left as it was)
          for (int e = 1; e < vp.ppi; ++e) {
            const int64_t pe = ((int64_t)(item.part + e) * p.max_q_len + qi) * p.n_q + head;
            if (qc == 0 && kh == 0) *reinterpret_cast<float2*>(p.part_ml + pe * 2) = make_float2(kNegBig, 0.f);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (abort_flag && tid == 0) {
    // A wait gave up.  Before the CTA releases its shared memory, wait (bounded) for the copies still in flight.
    const int issued = n_issued;
    for (int blk = max(0, issued - NS); blk < issued; ++blk) {
      const uint32_t bar = bar_full + 8 * (blk % NS);
      for (uint32_t i = 0; i < kWaitTries; ++i) {
        if (mbar_try_wait(bar, (blk / NS) & 1)) break;
        __nanosleep(64);
      }
    }
  }
  __syncthreads();
  if (warp == 8) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kCols) : "memory");
}

// Combine the split-K partials of one (sequence, KV group): warp = query head, lane = two dims.
__global__ void __launch_bounds__(256) attn_merge_kernel(const AttnParams p) {
  eb::pdl_wait();  // programmatic dependent launch: the predecessor in the stream has completed
  eb::pdl_trigger();
  const int seq = blockIdx.x;
  const int pb = p.seq_part[seq], pe = p.seq_part[seq + 1];
  if (pe - pb <= 1) return;  // written directly by attn_kernel
  if (pb < 0 || pe > p.part_slots) {  // partial range outside the scratch: leave the output alone and flag it
    if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(p.status, EB_DEV_BAD_INDEX);
    return;
  }
  const int head = blockIdx.y * 8 + (threadIdx.x >> 5);
  if (head >= p.n_q) return;
  const int lane = threadIdx.x & 31;
  const int q0 = p.q_off[seq], ql = p.q_off[seq + 1] - q0;
  const float sk = p.sinks[head] * 1.4426950408889634f;
  for (int qi = 0; qi < ql; ++qi) {
    float mf = sk;
    for (int j = pb + lane; j < pe; j += 32) {
      const int64_t row = ((int64_t)j * p.max_q_len + qi) * p.n_q + head;
      mf = fmaxf(mf, p.part_ml[row * 2]);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) mf = fmaxf(mf, __shfl_xor_sync(0xffffffffu, mf, o));
    float den = exp2f(sk - mf);
    float ax = 0.f, ay = 0.f;
    // partials in ascending order, 32 at a time: lane k holds (m, l) of partial base + k; the ones with an empty sum (no
    // visible key, or a slot its kernel did not use) are passed over without touching their accumulators
    for (int base = pb; base < pe; base += 32) {
      const int jl = base + lane;
      float2 ml = make_float2(kNegBig, 0.f);
      if (jl < pe) ml = *reinterpret_cast<const float2*>(p.part_ml + (((int64_t)jl * p.max_q_len + qi) * p.n_q + head) * 2);
      unsigned live = __ballot_sync(0xffffffffu, ml.y != 0.f);
      while (live) {
        const int k = __ffs(live) - 1;
        live &= live - 1;
        const float w = exp2f(__shfl_sync(0xffffffffu, ml.x, k) - mf);
        den += w * __shfl_sync(0xffffffffu, ml.y, k);
        const int64_t row = ((int64_t)(base + k) * p.max_q_len + qi) * p.n_q + head;
        const float2 a = *reinterpret_cast<const float2*>(p.part_acc + row * kHeadDim + lane * 2);
        ax += w * a.x;
        ay += w * a.y;
      }
    }
    const float inv = 1.0f / den;
    uint16_t* orow = p.out + (int64_t)(q0 + qi) * p.out_stride + (int64_t)head * kHeadDim;
    *reinterpret_cast<uint32_t*>(orow + lane * 2) = pack_bf16(ax * inv, ay * inv);
  }
}

// One thread per 16-byte chunk of a new K or V row.
__global__ void kv_append_kernel(uint4* cache, int32_t num_pages, int32_t n_kv, const uint4* k_new, const uint4* v_new,
                                 int64_t row_stride16, const int32_t* block_tables, int32_t bt_stride,
                                 const int32_t* tok_slot, const int32_t* positions, int32_t n_tokens, int32_t* status) {
  eb::pdl_wait();  // programmatic dependent launch: the predecessor in the stream has completed
  eb::pdl_trigger();
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int chunks_per_tok = 2 * n_kv * 8;  // K and V, 8 chunks of 16 bytes per head row
  if (idx >= (int64_t)n_tokens * chunks_per_tok) return;
  const int t = (int)(idx / chunks_per_tok);
  const int r = (int)(idx % chunks_per_tok);
  const int kv = r / (n_kv * 8), h = (r / 8) % n_kv, c = r % 8;
  const int pos = positions[t];
  const int32_t page = block_tables[(int64_t)tok_slot[t] * bt_stride + pos / kPage];
  if (page < 0 || page >= num_pages || pos < 0) {
    atomicOr(status, EB_DEV_BAD_INDEX);
    return;
  }
  const uint4* src = (kv ? v_new : k_new) + (int64_t)t * row_stride16 + h * 8 + c;
  // page = 2*n_kv head blocks of 16 rows of 8 chunks
  uint4* dst = cache + (((int64_t)page * 2 * n_kv + kv * n_kv + h) * kPage + pos % kPage) * 8 + c;
  *dst = *src;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

template <int MT, int WT, int HKV, int STAGES, int G>
int32_t launch_attn(const CUtensorMap& tm, const AttnParams& p, int n_items, cudaStream_t st) {
  const size_t smem = 1024 + (size_t)STAGES * kStageBytes + 2 * STAGES * sizeof(uint64_t) + kMaxItemPages * sizeof(int32_t);
  auto kfn = attn_kernel<MT, WT, HKV, STAGES, G>;
  static bool configured[64] = {false};  // the attribute is per device
  int dev = 0;
  EB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    EB_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  EB_CUDA(eb::launch(kfn, dim3(n_items), dim3((kComputeWarps * WT + 1) * 32), smem, st, tm, p));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

// Verify shapes on tcgen05 with 64-row tiles: grid = (items, KV heads), two CTAs per SM.
template <int G>
int32_t launch_attn_v64(EncodeTiledFn enc, const void* d_cache, int64_t cache_rows, const AttnParams& p, int n_items, int n_kv,
                        cudaStream_t st) {
  CUtensorMap tm;  // the cache as rows of 128 bytes; a copy is the 16 rows (tokens) of one head's K or V in one page
  const cuuint64_t gdim[2] = {(cuuint64_t)kHeadDim, (cuuint64_t)cache_rows};
  const cuuint64_t gstr[1] = {128};
  const cuuint32_t box[2] = {(cuuint32_t)kHeadDim, (cuuint32_t)kPage};
  const cuuint32_t estr[2] = {1, 1};
  CUresult cr = enc(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(d_cache), gdim, gstr, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  EB_REQUIRE(cr == CUDA_SUCCESS, EB_ERR_ARG, "attention: cuTensorMapEncodeTiled failed (%d)", (int)cr);
  V64Params vp;
  vp.n_kv = n_kv;
  vp.ppi = 8 / n_kv;
  const size_t smem = 1024 + 8192 + (size_t)kV64Stages * kV64Stage + (2 * kV64Stages + 7) * sizeof(uint64_t) + 8 +
                      kMaxItemPages * sizeof(int32_t);
  auto kfn = attn_v64_kernel<G>;
  static bool configured[64] = {false};  // the attribute is per device
  int dev = 0;
  EB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    EB_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  EB_CUDA(eb::launch(kfn, dim3((unsigned)n_items, (unsigned)n_kv), dim3(kV64Threads), smem, st, tm, p, vp));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

// Verify shapes (17..48 query rows per KV head) run on the tcgen05 kernel when the work items are long: full-attention
// layers, or windows of 2048 tokens and more.  Measured on 256 ragged sequences at q_len 5: 332 us against 526 us for
// the mma.sync kernel on full layers, but 66 us against 47 us on a 128-token window, whose items are two or three
// 64-key sub-blocks long.  EIDOLA_B200_ATTN_VERIFY=mma keeps every shape on the mma.sync kernel (read on every call so
// that a test can compare the two).
bool attn_verify_on_tcgen05(int window) {
  const char* v = getenv("EIDOLA_B200_ATTN_VERIFY");
  if (v && v[0] == 'm') return false;
  return window == 0 || window >= 2048;
}

template <int WT, int G>
int32_t dispatch_hkv(int n_kv, const CUtensorMap& tm, const AttnParams& p, int n_items, cudaStream_t st) {
  constexpr int ST = (WT == 1) ? 3 : 6;
  switch (n_kv) {
    case 8: return launch_attn<1, WT, 8, ST, G>(tm, p, n_items, st);
    case 4: return launch_attn<1, WT, 4, ST, G>(tm, p, n_items, st);
    case 2: return launch_attn<1, WT, 2, ST, G>(tm, p, n_items, st);
    case 1: return launch_attn<1, WT, 1, ST, G>(tm, p, n_items, st);
  }
  return eb::fail(EB_ERR_UNSUPPORTED, "attention: n_kv %d not in {1,2,4,8}", n_kv);
}

}  // namespace

extern "C" {

int32_t eb_kv_append(void* d_cache, int32_t num_pages, int32_t n_kv, int32_t head_dim, int32_t page_size,
                     const void* d_k_new, const void* d_v_new, int64_t row_stride, const int32_t* d_block_tables,
                     int32_t bt_stride, const int32_t* d_tok_slot, const int32_t* d_positions, int32_t n_tokens,
                     void* stream) {
  EB_REQUIRE(d_cache && d_k_new && d_v_new && d_block_tables && d_tok_slot && d_positions, EB_ERR_ARG,
             "eb_kv_append: null pointer");
  EB_REQUIRE(head_dim == kHeadDim && page_size == kPage, EB_ERR_UNSUPPORTED,
             "eb_kv_append: head_dim %d / page_size %d (built for 64 / 16)", head_dim, page_size);
  EB_REQUIRE(n_kv >= 1 && num_pages >= 1 && n_tokens >= 0 && bt_stride >= 1, EB_ERR_ARG, "eb_kv_append: bad size");
  EB_REQUIRE(row_stride >= (int64_t)n_kv * head_dim && row_stride % 8 == 0, EB_ERR_ARG,
             "eb_kv_append: row stride %lld (needs >= %d, multiple of 8)", (long long)row_stride, n_kv * head_dim);
  EB_REQUIRE(((uintptr_t)d_k_new % 16 == 0) && ((uintptr_t)d_v_new % 16 == 0) && ((uintptr_t)d_cache % 16 == 0),
             EB_ERR_ARG, "eb_kv_append: pointers must be 16-byte aligned");
  if (n_tokens == 0) return EB_OK;
  int32_t* status = eb::status_word();
  EB_REQUIRE(status, EB_ERR_NODEVICE, "eb_kv_append: no device");
  const int64_t total = (int64_t)n_tokens * 2 * n_kv * 8;
  EB_CUDA(eb::launch(kv_append_kernel, dim3((unsigned)eb::cdiv(total, 256)), dim3(256), 0, eb::as_stream(stream), 
      (uint4*)d_cache, num_pages, n_kv, (const uint4*)d_k_new, (const uint4*)d_v_new, row_stride / 8, d_block_tables,
      bt_stride, d_tok_slot, d_positions, n_tokens, status));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_attn_workspace(int32_t n_parts, int32_t max_q_len, int32_t n_q, int32_t head_dim, size_t* acc_bytes,
                          size_t* ml_bytes) {
  EB_REQUIRE(acc_bytes && ml_bytes && n_parts >= 0 && max_q_len >= 1 && n_q >= 1 && head_dim >= 1, EB_ERR_ARG,
             "eb_attn_workspace: bad argument");
  const size_t rows = (size_t)n_parts * max_q_len * n_q;
  *acc_bytes = rows * head_dim * sizeof(float);
  *ml_bytes = rows * 2 * sizeof(float);
  return EB_OK;
}

}  // extern "C"

namespace {

// Validation, tensor map, dispatch and merge shared by eb_attn_paged_sink and eb_attn_paged_sink_static: the two entry
// points differ only in whose memory holds the split-K partials and the status word.  `who` names the entry point in
// messages.  part_acc / part_ml hold a->n_parts partial slots.
int32_t run_attn(const eb_attn_args* a, float* part_acc, float* part_ml, int32_t* status, const char* who, void* stream) {
  EB_REQUIRE(a->d_q && a->d_out && a->d_cache && a->d_block_tables && a->d_seq_slots && a->d_q_off && a->d_ctx_lens &&
                 a->d_sinks && a->d_items && a->d_seq_part,
             EB_ERR_ARG, "%s: null pointer", who);
  EB_REQUIRE(a->head_dim == kHeadDim && a->page_size == kPage, EB_ERR_UNSUPPORTED, "%s: head_dim %d / page_size %d (built for 64 / 16)",
             who, a->head_dim, a->page_size);
  EB_REQUIRE(a->n_kv >= 1 && (a->n_q == a->n_kv * 8 || a->n_q == a->n_kv * 4), EB_ERR_UNSUPPORTED,
             "%s: %d query heads over %d KV heads (built for groups of 8 or 4)", who, a->n_q, a->n_kv);
  const int group = a->n_q / a->n_kv;
  EB_REQUIRE(a->max_q_len >= 1 && a->max_q_len * group <= 48, EB_ERR_UNSUPPORTED, "%s: max_q_len %d exceeds %d", who, a->max_q_len,
             48 / group);
  EB_REQUIRE(a->n_seqs >= 0 && a->n_items >= 0 && a->n_parts >= 0 && a->num_pages >= 1 && a->window >= 0, EB_ERR_ARG,
             "%s: negative size", who);
  EB_REQUIRE(a->q_stride % 2 == 0 && a->out_stride % 2 == 0 && (uintptr_t)a->d_q % 4 == 0 && (uintptr_t)a->d_out % 4 == 0,
             EB_ERR_ARG, "%s: q/out must be 4-byte aligned with even strides", who);
  EB_REQUIRE((uintptr_t)a->d_cache % 16 == 0, EB_ERR_ARG, "%s: cache must be 16-byte aligned", who);
  EB_REQUIRE(a->n_parts == 0 || (part_acc && part_ml), EB_ERR_ARG, "%s: null workspace", who);
  EB_REQUIRE(status, EB_ERR_NODEVICE, "%s: no device status word", who);
  if (a->n_seqs == 0 || a->n_items == 0) return EB_OK;
  const int64_t rows = (int64_t)a->num_pages * 2 * a->n_kv * kPage;
  EB_REQUIRE(rows < (1ll << 31), EB_ERR_UNSUPPORTED, "%s: cache of %lld rows exceeds a tensor map", who, (long long)rows);

  EncodeTiledFn enc = encode_tiled_fn();
  EB_REQUIRE(enc, EB_ERR_NODEVICE, "%s: driver entry point cuTensorMapEncodeTiled not found", who);
  CUtensorMap tm;
  const cuuint64_t gdim[2] = {(cuuint64_t)kHeadDim, (cuuint64_t)rows};
  const cuuint64_t gstr[1] = {128};
  const cuuint32_t box[2] = {(cuuint32_t)kHeadDim, (cuuint32_t)(2 * a->n_kv * kPage)};
  const cuuint32_t estr[2] = {1, 1};
  CUresult cr = enc(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(a->d_cache), gdim, gstr, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  EB_REQUIRE(cr == CUDA_SUCCESS, EB_ERR_ARG, "%s: cuTensorMapEncodeTiled failed (%d)", who, (int)cr);

  AttnParams p;
  p.q = (const uint16_t*)a->d_q;
  p.q_stride = a->q_stride;
  p.out = (uint16_t*)a->d_out;
  p.out_stride = a->out_stride;
  p.block_tables = a->d_block_tables;
  p.bt_stride = a->bt_stride;
  p.seq_slots = a->d_seq_slots;
  p.q_off = a->d_q_off;
  p.ctx_lens = a->d_ctx_lens;
  p.sinks = a->d_sinks;
  p.window = a->window;
  p.n_q = a->n_q;
  p.max_q_len = a->max_q_len;
  p.num_pages = a->num_pages;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.items = a->d_items;
  p.seq_part = a->d_seq_part;
  p.part_acc = part_acc;  // every partial row that the merge reads is written by this launch first: nothing to clear
  p.part_ml = part_ml;
  p.part_slots = a->n_parts;
  p.wait_tries = eb::wait_tries();
  p.status = status;

  cudaStream_t st = eb::as_stream(stream);
  const int mt = (a->max_q_len * group + 15) / 16;
  int32_t rc;
  if (mt >= 2 && attn_verify_on_tcgen05(a->window)) {
    rc = group == 8 ? launch_attn_v64<8>(enc, a->d_cache, rows, p, a->n_items, a->n_kv, st)
                    : launch_attn_v64<4>(enc, a->d_cache, rows, p, a->n_items, a->n_kv, st);
  } else if (group == 8) {
    if (mt == 1)
      rc = dispatch_hkv<1, 8>(a->n_kv, tm, p, a->n_items, st);
    else if (mt == 2)
      rc = dispatch_hkv<2, 8>(a->n_kv, tm, p, a->n_items, st);
    else
      rc = dispatch_hkv<3, 8>(a->n_kv, tm, p, a->n_items, st);
  } else {
    if (mt == 1)
      rc = dispatch_hkv<1, 4>(a->n_kv, tm, p, a->n_items, st);
    else if (mt == 2)
      rc = dispatch_hkv<2, 4>(a->n_kv, tm, p, a->n_items, st);
    else
      rc = dispatch_hkv<3, 4>(a->n_kv, tm, p, a->n_items, st);
  }
  if (rc != EB_OK) return rc;
  if (a->n_parts > a->n_seqs) {  // at least one sequence has more than one partial
    EB_CUDA(eb::launch(attn_merge_kernel, dim3((unsigned)a->n_seqs, (unsigned)((a->n_q + 7) / 8)), dim3(256), 0, st, p));
    EB_LAUNCH_CHECK();
  }
  return EB_OK;
}

// ---------------------------------------------------------------------------------------------
// Scratch of the entry point for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc where they need attention: a host that has handed all device
// memory to its own pool, a plugin that runs inside another runtime's allocator arena, a latency-critical thread
// that must not take the allocator's lock.  For them the split-K scratch (partial accumulators and their
// (max, sum) pairs) lives in the two file-scope device arrays below, which every GPU that loads the library holds
// until the process exits (16.5 MiB together).  The caller still owns every input and output.

constexpr int64_t kStaticRows = 65536;  // (partial slot, query position, query head) rows the scratch can hold

static __device__ __align__(256) float g_static_part_acc[kStaticRows * kHeadDim];  // 16 MiB
static __device__ __align__(256) float g_static_part_ml[kStaticRows * 2];          // 512 KiB
static __device__ __align__(256) int32_t g_static_status[64];                       // status word when the caller passes none

struct StaticScratch {
  std::once_flag once;
  cudaError_t err = cudaErrorNotReady;
  float* acc = nullptr;
  float* ml = nullptr;
  int32_t* status = nullptr;
};
StaticScratch g_static_scratch[64];  // per device: in host code the array names above are only host-side stand-ins,
                                     // the device addresses come from cudaGetSymbolAddress with that device current

// Resolves the device addresses of the scratch arrays once per device (thread-safe), with that device current.
int32_t static_scratch(StaticScratch** out) {
  int dev = -1;
  EB_CUDA(cudaGetDevice(&dev));
  EB_REQUIRE(dev >= 0 && dev < 64, EB_ERR_UNSUPPORTED, "eb_attn_paged_sink_static: device ordinal %d", dev);
  StaticScratch& sc = g_static_scratch[dev];
  std::call_once(sc.once, [&sc] {
    cudaError_t e = cudaGetSymbolAddress((void**)&sc.acc, g_static_part_acc);
    if (e == cudaSuccess) e = cudaGetSymbolAddress((void**)&sc.ml, g_static_part_ml);
    if (e == cudaSuccess) e = cudaGetSymbolAddress((void**)&sc.status, g_static_status);
    sc.err = e;
  });
  if (sc.err != cudaSuccess)
    return eb::fail((int32_t)sc.err, "eb_attn_paged_sink_static: cudaGetSymbolAddress: %s", cudaGetErrorString(sc.err));
  *out = &sc;
  return EB_OK;
}

}  // namespace

namespace eb {
// The library's built-in status word of the current device when eb_attn_paged_sink_static has resolved it, else nullptr
// (eb_status_read folds it into what it reports).
int32_t* static_status_word_if_ready() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  StaticScratch& sc = g_static_scratch[dev];
  return sc.err == cudaSuccess ? sc.status : nullptr;
}
}  // namespace eb

extern "C" {

int32_t eb_attn_paged_sink(const eb_attn_args* a, void* stream) {
  EB_REQUIRE(a, EB_ERR_ARG, "eb_attn_paged_sink: null args");
  return run_attn(a, (float*)a->d_part_acc, (float*)a->d_part_ml, eb::status_word(), "eb_attn_paged_sink", stream);
}

int32_t eb_attn_paged_sink_static(const eb_attn_args* a, int32_t* d_status, void* stream) {
  EB_REQUIRE(a, EB_ERR_ARG, "eb_attn_paged_sink_static: null args");
  EB_REQUIRE(a->n_parts >= 0 && a->max_q_len >= 1 && a->n_q >= 1, EB_ERR_ARG, "eb_attn_paged_sink_static: negative size");
  const int64_t need_rows = (int64_t)a->n_parts * a->max_q_len * a->n_q;
  EB_REQUIRE(need_rows <= kStaticRows, EB_ERR_NOMEM,
             "eb_attn_paged_sink_static: %d partial slots x %d query positions x %d heads = %lld rows exceed the built-in "
             "scratch of %lld rows; plan with a larger chunk_pages or use eb_attn_paged_sink with a caller workspace",
             a->n_parts, a->max_q_len, a->n_q, (long long)need_rows, (long long)kStaticRows);
  // Set-up, once per device, with that device current: the device addresses of the scratch arrays.
  StaticScratch* sc = nullptr;
  int32_t rc = static_scratch(&sc);
  if (rc != EB_OK) return rc;
  return run_attn(a, sc->acc, sc->ml, d_status ? d_status : sc->status, "eb_attn_paged_sink_static", stream);
}

int32_t eb_attn_static_status_read(int32_t* status) {
  EB_REQUIRE(status, EB_ERR_ARG, "eb_attn_static_status_read: null");
  StaticScratch* sc = nullptr;
  int32_t rc = static_scratch(&sc);
  if (rc != EB_OK) return rc;
  EB_CUDA(cudaMemcpy(status, sc->status, sizeof(int32_t), cudaMemcpyDeviceToHost));
  EB_CUDA(cudaMemset(sc->status, 0, sizeof(int32_t)));
  return EB_OK;
}

}  // extern "C"

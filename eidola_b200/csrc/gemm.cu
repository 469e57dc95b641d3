// Block-scaled FP8 (e4m3) GEMM on the sm_100a tensor cores (tcgen05.mma, accumulators in tensor memory),
// dense and grouped (one weight matrix per expert), plus the activation quantiser that feeds it.
//
//   Y[m][n] = bf16( sum_kb sx[blk(m)][kb] * sw[n/128][kb] * sum_{k in kb} X8[m][k] * W8[n][k] )
//
// Decode-shaped: the weight tile is the M operand of the MMA (128 weight rows), the tokens are the N operand
// (TN = 16..128 columns), so a few tokens still fill a 128-wide instruction and every CTA streams a
// 128-row band of W exactly once.  One pipeline stage is one 128-byte K block of both operands (TMA, 128-byte
// swizzle) = one scale block: its four K=32 MMAs start a fresh accumulator in tensor memory, and four epilogue
// warps fold finished blocks into registers with acc += (sx*sw) * block while the tensor core works on the
// next block in the other accumulator buffer.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = tensor-memory owner and MMA issuer,
// warps 2..5 = epilogue (tensor-memory lane quarter = warp % 4).  All waits are bounded.
//
// The reference project has no GEMM (inference is delegated, crates/eidola-server/src/backend.rs:421-433).
#include <cuda.h>
#include <stdlib.h>

#include <algorithm>
#include <cuda_runtime.h>

#include "common.h"
#include "tmap.h"

namespace {

constexpr int kThreads = 192;
constexpr int kTileN = 128;       // weight rows per CTA (MMA M)
constexpr int kBlockK = 128;      // bytes = e4m3 elements per K block
constexpr int kMaxKB = 128;       // K blocks per GEMM (K <= 16384)
constexpr int kMaxSplitRows = 512;  // split K only for decode-sized activations
constexpr uint32_t kWaitTries = 1u << 22;

struct GemmParams {
  const float* sx;
  const float* sw;
  uint16_t* y;
  float* y_part;  // fp32 partials [splits][rows][N] when splits > 1
  int64_t ldy;
  int32_t rows, N, K, n_groups, splits;
  const int32_t* seg_off;     // grouped: [n_groups+1]
  const int32_t* blk_off;     // grouped: [n_groups+1]
  const int32_t* tile_group;  // grouped: [max_tiles]
  const int32_t* tile_row0;   // grouped: [max_tiles]
  const int32_t* n_tiles;     // grouped: device scalar
  int32_t* status;
  uint32_t wait_tries;  // polls a bounded wait makes before it gives up (eb_wait_limit_set)
  int32_t w_tiled;      // weights are stored as contiguous 16 KiB tiles (eb_weight_tile_fp8), not row-major
  const uint8_t* w8;    // the weights' address (for L2 prefetches of tiles; the pipeline itself loads through the tensor map)
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

// One pipeline stage of weights: 128 weight rows x one 128-byte K block of group g, weight-row block nb, K block kb.
// Row-major weights [groups][N][K]: a box of 128 rows, 2880 bytes apart in HBM.  Tiled weights
// [groups][ceil(N/128)][ceil(K/128)][128 rows][128 bytes] (eb_weight_tile_fp8): the same box is 16 KiB of consecutive
// bytes, which HBM serves at its streaming rate instead of 128 separate 128-byte bursts.
__device__ __forceinline__ void load_w_tile(uint32_t dst, const CUtensorMap* map, const GemmParams& p, int g, int nb, int kb,
                                            uint32_t bar) {
  if (p.w_tiled) {
    const int NBw = (p.N + kTileN - 1) / kTileN, KBw = (p.K + kBlockK - 1) / kBlockK;
    tma_load_2d(dst, map, 0, ((g * NBw + nb) * KBw + kb) * kTileN, bar);
  } else {
    tma_load_2d(dst, map, kb * kBlockK, g * p.N + nb * kTileN, bar);
  }
}

// ---- tcgen05 wrappers
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], e4m3 x e4m3 -> fp32, M=128, N from the instruction descriptor, K=32.
__device__ __forceinline__ void tc_mma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Shared-memory matrix descriptor: K-major rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(1024u >> 4) << 32;  // stride byte offset
  d |= (uint64_t)1 << 46;             // descriptor version of sm_100
  d |= (uint64_t)2 << 61;             // SWIZZLE_128B
  return d;
}
// 32 lanes x 16 consecutive 32-bit columns of tensor memory -> 16 registers per thread.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

template <int TN>
struct Cfg {
  static constexpr int kStageBytes = kTileN * kBlockK + TN * kBlockK;
  // two CTAs share an SM (one streams while the other starts up or drains): <= 113 KB of shared memory and
  // <= 256 tensor-memory columns each
  static constexpr int kStages = (TN == 128) ? 3 : (TN == 64) ? 4 : 5;
  static constexpr uint32_t kTmemCols = (2 * TN < 32) ? 32 : 2 * TN;
  static constexpr size_t kSmem = 1024 + (size_t)kStages * kStageBytes + 256 + kMaxKB * sizeof(float);
};

template <int TN>
__global__ void __launch_bounds__(kThreads, 2)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const GemmParams p) {
  // Programmatic dependent launch: this grid may start while its predecessor in the stream drains.  Everything up
  // to pdl_wait() touches no memory the predecessor writes: barriers, tensor memory and (dense mode) the first
  // stages' weight tiles, which no kernel of the step produces.
  eb::pdl_trigger();
  using C = Cfg<TN>;
  constexpr int S = C::kStages;
  const bool grouped = p.n_groups > 1 || p.seg_off;
  const int nb = blockIdx.y, n0 = nb * kTileN;
  const int KB = (p.K + kBlockK - 1) / kBlockK;
  const int NB = (p.N + kTileN - 1) / kTileN;
  const int split = blockIdx.z;
  const int kb_per = (KB + p.splits - 1) / p.splits;
  const int kb0 = split * kb_per, kb1 = min(KB, kb0 + kb_per);
  int nkb = max(0, kb1 - kb0);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t stage0 = (raw + 1023u) & ~1023u;
  uint8_t* after = smem_raw + (stage0 - raw) + S * C::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(after);  // full[S], empty[S], tfull[2], tempty[2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(after + (2 * S + 4) * sizeof(uint64_t));
  float* sprod = reinterpret_cast<float*>(after + 256);
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t bar_full = smem_u32(&bars[0]), bar_empty = smem_u32(&bars[S]);
  const uint32_t bar_tfull = smem_u32(&bars[2 * S]), bar_tempty = smem_u32(&bars[2 * S + 2]);

  int prefilled = 0;
  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (!grouped) {  // the weight half of the first stages, ahead of the predecessor's completion
      prefilled = min(S, nkb);
      for (int i = 0; i < prefilled; ++i) {
        mbar_arrive_expect_tx(bar_full + 8 * i, C::kStageBytes);
        load_w_tile(stage0 + i * C::kStageBytes, &tm_w, p, 0, nb, kb0 + i, bar_full + 8 * i);
      }
    }
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
  eb::pdl_wait();  // the predecessor in the stream has completed and its writes are visible

  // ---- which tile
  int g = 0, row0 = 0, row_end = 0, xblk = 0;
  if (grouped) {
    const int t = blockIdx.x;
    if (t < *p.n_tiles) {
      g = p.tile_group[t];
      row0 = p.tile_row0[t];
      row_end = p.seg_off[g + 1];
      xblk = p.blk_off[g] + (row0 - p.seg_off[g]) / 128;
    } else {
      nkb = 0;  // no such tile: fall through to the common exit
    }
  } else {
    row0 = blockIdx.x * TN;
    row_end = p.rows;
    xblk = row0 / 128;
  }
  if (tid == 0) {
    // Fill the pipeline before the rest of the CTA has finished setting up (scale products, the set-up barrier):
    // the first stages are in flight one barrier round trip earlier.
    if (grouped) {
      prefilled = min(S, nkb);
      for (int i = 0; i < prefilled; ++i) {
        mbar_arrive_expect_tx(bar_full + 8 * i, C::kStageBytes);
        load_w_tile(stage0 + i * C::kStageBytes, &tm_w, p, g, nb, kb0 + i, bar_full + 8 * i);
      }
    }
    for (int i = 0; i < prefilled; ++i)
      tma_load_2d(stage0 + i * C::kStageBytes + kTileN * kBlockK, &tm_x, (kb0 + i) * kBlockK, row0, bar_full + 8 * i);
  }
  if (tid >= 64) {
    const float* swr = p.sw + ((int64_t)g * NB + nb) * KB;
    const float* sxr = p.sx + (int64_t)xblk * KB;
    for (int kb = tid - 64; kb < nkb; kb += 128) sprod[kb] = swr[kb0 + kb] * sxr[kb0 + kb];
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int i = prefilled; i < nkb; ++i) {
        const int s = i % S;
        if (i >= S && !mbar_wait(bar_empty + 8 * s, ((i / S) - 1) & 1, &abort_flag, p.status, p.wait_tries)) break;
        const uint32_t a_dst = stage0 + s * C::kStageBytes, b_dst = a_dst + kTileN * kBlockK;
        mbar_arrive_expect_tx(bar_full + 8 * s, C::kStageBytes);
        load_w_tile(a_dst, &tm_w, p, g, nb, kb0 + i, bar_full + 8 * s);
        tma_load_2d(b_dst, &tm_x, (kb0 + i) * kBlockK, row0, bar_full + 8 * s);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // instruction descriptor: fp32 accumulate, A and B e4m3, both K-major, N = TN, M = 128
      constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(kTileN >> 4) << 24);
      for (int i = 0; i < nkb; ++i) {
        const int s = i % S, b = i & 1;
        if (!mbar_wait(bar_full + 8 * s, (i / S) & 1, &abort_flag, p.status, p.wait_tries)) break;
        if (i >= 2 && !mbar_wait(bar_tempty + 8 * b, ((i >> 1) - 1) & 1, &abort_flag, p.status, p.wait_tries)) break;
        tc_fence_after();
        const uint32_t a_addr = stage0 + s * C::kStageBytes, b_addr = a_addr + kTileN * kBlockK;
        const uint64_t da = smem_desc_sw128(a_addr), db = smem_desc_sw128(b_addr);
#pragma unroll
        for (int k = 0; k < 4; ++k)  // 32 bytes of K per instruction: advance the start address field by 32 >> 4
          tc_mma_f8(tmem_base + b * TN, da + 2 * k, db + 2 * k, idesc, k > 0 ? 1u : 0u);
        tc_commit(bar_empty + 8 * s);  // stage reusable once these MMAs have read it
        tc_commit(bar_tfull + 8 * b);  // accumulator buffer complete
      }
    }
  } else {
    // ---------------- epilogue warps: lanes [32q, 32q+32) of tensor memory = weight rows n0 + 32q + lane
    const int q = warp & 3;
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
    float acc[TN];
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[j] = 0.f;
    for (int i = 0; i < nkb; ++i) {
      const int b = i & 1;
      if (!mbar_wait(bar_tfull + 8 * b, (i >> 1) & 1, &abort_flag, p.status, p.wait_tries)) break;
      tc_fence_after();
      const float sc = sprod[i];
#pragma unroll
      for (int c = 0; c < TN / 16; ++c) {
        float v[16];
        tmem_ld16(lane_base + b * TN + c * 16, v);
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[c * 16 + j] = fmaf(sc, v[j], acc[c * 16 + j]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * b);
    }
    const int n = n0 + q * 32 + lane;
    if (n < p.N && !abort_flag) {
      if (p.splits > 1) {
        float* yp = p.y_part + ((int64_t)split * p.rows) * p.N;
#pragma unroll
        for (int j = 0; j < TN; ++j)
          if (row0 + j < row_end) yp[(int64_t)(row0 + j) * p.N + n] = acc[j];
      } else {
#pragma unroll
        for (int j = 0; j < TN; ++j)
          if (row0 + j < row_end) {
            uint32_t h;
            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(h) : "f"(0.f), "f"(acc[j]));
            p.y[(int64_t)(row0 + j) * p.ldy + n] = (uint16_t)(h & 0xFFFFu);
          }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, C::kTmemCols);
}

// ---------------------------------------------------------------------------------------------
// Persistent variant: at most two CTAs per SM walk the work list (token tile fastest, then weight tile, then K
// split) with a stride of the grid size.  The stage ring and the tensor-memory buffers keep rotating across
// tiles, so the producer is already loading the next tile while the epilogue warps store the current one, and the
// per-CTA set-up (barriers, tensor-memory allocation) is paid once per SM instead of once per tile.
template <int TN>
struct PCfg {
  static constexpr int kStageBytes = kTileN * kBlockK + TN * kBlockK;
  static constexpr int kStages = (TN == 128) ? 3 : (TN == 64) ? 4 : 5;
  static constexpr int kBufs = (TN == 128) ? 2 : 4;  // accumulator buffers in tensor memory
  static constexpr uint32_t kTmemCols = (kBufs * TN < 32) ? 32 : kBufs * TN;
  static constexpr size_t kSmem = 1024 + (size_t)kStages * kStageBytes + 256;
};

struct TileInfo {
  int g, row0, row_end, xblk, nb, n0, split, kb0, nkb;
};

__device__ __forceinline__ TileInfo decode_tile(const GemmParams& p, int w, int TT, int NB, int KB, int tn) {
  TileInfo t;
  const int tt = w % TT;
  t.nb = (w / TT) % NB;
  t.split = w / (TT * NB);
  t.n0 = t.nb * kTileN;
  if (p.seg_off) {
    t.g = p.tile_group[tt];
    t.row0 = p.tile_row0[tt];
    t.row_end = p.seg_off[t.g + 1];
    t.xblk = p.blk_off[t.g] + (t.row0 - p.seg_off[t.g]) / 128;
  } else {
    t.g = 0;
    t.row0 = tt * tn;
    t.row_end = p.rows;
    t.xblk = t.row0 / 128;
  }
  const int kb_per = (KB + p.splits - 1) / p.splits;
  t.kb0 = t.split * kb_per;
  t.nkb = max(0, min(KB, t.kb0 + kb_per) - t.kb0);
  return t;
}

template <int TN>
__global__ void __launch_bounds__(kThreads, 2)
gemm_fp8_persistent_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                           const GemmParams p) {
  eb::pdl_trigger();  // programmatic dependent launch: set-up below overlaps the predecessor's tail
  using C = PCfg<TN>;
  constexpr int S = C::kStages, NBUF = C::kBufs;
  const int KB = (p.K + kBlockK - 1) / kBlockK;
  const int NB = (p.N + kTileN - 1) / kTileN;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t stage0 = (raw + 1023u) & ~1023u;
  uint8_t* after = smem_raw + (stage0 - raw) + S * C::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(after);  // full[S], empty[S], tfull[NBUF], tempty[NBUF]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(after + (2 * S + 2 * NBUF) * sizeof(uint64_t));
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t bar_full = smem_u32(&bars[0]), bar_empty = smem_u32(&bars[S]);
  const uint32_t bar_tfull = smem_u32(&bars[2 * S]), bar_tempty = smem_u32(&bars[2 * S + NBUF]);
  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < NBUF; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
  if (tid == 32 * 2 && p.w_tiled) {
    // While the predecessor drains: pull the first K blocks of this CTA's first weight tile into L2.  The weights do
    // not depend on the predecessor; which tile comes first does (grouped: the tile table), so it is guessed -- one
    // token tile per group, the common case in a decode batch -- and a wrong guess costs a little bandwidth, nothing else.
    const int TTg = p.seg_off ? p.n_groups : (p.rows + TN - 1) / TN;
    const int w0 = blockIdx.x, nb0 = w0 / TTg, g0 = p.seg_off ? w0 % TTg : 0;
    if (nb0 < NB) {
      const uint8_t* src = p.w8 + ((int64_t)(g0 * NB + nb0) * KB) * (kTileN * kBlockK);
      const uint32_t bytes = (uint32_t)min(KB, 8) * (kTileN * kBlockK);
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  eb::pdl_wait();  // the predecessor in the stream has completed and its writes are visible
  const int TT = p.seg_off ? *p.n_tiles : (p.rows + TN - 1) / TN;
  const int n_work = TT * NB * p.splits;  // a CTA beyond the work list runs no loop iteration and leaves below

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;  // K blocks issued by this CTA so far, over all its tiles
      bool ok = true;
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
        const TileInfo t = decode_tile(p, w, TT, NB, KB, TN);
        for (int i = 0; i < t.nkb; ++i, ++it) {
          const uint32_t s = it % S;
          if (it >= (uint32_t)S && !mbar_wait(bar_empty + 8 * s, ((it / S) - 1) & 1, &abort_flag, p.status, p.wait_tries)) {
            ok = false;
            break;
          }
          const uint32_t a_dst = stage0 + s * C::kStageBytes, b_dst = a_dst + kTileN * kBlockK;
          mbar_arrive_expect_tx(bar_full + 8 * s, C::kStageBytes);
          load_w_tile(a_dst, &tm_w, p, t.g, t.nb, t.kb0 + i, bar_full + 8 * s);
          tma_load_2d(b_dst, &tm_x, (t.kb0 + i) * kBlockK, t.row0, bar_full + 8 * s);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(kTileN >> 4) << 24);
      uint32_t it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
        const TileInfo t = decode_tile(p, w, TT, NB, KB, TN);
        for (int i = 0; i < t.nkb; ++i, ++it) {
          const uint32_t s = it % S, b = it % NBUF;
          if (!mbar_wait(bar_full + 8 * s, (it / S) & 1, &abort_flag, p.status, p.wait_tries) ||
              (it >= (uint32_t)NBUF && !mbar_wait(bar_tempty + 8 * b, ((it / NBUF) - 1) & 1, &abort_flag, p.status, p.wait_tries))) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = stage0 + s * C::kStageBytes, b_addr = a_addr + kTileN * kBlockK;
          const uint64_t da = smem_desc_sw128(a_addr), db = smem_desc_sw128(b_addr);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_f8(tmem_base + b * TN, da + 2 * k, db + 2 * k, idesc, k > 0 ? 1u : 0u);
          tc_commit(bar_empty + 8 * s);
          tc_commit(bar_tfull + 8 * b);
        }
      }
    }
  } else {
    const int q = warp & 3;
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
    uint32_t it = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
      const TileInfo t = decode_tile(p, w, TT, NB, KB, TN);
      // scale products of this tile's K blocks, block kb held by lane kb % 32 in register kb / 32
      float sreg[kMaxKB / 32];
      {
        const float* swr = p.sw + ((int64_t)t.g * NB + t.nb) * KB + t.kb0;
        const float* sxr = p.sx + (int64_t)t.xblk * KB + t.kb0;
#pragma unroll
        for (int j = 0; j < kMaxKB / 32; ++j) {
          const int kb = lane + 32 * j;
          sreg[j] = kb < t.nkb ? swr[kb] * sxr[kb] : 0.f;
        }
      }
      float acc[TN];
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[j] = 0.f;
      for (int i = 0; i < t.nkb; ++i, ++it) {
        const uint32_t b = it % NBUF;
        if (!mbar_wait(bar_tfull + 8 * b, (it / NBUF) & 1, &abort_flag, p.status, p.wait_tries)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const int jr = i >> 5;
        const float mine = jr == 0 ? sreg[0] : jr == 1 ? sreg[1] : jr == 2 ? sreg[2] : sreg[3];
        const float sc = __shfl_sync(0xffffffffu, mine, i & 31);
#pragma unroll
        for (int c = 0; c < TN / 16; ++c) {
          float v[16];
          tmem_ld16(lane_base + b * TN + c * 16, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[c * 16 + j] = fmaf(sc, v[j], acc[c * 16 + j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tempty + 8 * b);
      }
      const int n = t.n0 + q * 32 + lane;
      if (ok && n < p.N) {
        if (p.splits > 1) {
          float* yp = p.y_part + ((int64_t)t.split * p.rows) * p.N;
#pragma unroll
          for (int j = 0; j < TN; ++j)
            if (t.row0 + j < t.row_end) yp[(int64_t)(t.row0 + j) * p.N + n] = acc[j];
        } else {
#pragma unroll
          for (int j = 0; j < TN; ++j)
            if (t.row0 + j < t.row_end) {
              uint32_t h;
              asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(h) : "f"(0.f), "f"(acc[j]));
              p.y[(int64_t)(t.row0 + j) * p.ldy + n] = (uint16_t)(h & 0xFFFFu);
            }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, C::kTmemCols);
}

// ---------------------------------------------------------------------------------------------
// Prefill-sized dense GEMM (hundreds of tokens and more): compute bound, so the tile is as large as one CTA's
// tensor memory allows.  Tokens are the MMA's M operand here (128 per tile) and 256 weight rows its N operand:
// a thread of the epilogue then owns one token and 128 consecutive outputs, which it stores as 16-byte vectors.
// One persistent CTA per SM, 384 threads in three warpgroups: warpgroup 0 holds the TMA producer (warp 0) and the
// MMA issuer (warp 1) and gives its registers away; warpgroups 1 and 2 are the epilogue (tensor-memory lane
// quarter = warp % 4, warpgroup 1 takes accumulator columns 0..127 and warpgroup 2 columns 128..255) and claim
// 232 registers per thread for the 128 running sums plus two 32-column loads in flight.
constexpr int kBigThreads = 384;
constexpr int kBigTokens = 128;  // MMA M
constexpr int kBigRows = 256;    // weight rows per tile, MMA N
constexpr int kBigStages = 4;
constexpr int kBigStageBytes = (kBigTokens + kBigRows) * kBlockK;
constexpr size_t kBigSmem = 1024 + (size_t)kBigStages * kBigStageBytes + 256;

#define EB_R8(a, o) "=r"(a[o]), "=r"(a[o + 1]), "=r"(a[o + 2]), "=r"(a[o + 3]), "=r"(a[o + 4]), "=r"(a[o + 5]), "=r"(a[o + 6]), "=r"(a[o + 7])
#define EB_RW8(a, o) "+r"(a[o]), "+r"(a[o + 1]), "+r"(a[o + 2]), "+r"(a[o + 3]), "+r"(a[o + 4]), "+r"(a[o + 5]), "+r"(a[o + 6]), "+r"(a[o + 7])
// 32 lanes x 64 consecutive columns, issued without waiting; tmem_wait64 makes the registers valid.
__device__ __forceinline__ void tmem_ld64_issue(uint32_t taddr, uint32_t (&r)[64]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,"
      "%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,"
      "%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];"
      : EB_R8(r, 0), EB_R8(r, 8), EB_R8(r, 16), EB_R8(r, 24), EB_R8(r, 32), EB_R8(r, 40), EB_R8(r, 48), EB_R8(r, 56)
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait64(uint32_t (&r)[64]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : EB_RW8(r, 0), EB_RW8(r, 8), EB_RW8(r, 16), EB_RW8(r, 24), EB_RW8(r, 32), EB_RW8(r, 40), EB_RW8(r, 48),
                 EB_RW8(r, 56)
               :
               : "memory");
}

__global__ void __launch_bounds__(kBigThreads, 1)
gemm_fp8_big_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const GemmParams p) {
  eb::pdl_trigger();  // programmatic dependent launch: set-up below overlaps the predecessor's tail
  constexpr int S = kBigStages, NBUF = 2;
  const int KB = (p.K + kBlockK - 1) / kBlockK;
  const int NB2 = (p.N + kBigRows - 1) / kBigRows;
  const int NB = (p.N + kTileN - 1) / kTileN;  // scale blocks along N
  const int TT = (p.rows + kBigTokens - 1) / kBigTokens;
  const int n_work = TT * NB2;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t stage0 = (raw + 1023u) & ~1023u;
  uint8_t* after = smem_raw + (stage0 - raw) + S * kBigStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(after);  // full[S], empty[S], tfull[NBUF], tempty[NBUF]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(after + (2 * S + 2 * NBUF) * sizeof(uint64_t));
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t bar_full = smem_u32(&bars[0]), bar_empty = smem_u32(&bars[S]);
  const uint32_t bar_tfull = smem_u32(&bars[2 * S]), bar_tempty = smem_u32(&bars[2 * S + NBUF]);
  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < NBUF; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, 8);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  eb::pdl_wait();  // the predecessor in the stream has completed and its writes are visible

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0 && lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
        const int row0 = (w % TT) * kBigTokens, n0 = (w / TT) * kBigRows;
        for (int i = 0; i < KB; ++i, ++it) {
          const uint32_t s = it % S;
          if (it >= (uint32_t)S && !mbar_wait(bar_empty + 8 * s, ((it / S) - 1) & 1, &abort_flag, p.status, p.wait_tries)) {
            ok = false;
            break;
          }
          const uint32_t a_dst = stage0 + s * kBigStageBytes, b_dst = a_dst + kBigTokens * kBlockK;
          mbar_arrive_expect_tx(bar_full + 8 * s, kBigStageBytes);
          tma_load_2d(a_dst, &tm_x, i * kBlockK, row0, bar_full + 8 * s);
          if (p.w_tiled) {  // 256 weight rows = two 16 KiB tiles (a block beyond the last one is filled with zeros)
            load_w_tile(b_dst, &tm_w, p, 0, n0 / kTileN, i, bar_full + 8 * s);
            load_w_tile(b_dst + kTileN * kBlockK, &tm_w, p, 0, n0 / kTileN + 1, i, bar_full + 8 * s);
          } else {
            tma_load_2d(b_dst, &tm_w, i * kBlockK, n0, bar_full + 8 * s);
          }
        }
      }
    } else if (warp == 1 && lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(kBigRows >> 3) << 17) | ((uint32_t)(kBigTokens >> 4) << 24);
      uint32_t it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
        for (int i = 0; i < KB; ++i, ++it) {
          const uint32_t s = it % S, b = it % NBUF;
          if (!mbar_wait(bar_full + 8 * s, (it / S) & 1, &abort_flag, p.status, p.wait_tries) ||
              (it >= (uint32_t)NBUF && !mbar_wait(bar_tempty + 8 * b, ((it / NBUF) - 1) & 1, &abort_flag, p.status, p.wait_tries))) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = stage0 + s * kBigStageBytes, b_addr = a_addr + kBigTokens * kBlockK;
          const uint64_t da = smem_desc_sw128(a_addr), db = smem_desc_sw128(b_addr);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_f8(tmem_base + b * kBigRows, da + 2 * k, db + 2 * k, idesc, k > 0 ? 1u : 0u);
          tc_commit(bar_empty + 8 * s);
          tc_commit(bar_tfull + 8 * b);
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    const int q = warp & 3, h = (warp - 4) >> 2;
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16) + h * 128;
    const bool vec_ok = (p.ldy % 8 == 0) && (p.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.y) & 15) == 0);
    uint32_t it = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
      const int tt = w % TT, row0 = tt * kBigTokens, n0 = (w / TT) * kBigRows + h * 128;
      float sreg[kMaxKB / 32];
      {
        const int nblk = min(n0 / kTileN, NB - 1);
        const float* swr = p.sw + (int64_t)nblk * KB;
        const float* sxr = p.sx + (int64_t)tt * KB;
#pragma unroll
        for (int j = 0; j < kMaxKB / 32; ++j) {
          const int kb = lane + 32 * j;
          sreg[j] = kb < KB ? swr[kb] * sxr[kb] : 0.f;
        }
      }
      float acc[128];
#pragma unroll
      for (int j = 0; j < 128; ++j) acc[j] = 0.f;
      for (int i = 0; i < KB; ++i, ++it) {
        const uint32_t b = it % NBUF;
        if (!mbar_wait(bar_tfull + 8 * b, (it / NBUF) & 1, &abort_flag, p.status, p.wait_tries)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const int jr = i >> 5;
        const float mine = jr == 0 ? sreg[0] : jr == 1 ? sreg[1] : jr == 2 ? sreg[2] : sreg[3];
        const float sc = __shfl_sync(0xffffffffu, mine, i & 31);
        const uint32_t src = lane_base + b * kBigRows;
        uint32_t v[64];
        tmem_ld64_issue(src, v);
        tmem_wait64(v);
#pragma unroll
        for (int j = 0; j < 64; ++j) acc[j] = fmaf(sc, __uint_as_float(v[j]), acc[j]);
        tmem_ld64_issue(src + 64, v);
        tmem_wait64(v);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tempty + 8 * b);  // the accumulator buffer is free before the last 64 sums
#pragma unroll
        for (int j = 0; j < 64; ++j) acc[64 + j] = fmaf(sc, __uint_as_float(v[j]), acc[64 + j]);
      }
      const int r = row0 + q * 32 + lane;
      if (ok && r < p.rows && n0 < p.N) {
        uint16_t* yr = p.y + (int64_t)r * p.ldy + n0;
        if (vec_ok) {
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            if (n0 + c * 8 < p.N) {
              uint32_t h4[4];
#pragma unroll
              for (int j = 0; j < 4; ++j)
                asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(h4[j]) : "f"(acc[c * 8 + 2 * j + 1]), "f"(acc[c * 8 + 2 * j]));
              *reinterpret_cast<uint4*>(yr + c * 8) = make_uint4(h4[0], h4[1], h4[2], h4[3]);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 128; ++j)
            if (n0 + j < p.N) {
              uint32_t hh;
              asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(hh) : "f"(0.f), "f"(acc[j]));
              yr[j] = (uint16_t)(hh & 0xFFFFu);
            }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ---------------------------------------------------------------------------------------------
// Issue-rate microbenchmark of the FP8 tensor path: the denominator for "fraction of FP8 peak".  Every CTA (one per
// SM) fills two operand stages in shared memory with pseudo-random e4m3 codes once, then one thread issues `blocks`
// groups of four tcgen05.mma.kind::f8f6f4 (M = 128, N = 256, K = 32 each) back to back, alternating between the two
// stages and two accumulators in tensor memory.  Nothing is loaded from global memory and nothing is read back, so the
// time is the tensor pipe's alone: 2 * 128 * 256 * 128 flop per group per SM.
constexpr int kPeakStageBytes = (128 + 256) * kBlockK;
constexpr size_t kPeakSmem = 1024 + 2 * kPeakStageBytes + 64;

__global__ void __launch_bounds__(128, 1) fp8_mma_peak_kernel(int blocks, int32_t* status, uint32_t wait_tries) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t stage0 = (raw + 1023u) & ~1023u;
  uint8_t* stages = smem_raw + (stage0 - raw);
  uint64_t* bar = reinterpret_cast<uint64_t*>(stages + 2 * kPeakStageBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;
  // operands: hashed bytes with the exponent field kept below all-ones (no NaN codes), so the data toggles as real
  // activations and weights would
  for (int i = tid; i < 2 * kPeakStageBytes / 4; i += blockDim.x) {
    uint32_t h = (uint32_t)i * 2654435761u + blockIdx.x * 40503u;
    h ^= h >> 15;
    h *= 2246822519u;
    h ^= h >> 13;
    reinterpret_cast<uint32_t*>(stages)[i] = h & 0xBFBFBFBFu;
  }
  if (tid == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes visible to the tensor core
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (tid == 0) {
    constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    for (int i = 0; i < blocks; ++i) {
      const uint32_t a_addr = stage0 + (i & 1) * kPeakStageBytes, b_addr = a_addr + 128 * kBlockK;
      const uint64_t da = smem_desc_sw128(a_addr), db = smem_desc_sw128(b_addr);
#pragma unroll
      for (int k = 0; k < 4; ++k) tc_mma_f8(tmem_base + (i & 1) * 256, da + 2 * k, db + 2 * k, idesc, (i > 1 || k > 0) ? 1u : 0u);
    }
    tc_commit(smem_u32(bar));
    mbar_wait(smem_u32(bar), 0, &abort_flag, status, wait_tries);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// Row-major e4m3 weights [groups][N][K] -> tiles [groups][ceil(N/128)][ceil(K/128)][128][128], zero padded.
// One CTA per tile, 256 threads x four 16-byte chunks.
__global__ void __launch_bounds__(256) weight_tile_kernel(const uint8_t* src, uint8_t* dst, int N, int K) {
  const int KBw = (K + kBlockK - 1) / kBlockK, NBw = (N + kTileN - 1) / kTileN;
  const int64_t tile = blockIdx.x;
  const int kb = (int)(tile % KBw), nb = (int)((tile / KBw) % NBw);
  const int64_t g = tile / ((int64_t)KBw * NBw);
  uint4* out = reinterpret_cast<uint4*>(dst + tile * (kTileN * kBlockK));
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int ch = threadIdx.x + 256 * q;  // chunk of the tile: row ch / 8, bytes [16 * (ch % 8), +16)
    const int r = ch >> 3, c = (ch & 7) * 16;
    const int n = nb * kTileN + r, k = kb * kBlockK + c;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (n < N && k < K) v = *reinterpret_cast<const uint4*>(src + (g * N + n) * (int64_t)K + k);  // K is a multiple of 16
    out[ch] = v;
  }
}

// Sum split-K partials in split order and round to bf16.
__global__ void gemm_splitk_reduce_kernel(const float* part, uint16_t* y, int64_t ldy, int rows, int N, int splits) {
  eb::pdl_wait();  // programmatic dependent launch: the predecessor in the stream has completed
  eb::pdl_trigger();
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)rows * N) return;
  float a = 0.f;
  for (int s = 0; s < splits; ++s) a += part[(int64_t)s * rows * N + idx];
  uint32_t h;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(h) : "f"(0.f), "f"(a));
  y[(idx / N) * ldy + idx % N] = (uint16_t)(h & 0xFFFFu);
}

// Token-tile table of a grouped GEMM: for group g with rows [seg_off[g], seg_off[g+1]) emit one tile per TN rows.
// Also the exclusive prefix of 128-row scale blocks.  One CTA; n_groups <= 1024.
__global__ void gemm_tiles_kernel(const int32_t* seg_off, int n_groups, int tn, int max_tiles, int32_t* blk_off,
                                  int32_t* tile_group, int32_t* tile_row0, int32_t* n_tiles, int32_t* status) {
  eb::pdl_wait();  // programmatic dependent launch: the predecessor in the stream has completed
  eb::pdl_trigger();
  __shared__ int32_t t_off[1025], b_off[1025];
  for (int g = threadIdx.x; g < n_groups; g += blockDim.x) {
    const int len = seg_off[g + 1] - seg_off[g];
    t_off[g + 1] = (len + tn - 1) / tn;
    b_off[g + 1] = (len + 127) / 128;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    t_off[0] = b_off[0] = 0;
    for (int g = 0; g < n_groups; ++g) {
      t_off[g + 1] += t_off[g];
      b_off[g + 1] += b_off[g];
    }
    int nt = t_off[n_groups];
    if (nt > max_tiles) {
      atomicOr(status, EB_DEV_BAD_INDEX);
      nt = max_tiles;
    }
    *n_tiles = nt;
  }
  __syncthreads();
  for (int g = threadIdx.x; g <= n_groups; g += blockDim.x) blk_off[g] = b_off[g];
  for (int g = threadIdx.x; g < n_groups; g += blockDim.x)
    for (int t = t_off[g]; t < t_off[g + 1] && t < max_tiles; ++t) {
      tile_group[t] = g;
      tile_row0[t] = seg_off[g] + (t - t_off[g]) * tn;
    }
}

// x / s, correctly rounded, for a divisor shared by many elements: r = RN(1 / s), q = RN(x r), q' = RN(q + r (x - q s)).
// With the reciprocal correctly rounded and q within one ulp of the quotient, q' is the correctly rounded quotient
// (Markstein's division) as long as the residual x - q s does not underflow and the divisor's significand is not all
// ones.  Divisors outside [2^-64, 2^64] or with such a significand take the IEEE division; for the others an element
// small enough for the residual to underflow has a quotient below 2^-12, which e4m3 rounds to zero either way
// (checked against x / s over 2 * 10^7 random bf16 x and fp32 s on the host).  Three dependent FMAs per element.
__device__ __forceinline__ bool exact_div_plain(float s) {
  return (__float_as_uint(s) & 0x7FFFFFu) == 0x7FFFFFu || !(s >= 0x1p-64f && s <= 0x1p64f);
}
__device__ __forceinline__ float exact_div(float x, float s, float r, bool plain) {
  if (plain) return __fdiv_rn(x, s);
  const float q = __fmul_rn(x, r);
  const float c = __fmaf_rn(__fmaf_rn(-q, s, x), r, q);
  return q == 0.f ? q : c;  // a zero keeps its sign (the correction term would turn -0 into +0)
}

// Destinations of a quantiser launch whose result is one column band of an operand that every rank of a tensor-parallel
// group assembles (size == 0: a plain launch into `codes` / `scales`): rank p receives the codes at codes[p] (row pitch
// ldc) and the scales at scales[p] (lds scales per row block); the launch raises the collective's flags itself.
struct QuantPeers {
  uint8_t* codes[eb::kPeerMaxRanks];
  float* scales[eb::kPeerMaxRanks];
  int64_t ldc;
  int32_t lds, size, chunk;  // chunk > 0: rows [p * chunk, +chunk) go to rank p only (its token slice); 0: all rows to all
  eb::PeerPlanes arrive;
};

// Activation quantiser: one CTA per (128-row block, 128-column block) of a bf16 matrix.
// NT threads; thread t holds 2048 / NT rows x one 16-byte chunk; block amax -> scale -> e4m3.  Grids with fewer CTAs
// than SMs run 1024 threads (32 warps hide each other's load and arithmetic latency), large grids 512.
// MODE 0: value = x[src_row(r)][c] (src_row = identity when row_map is null).
// MODE 1: x holds [gate | up] halves of width `cols`; value = bf16( gate/(1+exp(-gate)) * up ).
template <int MODE, int NT>
__global__ void __launch_bounds__(NT, NT == 1024 ? 1 : 2)
quant_act_kernel(const uint16_t* x, int64_t ldx, int rows, int cols, const int32_t* seg_off, int n_groups,
                 const int32_t* row_map, int src_rows, uint8_t* codes, float* scales, int32_t* status, const QuantPeers qp) {
  constexpr int RPT = 2048 / NT;   // rows per thread
  constexpr int RSTEP = NT / 16;   // rows between a thread's consecutive chunks
  eb::pdl_wait();  // programmatic dependent launch: the predecessor in the stream has completed
  eb::pdl_trigger();
  const int blk = blockIdx.y, cb = blockIdx.x, n_cb = gridDim.x;
  int r0, r1;
  if (seg_off) {
    // Row range of scale block `blk`: blocks restart at every segment start.  Warp 0 scans the segments 32 at a time.
    __shared__ int s_r0, s_r1;
    if (threadIdx.x < 32) {
      const int lane = threadIdx.x;
      int base = 0;
      bool found = false;
      for (int g0 = 0; g0 < n_groups && !found; g0 += 32) {
        const int g = g0 + lane;
        const int lo = g < n_groups ? seg_off[g] : 0, hi = g < n_groups ? seg_off[g + 1] : 0;
        const int cnt = (hi - lo + 127) / 128;
        int incl = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int v = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += v;
        }
        const int first = base + incl - cnt;
        const bool hit = cnt > 0 && blk >= first && blk < base + incl;
        if (hit) {
          s_r0 = lo + (blk - first) * 128;
          s_r1 = min(lo + (blk - first) * 128 + 128, hi);
        }
        found = __any_sync(0xffffffffu, hit);
        base += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (!found && lane == 0) s_r0 = -1;
    }
    __syncthreads();
    if (s_r0 < 0) return;
    r0 = s_r0;
    r1 = s_r1;
  } else {
    r0 = blk * 128;
    r1 = min(r0 + 128, rows);
    if (r0 >= rows) return;
  }
  const int p_lo = qp.chunk > 0 ? r0 / qp.chunk : 0, p_hi = qp.chunk > 0 ? p_lo + 1 : qp.size;  // receivers of this row block
  const int c0 = cb * 128;
  const int chunk = threadIdx.x & 15, rsub = threadIdx.x >> 4;
  const int col = c0 + chunk * 8;
  const bool col_ok = col < cols;  // cols is a multiple of 8
  uint4 v[RPT];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = r0 + rsub + i * RSTEP;
    v[i] = make_uint4(0, 0, 0, 0);
    if (col_ok && r < r1) {
      int sr = r;
      if (MODE == 0 && row_map) {
        sr = row_map[r];
        if (sr < 0 || sr >= src_rows) {
          atomicOr(status, EB_DEV_BAD_INDEX);
          sr = 0;
        }
      }
      v[i] = *reinterpret_cast<const uint4*>(x + (int64_t)sr * ldx + col);
      if (MODE == 1) {
        const uint4 u = *reinterpret_cast<const uint4*>(x + (int64_t)sr * ldx + cols + col);
        const uint32_t gw[4] = {v[i].x, v[i].y, v[i].z, v[i].w}, uw[4] = {u.x, u.y, u.z, u.w};
        uint32_t o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float g0 = __uint_as_float(gw[k] << 16), g1 = __uint_as_float(gw[k] & 0xFFFF0000u);
          const float u0 = __uint_as_float(uw[k] << 16), u1 = __uint_as_float(uw[k] & 0xFFFF0000u);
          const float a0 = __fmul_rn(__fdiv_rn(g0, 1.0f + expf(-g0)), u0);
          const float a1 = __fmul_rn(__fdiv_rn(g1, 1.0f + expf(-g1)), u1);
          asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o[k]) : "f"(a1), "f"(a0));
        }
        v[i] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
    const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      amax = fmaxf(amax, fabsf(__uint_as_float(w[k] << 16)));
      amax = fmaxf(amax, fabsf(__uint_as_float(w[k] & 0xFFFF0000u)));
    }
  }
  __shared__ float red[NT / 32];
#pragma unroll
  for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int w = 1; w < NT / 32; ++w) amax = fmaxf(amax, red[w]);
  const float s = amax > 0.f ? __fdiv_rn(amax, 448.0f) : 1.0f;
  if (threadIdx.x == 0) {
    if (qp.size == 0) {
      scales[(int64_t)blk * n_cb + cb] = s;
    } else {
      for (int pr = p_lo; pr < p_hi; ++pr) qp.scales[pr][(int64_t)blk * qp.lds + cb] = s;
    }
  }
  const float rs = __frcp_rn(s);
  const bool plain = exact_div_plain(s);
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int r = r0 + rsub + i * RSTEP;
    if (!(col_ok && r < r1)) continue;
    const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
    uint32_t o[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      uint16_t lo16, hi16;
      const float a0 = exact_div(__uint_as_float(w[2 * k] << 16), s, rs, plain);
      const float a1 = exact_div(__uint_as_float(w[2 * k] & 0xFFFF0000u), s, rs, plain);
      const float a2 = exact_div(__uint_as_float(w[2 * k + 1] << 16), s, rs, plain);
      const float a3 = exact_div(__uint_as_float(w[2 * k + 1] & 0xFFFF0000u), s, rs, plain);
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo16) : "f"(a1), "f"(a0));
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi16) : "f"(a3), "f"(a2));
      o[k] = (uint32_t)lo16 | ((uint32_t)hi16 << 16);
    }
    if (qp.size == 0) {
      *reinterpret_cast<uint2*>(codes + (int64_t)r * cols + col) = make_uint2(o[0], o[1]);
    } else {
      for (int pr = p_lo; pr < p_hi; ++pr) *reinterpret_cast<uint2*>(qp.codes[pr] + (int64_t)r * qp.ldc + col) = make_uint2(o[0], o[1]);
    }
  }
  if (qp.size) eb::peer_arrive_cta(qp.arrive);  // (such a launch has no segments: every CTA has a block and gets here)
}

template <int TN>
int32_t launch_gemm(const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, dim3 grid, cudaStream_t st) {
  auto kfn = gemm_fp8_kernel<TN>;
  static bool configured[64] = {false};  // the attribute is per device
  int dev = 0;
  EB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    EB_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<TN>::kSmem));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  EB_CUDA(eb::launch(kfn, dim3(grid), dim3(kThreads), Cfg<TN>::kSmem, st, tw, tx, p));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int sm_count_now() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!cached[dev]) {
    int n = 148;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n;
  }
  return cached[dev];
}

// Which kernel runs a GEMM: the persistent one pays off once the tiles exceed what the GPU holds at a time (two CTAs
// per SM); below that the one-tile-per-CTA kernel starts its loads sooner.  EIDOLA_B200_GEMM_LEGACY=1 forces the
// one-tile kernel, =0 the persistent one (for A/B timing).
bool gemm_persistent(int64_t work_upper, int sms) {
  static const int mode = [] {
    const char* v = getenv("EIDOLA_B200_GEMM_LEGACY");
    return !v ? -1 : (v[0] == '1' ? 1 : 0);
  }();
  if (mode >= 0) return mode == 0;
  return work_upper > 2ll * sms;
}

template <int TN>
int32_t launch_gemm_persistent(const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, int64_t work_upper,
                               cudaStream_t st) {
  auto kfn = gemm_fp8_persistent_kernel<TN>;
  static bool configured[64] = {false};  // the attribute is per device
  int dev = 0;
  EB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    EB_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PCfg<TN>::kSmem));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const int sms = sm_count_now();
  const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(work_upper, 2ll * sms));
  EB_CUDA(eb::launch(kfn, dim3(grid), dim3(kThreads), PCfg<TN>::kSmem, st, tw, tx, p));
  return EB_OK;
}

// Dense GEMMs of 512 tokens and more take the 128-token x 256-row kernel unless the caller fixed a tile or a split.
// EIDOLA_B200_GEMM_BIG=0 keeps them on the decode kernels (for A/B timing).
bool gemm_big(int rows, int N, int tile_tokens, int splits) {
  static const bool on = [] {
    const char* v = getenv("EIDOLA_B200_GEMM_BIG");
    return !(v && v[0] == '0');
  }();
  // 512 tokens and more; from 256 tokens on when the weight matrix is so tall (an LM head) that the decode kernels'
  // re-reading of the activations through L2 costs more than half-empty 128-token tiles
  return on && (rows >= 512 || (rows >= 256 && N >= 65536)) && tile_tokens == 0 && splits <= 1;
}

int pick_tn(int64_t rows_per_group) {
  if (rows_per_group <= 16) return 16;
  if (rows_per_group <= 32) return 32;
  if (rows_per_group <= 64) return 64;
  return 128;
}

int32_t run_gemm(const eb_gemm_args* a, bool grouped, cudaStream_t st, int32_t* splits_used = nullptr) {
  EB_REQUIRE(a->d_x8 && a->d_sx && a->d_w8 && a->d_sw && a->d_y, EB_ERR_ARG, "gemm: null pointer");
  EB_REQUIRE(a->rows >= 0 && a->N >= 1 && a->K >= 16 && a->n_groups >= 1, EB_ERR_ARG, "gemm: bad size");
  EB_REQUIRE(a->K % 16 == 0, EB_ERR_UNSUPPORTED, "gemm: K %d must be a multiple of 16", a->K);
  EB_REQUIRE(a->K <= kMaxKB * kBlockK, EB_ERR_UNSUPPORTED, "gemm: K %d exceeds %d", a->K, kMaxKB * kBlockK);
  EB_REQUIRE(a->ldy >= a->N, EB_ERR_ARG, "gemm: ldy %lld < N %d", (long long)a->ldy, a->N);
  EB_REQUIRE(a->n_groups <= 1024, EB_ERR_UNSUPPORTED, "gemm: %d groups (at most 1024)", a->n_groups);
  EB_REQUIRE((int64_t)a->n_groups * a->N < (1ll << 31), EB_ERR_UNSUPPORTED, "gemm: weight rows exceed a tensor map");
  if (a->rows == 0) return EB_OK;
  int32_t* status = eb::status_word();
  EB_REQUIRE(status, EB_ERR_NODEVICE, "gemm: no device");

  GemmParams p = {};
  p.sx = a->d_sx;
  p.sw = a->d_sw;
  p.y = (uint16_t*)a->d_y;
  p.ldy = a->ldy;
  p.rows = a->rows;
  p.N = a->N;
  p.K = a->K;
  p.n_groups = a->n_groups;
  p.status = status;
  p.wait_tries = eb::wait_tries();
  p.splits = 1;
  p.w_tiled = a->w_tiled ? 1 : 0;
  p.w8 = (const uint8_t*)a->d_w8;
  // tiled weights: rows of the tensor map are the 128-byte rows of all tiles, one after the other
  const uint64_t tiled_rows = (uint64_t)a->n_groups * ((a->N + kTileN - 1) / kTileN) * ((a->K + kBlockK - 1) / kBlockK) * kTileN;
  EB_REQUIRE(!a->w_tiled || tiled_rows < (1ull << 31), EB_ERR_UNSUPPORTED, "gemm: tiled weights exceed a tensor map");

  const int KB = (a->K + kBlockK - 1) / kBlockK;
  const int nb = (a->N + kTileN - 1) / kTileN;
  int tn, token_tiles;
  if (grouped) {
    EB_REQUIRE(a->d_seg_off && a->d_work, EB_ERR_ARG, "grouped gemm: null segment offsets or workspace");
    tn = a->tile_tokens ? a->tile_tokens : pick_tn((a->rows + a->n_groups - 1) / a->n_groups);
    EB_REQUIRE(tn == 16 || tn == 32 || tn == 64 || tn == 128, EB_ERR_ARG, "gemm: tile_tokens %d not in {16,32,64,128}", tn);
    token_tiles = a->rows / tn + a->n_groups;
    const size_t need = sizeof(int32_t) * ((size_t)a->n_groups + 2 + 2 * (size_t)token_tiles);
    EB_REQUIRE(a->work_bytes >= need, EB_ERR_ARG, "grouped gemm: workspace of %zu bytes, %zu needed (eb_gemm_workspace)",
               a->work_bytes, need);
    int32_t* w = (int32_t*)a->d_work;
    int32_t* blk_off = w;
    int32_t* n_tiles = w + (a->n_groups + 1);
    int32_t* tile_group = n_tiles + 1;
    int32_t* tile_row0 = tile_group + token_tiles;
    if (!a->tiles_ready) {
      EB_CUDA(eb::launch(gemm_tiles_kernel, dim3(1), dim3(256), 0, st, a->d_seg_off, a->n_groups, tn, token_tiles, blk_off, tile_group, tile_row0,
                                           n_tiles, status));
      EB_LAUNCH_CHECK();
    }
    p.seg_off = a->d_seg_off;
    p.blk_off = blk_off;
    p.tile_group = tile_group;
    p.tile_row0 = tile_row0;
    p.n_tiles = n_tiles;
  } else {
    tn = a->tile_tokens ? a->tile_tokens : pick_tn(a->rows);
    EB_REQUIRE(tn == 16 || tn == 32 || tn == 64 || tn == 128, EB_ERR_ARG, "gemm: tile_tokens %d not in {16,32,64,128}", tn);
    // a GEMM too small to fill the GPU with 128-token tiles runs 64-token tiles before it splits K: no partial planes
    if (!a->tile_tokens && a->splits == 0 && tn == 128 && nb * ((a->rows + 127) / 128) < 120 && a->rows > 64) tn = 64;
    token_tiles = (a->rows + tn - 1) / tn;
    // split K when the tiles alone cannot fill the GPU and the caller lent a partial buffer
    int splits = a->splits;
    if (splits == 0) {
      splits = 1;
      if (a->d_work && a->rows <= kMaxSplitRows) {
        const int tiles = nb * token_tiles;
        const size_t per_split = sizeof(float) * (size_t)a->rows * a->N;
        while (tiles * splits < 120 && splits * 2 <= 8 && KB / (splits * 2) >= 4 && per_split * (splits * 2) <= a->work_bytes)
          splits *= 2;
      }
    }
    EB_REQUIRE(splits >= 1 && splits <= KB, EB_ERR_ARG, "gemm: splits %d outside 1..%d", splits, KB);
    EB_REQUIRE(splits == 1 || (a->d_work && a->rows <= kMaxSplitRows && splits <= 8), EB_ERR_ARG,
               "gemm: split K needs a workspace, at most %d rows and at most 8 splits", kMaxSplitRows);
    EB_REQUIRE(splits == 1 || sizeof(float) * (size_t)splits * a->rows * a->N <= a->work_bytes, EB_ERR_ARG,
               "gemm: %d K splits need %zu workspace bytes, the caller lent %zu", splits,
               sizeof(float) * (size_t)splits * a->rows * a->N, a->work_bytes);
    p.splits = splits;
    p.y_part = (float*)a->d_work;
  }
  EB_REQUIRE(nb <= 65535, EB_ERR_UNSUPPORTED, "gemm: %d weight tiles exceed the grid", nb);

  if (!grouped && gemm_big(a->rows, a->N, a->tile_tokens, a->splits)) {
    CUtensorMap bw, bx;
    int32_t brc = a->w_tiled ? eb::make_tmap_2d_sw128(&bw, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->d_w8, tiled_rows, kBlockK, kBlockK, kTileN)
                             : eb::make_tmap_2d_sw128(&bw, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->d_w8, (uint64_t)a->N, (uint64_t)a->K,
                                                      (uint64_t)a->K, kBigRows);
    if (brc != EB_OK) return brc;
    brc = eb::make_tmap_2d_sw128(&bx, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->d_x8, (uint64_t)a->rows, (uint64_t)a->K, (uint64_t)a->K,
                                 kBigTokens);
    if (brc != EB_OK) return brc;
    static bool configured[64] = {false};  // the attribute is per device
    int dev = 0;
    EB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
      EB_CUDA(cudaFuncSetAttribute(gemm_fp8_big_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBigSmem));
      if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const int64_t work = (int64_t)((a->rows + kBigTokens - 1) / kBigTokens) * ((a->N + kBigRows - 1) / kBigRows);
    const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(work, sm_count_now()));
    p.splits = 1;
    EB_CUDA(eb::launch(gemm_fp8_big_kernel, dim3(grid), dim3(kBigThreads), kBigSmem, st, bw, bx, p));
    if (splits_used) *splits_used = 1;
    return EB_OK;
  }

  CUtensorMap tw, tx;
  int32_t rc = a->w_tiled ? eb::make_tmap_2d_sw128(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->d_w8, tiled_rows, kBlockK, kBlockK, kTileN)
                          : eb::make_tmap_2d_sw128(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->d_w8, (uint64_t)a->n_groups * a->N,
                                                   (uint64_t)a->K, (uint64_t)a->K, kTileN);
  if (rc != EB_OK) return rc;
  rc = eb::make_tmap_2d_sw128(&tx, CU_TENSOR_MAP_DATA_TYPE_UINT8, a->d_x8, (uint64_t)a->rows, (uint64_t)a->K,
                              (uint64_t)a->K, (uint32_t)tn);
  if (rc != EB_OK) return rc;

  const int64_t work_upper = (int64_t)token_tiles * nb * p.splits;
  if (gemm_persistent(work_upper, sm_count_now())) {
    switch (tn) {
      case 16: rc = launch_gemm_persistent<16>(tw, tx, p, work_upper, st); break;
      case 32: rc = launch_gemm_persistent<32>(tw, tx, p, work_upper, st); break;
      case 64: rc = launch_gemm_persistent<64>(tw, tx, p, work_upper, st); break;
      default: rc = launch_gemm_persistent<128>(tw, tx, p, work_upper, st); break;
    }
    if (rc != EB_OK) return rc;
    if (splits_used) *splits_used = p.splits;
    if (p.splits > 1 && !splits_used) {
      const int64_t total = (int64_t)a->rows * a->N;
      EB_CUDA(eb::launch(gemm_splitk_reduce_kernel, dim3((unsigned)eb::cdiv(total, 256)), dim3(256), 0, st, p.y_part, p.y, p.ldy,
                         a->rows, a->N, p.splits));
    }
    return EB_OK;
  }
  const dim3 grid((unsigned)token_tiles, (unsigned)nb, (unsigned)p.splits);  // token tile fastest: CTAs sharing a weight tile run together
  switch (tn) {
    case 16: rc = launch_gemm<16>(tw, tx, p, grid, st); break;
    case 32: rc = launch_gemm<32>(tw, tx, p, grid, st); break;
    case 64: rc = launch_gemm<64>(tw, tx, p, grid, st); break;
    default: rc = launch_gemm<128>(tw, tx, p, grid, st); break;
  }
  if (rc != EB_OK) return rc;
  if (splits_used) *splits_used = p.splits;
  if (p.splits > 1 && !splits_used) {
    const int64_t total = (int64_t)a->rows * a->N;
    EB_CUDA(eb::launch(gemm_splitk_reduce_kernel, dim3((unsigned)eb::cdiv(total, 256)), dim3(256), 0, st, p.y_part, p.y, p.ldy, a->rows, a->N,
                                                                              p.splits));
    EB_LAUNCH_CHECK();
  }
  return EB_OK;
}

}  // namespace

extern "C" {

int32_t eb_gemm_workspace(int32_t rows, int32_t N, int32_t n_groups, size_t* bytes) {
  EB_REQUIRE(bytes && rows >= 0 && N >= 1 && n_groups >= 1, EB_ERR_ARG, "eb_gemm_workspace: bad argument");
  // grouped: blk_off[n_groups+1], n_tiles, tile_group[max], tile_row0[max] with max = rows/16 + n_groups
  const size_t max_tiles = (size_t)rows / 16 + n_groups;
  const size_t tiles_bytes = sizeof(int32_t) * ((size_t)n_groups + 2 + 2 * max_tiles);
  // dense: up to 8 split-K partials, only offered for decode-sized row counts
  const size_t split_bytes = (n_groups == 1 && rows <= kMaxSplitRows) ? sizeof(float) * 8 * (size_t)rows * N : 0;
  *bytes = tiles_bytes > split_bytes ? tiles_bytes : split_bytes;
  return EB_OK;
}

int32_t eb_gemm_fp8_block(const eb_gemm_args* a, void* stream) {
  EB_REQUIRE(a, EB_ERR_ARG, "eb_gemm_fp8_block: null args");
  EB_REQUIRE(a->n_groups == 1, EB_ERR_ARG, "eb_gemm_fp8_block: n_groups must be 1 (use eb_gemm_fp8_grouped)");
  return run_gemm(a, false, eb::as_stream(stream));
}

int32_t eb_gemm_fp8_block_partial(const eb_gemm_args* a, int32_t* splits_used, void* stream) {
  EB_REQUIRE(a && splits_used, EB_ERR_ARG, "eb_gemm_fp8_block_partial: null args");
  EB_REQUIRE(a->n_groups == 1, EB_ERR_ARG, "eb_gemm_fp8_block_partial: n_groups must be 1");
  return run_gemm(a, false, eb::as_stream(stream), splits_used);
}

int32_t eb_gemm_group_tiles(const int32_t* d_seg_off, int32_t n_groups, int32_t rows, int32_t tile_tokens, void* d_work,
                            void* stream) {
  EB_REQUIRE(d_seg_off && d_work, EB_ERR_ARG, "eb_gemm_group_tiles: null pointer");
  EB_REQUIRE(n_groups >= 1 && n_groups <= 1024 && rows >= 0, EB_ERR_ARG, "eb_gemm_group_tiles: bad size");
  EB_REQUIRE(tile_tokens == 16 || tile_tokens == 32 || tile_tokens == 64 || tile_tokens == 128, EB_ERR_ARG,
             "eb_gemm_group_tiles: tile_tokens %d not in {16,32,64,128}", tile_tokens);
  int32_t* status = eb::status_word();
  EB_REQUIRE(status, EB_ERR_NODEVICE, "eb_gemm_group_tiles: no device");
  const int token_tiles = rows / tile_tokens + n_groups;
  int32_t* w = (int32_t*)d_work;
  int32_t* n_tiles = w + (n_groups + 1);
  int32_t* tile_group = n_tiles + 1;
  EB_CUDA(eb::launch(gemm_tiles_kernel, dim3(1), dim3(256), 0, eb::as_stream(stream), d_seg_off, n_groups, tile_tokens, token_tiles, w, tile_group,
                                                          tile_group + token_tiles, n_tiles, status));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_fp8_mma_peak(int32_t blocks, int32_t reps, float* best_ms, double* tflops) {
  EB_REQUIRE(blocks >= 1 && blocks <= (1 << 16) && reps >= 1 && reps <= 64, EB_ERR_ARG, "eb_fp8_mma_peak: blocks %d / reps %d",
             blocks, reps);
  int32_t* status = eb::status_word();
  EB_REQUIRE(status, EB_ERR_NODEVICE, "eb_fp8_mma_peak: no device");
  static bool configured[64] = {false};
  int dev = 0;
  EB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    EB_CUDA(cudaFuncSetAttribute(fp8_mma_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPeakSmem));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const int sms = sm_count_now();
  cudaEvent_t e0, e1;
  EB_CUDA(cudaEventCreate(&e0));
  EB_CUDA(cudaEventCreate(&e1));
  float best = 0.f;
  cudaError_t err = cudaSuccess;
  for (int r = 0; r <= reps && err == cudaSuccess; ++r) {  // repetition 0 is a warm-up
    cudaEventRecord(e0, nullptr);
    fp8_mma_peak_kernel<<<sms, 128, kPeakSmem>>>(blocks, status, eb::wait_tries());
    cudaEventRecord(e1, nullptr);
    err = cudaGetLastError();
    if (err == cudaSuccess) err = cudaEventSynchronize(e1);
    float ms = 0.f;
    if (err == cudaSuccess) err = cudaEventElapsedTime(&ms, e0, e1);
    if (r >= 1 && (best == 0.f || ms < best)) best = ms;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (err != cudaSuccess) return eb::fail((int32_t)err, "eb_fp8_mma_peak: %s", cudaGetErrorString(err));
  if (best_ms) *best_ms = best;
  if (tflops) *tflops = best > 0.f ? 2.0 * 128 * 256 * 128 * (double)blocks * sms / (best * 1e-3) / 1e12 : 0.0;
  return EB_OK;
}

int32_t eb_weight_tiled_bytes(int32_t n_groups, int32_t N, int32_t K, size_t* bytes) {
  EB_REQUIRE(bytes && n_groups >= 1 && N >= 1 && K >= 16, EB_ERR_ARG, "eb_weight_tiled_bytes: bad argument");
  *bytes = (size_t)n_groups * ((N + kTileN - 1) / kTileN) * ((K + kBlockK - 1) / kBlockK) * (kTileN * kBlockK);
  return EB_OK;
}

int32_t eb_weight_tile_fp8(const void* d_w8, int32_t n_groups, int32_t N, int32_t K, void* d_tiled, void* stream) {
  EB_REQUIRE(d_w8 && d_tiled, EB_ERR_ARG, "eb_weight_tile_fp8: null pointer");
  EB_REQUIRE(n_groups >= 1 && N >= 1 && K >= 16 && K % 16 == 0, EB_ERR_ARG, "eb_weight_tile_fp8: bad size (K a multiple of 16)");
  EB_REQUIRE(((uintptr_t)d_w8 % 16 == 0) && ((uintptr_t)d_tiled % 16 == 0), EB_ERR_ARG, "eb_weight_tile_fp8: 16-byte alignment");
  const int64_t tiles = (int64_t)n_groups * ((N + kTileN - 1) / kTileN) * ((K + kBlockK - 1) / kBlockK);
  EB_REQUIRE(tiles < (1ll << 31), EB_ERR_UNSUPPORTED, "eb_weight_tile_fp8: too many tiles");
  weight_tile_kernel<<<(unsigned)tiles, 256, 0, eb::as_stream(stream)>>>((const uint8_t*)d_w8, (uint8_t*)d_tiled, N, K);
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_gemm_fp8_grouped(const eb_gemm_args* a, void* stream) {
  EB_REQUIRE(a, EB_ERR_ARG, "eb_gemm_fp8_grouped: null args");
  return run_gemm(a, true, eb::as_stream(stream));
}

static int32_t run_quant(int mode, const void* d_x, int64_t ldx, int32_t rows, int32_t cols, const int32_t* d_seg_off,
                         int32_t n_groups, const int32_t* d_row_map, int32_t src_rows, void* d_codes, void* d_scales,
                         void* stream) {
  EB_REQUIRE(d_x && d_codes && d_scales, EB_ERR_ARG, "quantise: null pointer");
  EB_REQUIRE(rows >= 0 && cols >= 8 && cols % 8 == 0 && ldx >= (mode ? 2 : 1) * (int64_t)cols && ldx % 8 == 0, EB_ERR_ARG,
             "quantise: cols %d / ldx %lld must be multiples of 8", cols, (long long)ldx);
  EB_REQUIRE(n_groups >= 1, EB_ERR_ARG, "quantise: n_groups %d", n_groups);
  EB_REQUIRE(((uintptr_t)d_x % 16 == 0) && ((uintptr_t)d_codes % 8 == 0), EB_ERR_ARG, "quantise: alignment");
  if (rows == 0) return EB_OK;
  int32_t* status = eb::status_word();
  EB_REQUIRE(status, EB_ERR_NODEVICE, "quantise: no device");
  const int n_blk = d_seg_off ? rows / 128 + n_groups : (rows + 127) / 128;
  EB_REQUIRE(n_blk <= 65535, EB_ERR_UNSUPPORTED, "quantise: %d row blocks exceed the grid", n_blk);
  const dim3 grid((unsigned)((cols + 127) / 128), (unsigned)n_blk);
  const bool few = (int64_t)grid.x * grid.y < 2 * (int64_t)sm_count_now();  // few CTAs: more warps each
  const uint16_t* xs = (const uint16_t*)d_x;
  uint8_t* cs = (uint8_t*)d_codes;
  float* ss = (float*)d_scales;
  cudaStream_t st = eb::as_stream(stream);
  if (mode == 0 && few)
    EB_CUDA(eb::launch(quant_act_kernel<0, 1024>, dim3(grid), dim3(1024), 0, st, xs, ldx, rows, cols, d_seg_off, n_groups, d_row_map, src_rows, cs, ss, status, QuantPeers{}));
  else if (mode == 0)
    EB_CUDA(eb::launch(quant_act_kernel<0, 512>, dim3(grid), dim3(512), 0, st, xs, ldx, rows, cols, d_seg_off, n_groups, d_row_map, src_rows, cs, ss, status, QuantPeers{}));
  else if (few)
    EB_CUDA(eb::launch(quant_act_kernel<1, 1024>, dim3(grid), dim3(1024), 0, st, xs, ldx, rows, cols, d_seg_off, n_groups, (const int32_t*)nullptr, rows, cs, ss, status, QuantPeers{}));
  else
    EB_CUDA(eb::launch(quant_act_kernel<1, 512>, dim3(grid), dim3(512), 0, st, xs, ldx, rows, cols, d_seg_off, n_groups, (const int32_t*)nullptr, rows, cs, ss, status, QuantPeers{}));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_quant_act_block128(const void* d_x, int64_t ldx, int32_t rows, int32_t cols, const int32_t* d_seg_off,
                              int32_t n_groups, void* d_codes, void* d_scales, void* stream) {
  return run_quant(0, d_x, ldx, rows, cols, d_seg_off, n_groups, nullptr, rows, d_codes, d_scales, stream);
}

int32_t eb_quant_act_block128_to_peers(eb_symm* s, const void* d_x, int64_t ldx, int32_t rows, int32_t cols, int64_t codes_off,
                                       int64_t ld_codes, int64_t scales_off, int32_t ld_scales, int32_t slice_rows, int32_t* seq,
                                       void* stream) {
  EB_REQUIRE(s && d_x && seq, EB_ERR_ARG, "eb_quant_act_block128_to_peers: null pointer");
  EB_REQUIRE(rows >= 1 && cols >= 128 && cols % 128 == 0 && ldx >= cols && ldx % 8 == 0 && ((uintptr_t)d_x % 16 == 0), EB_ERR_ARG,
             "eb_quant_act_block128_to_peers: rows %d, cols %d (a multiple of 128), ldx %lld", rows, cols, (long long)ldx);
  EB_REQUIRE(slice_rows >= 0 && slice_rows % 128 == 0, EB_ERR_ARG, "eb_quant_act_block128_to_peers: slices of %d rows (whole 128-row blocks)", slice_rows);
  eb::PeerPlanes pp;
  int32_t rc = eb::symm_peer_planes(s, 0, 0, 0, &pp, seq);  // dst[p] = base of rank p's arena
  if (rc != EB_OK) return rc;
  void* base = nullptr;
  size_t arena_bytes = 0;
  rc = eb_symm_ptr(s, pp.rank, &base, &arena_bytes);
  if (rc != EB_OK) return rc;
  const int64_t n_rb = (rows + 127) / 128, band = (int64_t)pp.size * cols;
  EB_REQUIRE(codes_off >= 0 && codes_off % 8 == 0 && ld_codes >= band && ld_codes % 8 == 0 && scales_off >= 0 && scales_off % 4 == 0 &&
                 ld_scales >= band / 128 && codes_off + (int64_t)(rows - 1) * ld_codes + band <= (int64_t)arena_bytes &&
                 scales_off + ((n_rb - 1) * ld_scales + band / 128) * 4 <= (int64_t)arena_bytes,
             EB_ERR_ARG, "eb_quant_act_block128_to_peers: the gathered operand leaves the arena of %zu bytes", arena_bytes);
  int32_t* status = eb::status_word();
  EB_REQUIRE(status, EB_ERR_NODEVICE, "eb_quant_act_block128_to_peers: no device");
  QuantPeers qp = {};
  qp.size = pp.size;
  qp.ldc = ld_codes;
  qp.lds = ld_scales;
  qp.chunk = slice_rows;
  qp.arrive = pp;
  for (int p = 0; p < pp.size; ++p) {
    qp.codes[p] = pp.dst[p] + codes_off + (int64_t)pp.rank * cols;
    qp.scales[p] = reinterpret_cast<float*>(pp.dst[p] + scales_off) + (int64_t)pp.rank * (cols / 128);
  }
  const dim3 grid((unsigned)(cols / 128), (unsigned)n_rb);
  EB_CUDA(eb::launch(quant_act_kernel<0, 1024>, dim3(grid), dim3(1024), 0, eb::as_stream(stream), (const uint16_t*)d_x, ldx, rows, cols,
                     (const int32_t*)nullptr, 1, (const int32_t*)nullptr, rows, (uint8_t*)nullptr, (float*)nullptr, status, qp));
  EB_LAUNCH_CHECK();
  return EB_OK;
}

int32_t eb_quant_gather_block128(const void* d_x, int64_t ldx, int32_t src_rows, const int32_t* d_row_map, int32_t rows,
                                 int32_t cols, const int32_t* d_seg_off, int32_t n_groups, void* d_codes,
                                 void* d_scales, void* stream) {
  EB_REQUIRE(d_row_map && src_rows >= 1, EB_ERR_ARG, "eb_quant_gather_block128: null row map");
  return run_quant(0, d_x, ldx, rows, cols, d_seg_off, n_groups, d_row_map, src_rows, d_codes, d_scales, stream);
}

int32_t eb_quant_silu_mul_block128(const void* d_gate_up, int64_t ld, int32_t rows, int32_t cols,
                                   const int32_t* d_seg_off, int32_t n_groups, void* d_codes, void* d_scales,
                                   void* stream) {
  return run_quant(1, d_gate_up, ld, rows, cols, d_seg_off, n_groups, nullptr, rows, d_codes, d_scales, stream);
}

}  // extern "C"

/*
 * TEST INFRASTRUCTURE -- not part of the product.  Only tests/, the smoke check
 * and the benchmark's CPU-baseline leg may load this code.
 *
 * Host evaluation of the synthetic-tensor definition in include/eb_synth.h.
 * This translation unit is compiled with -ffp-contract=off so that every
 * operation rounds exactly as the device intrinsics do.
 *
 * Parity unpinned: the reference project (eidola-ai/eidola) contains no tensor
 * code and no golden vectors for this path; see oracle.cpp's header.
 */
#include <stdint.h>
#include <stddef.h>

#include <omp.h>
#include <pthread.h>
#include <sched.h>

#include "../include/eb_synth.h"

extern "C" {

/* Threads the oracle may use (launchers such as torchrun export OMP_NUM_THREADS=1); returns the value in effect. */
int orc_set_threads(int n) {
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
}

/* The same, and every worker thread but the calling one is pinned to one of the CPUs the process may run on (worker t
 * to the t-th allowed CPU, round robin), so that repeated timings see the same placement.  The calling thread keeps
 * its affinity: the host program's own scheduling is left alone.  Returns the number of threads. */
int orc_set_threads_pinned(int n) {
  cpu_set_t allowed;
  CPU_ZERO(&allowed);
  int cpus[1024], n_cpu = 0;
  if (sched_getaffinity(0, sizeof(allowed), &allowed) == 0)
    for (int c = 0; c < CPU_SETSIZE && n_cpu < 1024; ++c)
      if (CPU_ISSET(c, &allowed)) cpus[n_cpu++] = c;
  if (n > 0) omp_set_num_threads(n);
  const int nt = omp_get_max_threads();
  if (n_cpu > 0) {
#pragma omp parallel num_threads(nt)
    {
      const int t = omp_get_thread_num();
      if (t > 0) {
        cpu_set_t one;
        CPU_ZERO(&one);
        CPU_SET(cpus[t % n_cpu], &one);
        pthread_setaffinity_np(pthread_self(), sizeof(one), &one);
      }
    }
  }
  return nt;
}

/* out[i] = scale * N(0,1)(seed, stream, idx0 + i) */
void orc_synth_normal_f32(uint64_t seed, uint64_t stream, uint64_t idx0, int64_t n, float scale, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) out[i] = eb_normal(seed, stream, idx0 + (uint64_t)i) * scale;
}

void orc_synth_normal_bf16(uint64_t seed, uint64_t stream, uint64_t idx0, int64_t n, float scale, uint16_t* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) out[i] = eb_bf16_from_f32(eb_normal(seed, stream, idx0 + (uint64_t)i) * scale);
}

void orc_synth_uniform_f32(uint64_t seed, uint64_t stream, uint64_t idx0, int64_t n, float lo, float hi, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) out[i] = eb_uniform(seed, stream, idx0 + (uint64_t)i, lo, hi);
}

/* e4m3 codes whose decoded values are round(N(0,1)*scale) -- used for the GEMM sweep inputs. */
void orc_synth_normal_e4m3(uint64_t seed, uint64_t stream, uint64_t idx0, int64_t n, float scale, uint8_t* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) out[i] = eb_f32_to_e4m3(eb_normal(seed, stream, idx0 + (uint64_t)i) * scale);
}

void orc_e4m3_encode(const float* x, uint8_t* q, int64_t n) {
  for (int64_t i = 0; i < n; ++i) q[i] = eb_f32_to_e4m3(x[i]);
}
void orc_e4m3_decode(const uint8_t* q, float* x, int64_t n) {
  for (int64_t i = 0; i < n; ++i) x[i] = eb_e4m3_to_f32(q[i]);
}
void orc_bf16_encode(const float* x, uint16_t* h, int64_t n) {
  for (int64_t i = 0; i < n; ++i) h[i] = eb_bf16_from_f32(x[i]);
}
void orc_bf16_decode(const uint16_t* h, float* x, int64_t n) {
  for (int64_t i = 0; i < n; ++i) x[i] = eb_bf16_to_f32(h[i]);
}

/*
 * Random-init weight block generator: W[r][c] = std * N(0,1)(seed, stream, r*cols + c),
 * quantised per 128x128 block: s = amax/448 (1 if the block is all zero), code = e4m3(W/s).
 * codes: [rows][cols] row-major; scales: [ceil(rows/128)][ceil(cols/128)].
 * row0/nrows select a horizontal band of the global tensor (row0 must be a multiple of 128),
 * so a rank can generate only its shard; indices stay global.
 */
void orc_synth_weight_fp8(uint64_t seed, uint64_t stream, int64_t rows_total, int64_t cols, int64_t row0, int64_t nrows,
                          float std, uint8_t* codes, float* scales) {
  (void)rows_total;
  const int64_t rb = (nrows + 127) / 128, cb = (cols + 127) / 128;
#pragma omp parallel for schedule(dynamic) collapse(2)
  for (int64_t br = 0; br < rb; ++br) {
    for (int64_t bc = 0; bc < cb; ++bc) {
      const int64_t r_lo = br * 128, r_hi = (r_lo + 128 < nrows) ? r_lo + 128 : nrows;
      const int64_t c_lo = bc * 128, c_hi = (c_lo + 128 < cols) ? c_lo + 128 : cols;
      float amax = 0.f;
      for (int64_t r = r_lo; r < r_hi; ++r)
        for (int64_t c = c_lo; c < c_hi; ++c) {
          float v = eb_normal(seed, stream, (uint64_t)((row0 + r) * cols + c)) * std;
          float a = v < 0 ? -v : v;
          if (a > amax) amax = a;
        }
      const float s = amax > 0.f ? amax / 448.0f : 1.0f;
      scales[br * cb + bc] = s;
      for (int64_t r = r_lo; r < r_hi; ++r)
        for (int64_t c = c_lo; c < c_hi; ++c) {
          float v = eb_normal(seed, stream, (uint64_t)((row0 + r) * cols + c)) * std;
          codes[r * cols + c] = eb_f32_to_e4m3(v / s);
        }
    }
  }
}

/*
 * Activation quantiser: bf16 rows -> e4m3 with one fp32 scale per (128-row block, 128-column block).
 * Rows are grouped in segments (seg_off[n_seg+1]); 128-row blocks restart at each segment start, so a
 * grouped (per-expert) GEMM sees whole blocks.  Block index of (segment g, block b) = blk_off[g] + b where
 * blk_off is the exclusive prefix sum of ceil(len_g/128).  scales: [n_blocks][ceil(cols/128)].
 */
void orc_quant_act_block128(const uint16_t* x, int64_t cols, const int32_t* seg_off, int32_t n_seg, uint8_t* codes,
                            float* scales) {
  const int64_t cb = (cols + 127) / 128;
  int64_t blk = 0;
  for (int32_t g = 0; g < n_seg; ++g) {
    const int64_t lo = seg_off[g], hi = seg_off[g + 1];
    for (int64_t r0 = lo; r0 < hi; r0 += 128, ++blk) {
      const int64_t r1 = (r0 + 128 < hi) ? r0 + 128 : hi;
      for (int64_t bc = 0; bc < cb; ++bc) {
        const int64_t c0 = bc * 128, c1 = (c0 + 128 < cols) ? c0 + 128 : cols;
        float amax = 0.f;
        for (int64_t r = r0; r < r1; ++r)
          for (int64_t c = c0; c < c1; ++c) {
            float v = eb_bf16_to_f32(x[r * cols + c]);
            float a = v < 0 ? -v : v;
            if (a > amax) amax = a;
          }
        const float s = amax > 0.f ? amax / 448.0f : 1.0f;
        scales[blk * cb + bc] = s;
        for (int64_t r = r0; r < r1; ++r)
          for (int64_t c = c0; c < c1; ++c) codes[r * cols + c] = eb_f32_to_e4m3(eb_bf16_to_f32(x[r * cols + c]) / s);
      }
    }
  }
}

} /* extern "C" */

/*
 * TEST INFRASTRUCTURE -- not part of the product.  Only tests/, the smoke check
 * and the benchmark's CPU-baseline leg may load this code; the CUDA library never
 * links, loads or calls it.
 *
 * Plain CPU restatement of the decode-step math: block-scaled e4m3 GEMM, paged
 * KV append, paged sink attention (full and sliding-window layers, GQA, ragged
 * query lengths), RMSNorm, rotary embedding, top-k router, gated-MLP experts,
 * greedy argmax, and a whole decoder step built from them.
 *
 * PARITY UNPINNED.  The reference project (eidola-ai/eidola) does not contain
 * this arithmetic in any language: its server forwards chat requests to a remote
 * provider (crates/eidola-server/src/backend.rs:421-433, docs/server.md:102-104)
 * and its client supervises a third-party `llama-server` child process
 * (crates/eidola-app-core/src/local_models.rs:1612-1626; llama.cpp tag b9960 pinned
 * in flake.nix:614-623, source not vendored).  No reference test asserts a logit, a
 * token id, a block table or a routing decision.  The math below therefore follows
 * the written configuration of the benchmark (head counts, page size, window,
 * sink term in the softmax denominator, per-128x128 block scales, top-4 softmax
 * routing), and the choices that configuration leaves open are fixed here:
 *   RMSNorm eps 1e-5 with fp32 reduction; rotary = rotate-half pairs (i, i+D/2);
 *   experts = down( silu(gate(x)) * up(x) ); router weights bf16, logits fp32 with
 *   a fixed 32-lane strided summation order; residual stream bf16; LM head fp8
 *   block-scaled like every other linear; ties in top-k and argmax go to the lower index.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <vector>

#include "../include/eb_synth.h"

namespace {

inline float bf(uint16_t h) { return eb_bf16_to_f32(h); }
inline uint16_t tobf(float f) { return eb_bf16_from_f32(f); }

struct E4Table {
  float v[256];
  E4Table() {
    for (int i = 0; i < 256; ++i) v[i] = eb_e4m3_to_f32((uint8_t)i);
  }
};
const E4Table g_e4;

inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

/* Sum of 16 lane accumulators in a fixed tree order. */
inline float tree16(const float* a) {
  float b[8];
  for (int i = 0; i < 8; ++i) b[i] = a[i] + a[i + 8];
  for (int i = 0; i < 4; ++i) b[i] = b[i] + b[i + 4];
  return (b[0] + b[2]) + (b[1] + b[3]);
}

/*
 * One row-segment times one weight matrix:
 *   y[m][n] = bf16( sum_kb sx[xb(m)][kb] * sw[n/128][kb] * sum_{k in kb} X8[m][k] * W8[n][k] )
 * X rows [m0, m1) all belong to the same 128-row scale block `xblk`.
 */
void gemm_rows(const uint8_t* x8, const float* sx_row, const uint8_t* w8, const float* sw, int64_t m0, int64_t m1,
               int64_t N, int64_t K, uint16_t* y, int64_t ldy) {
  const int64_t kb_n = cdiv(K, 128);
  const int64_t rows = m1 - m0;
  std::vector<float> xf((size_t)rows * K);
  for (int64_t m = 0; m < rows; ++m)
    for (int64_t k = 0; k < K; ++k) xf[m * K + k] = g_e4.v[x8[(m0 + m) * K + k]];
#pragma omp parallel
  {
    std::vector<float> wf((size_t)K);
#pragma omp for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
      for (int64_t k = 0; k < K; ++k) wf[k] = g_e4.v[w8[n * K + k]];
      const float* swn = sw + (n / 128) * kb_n;
      for (int64_t m = 0; m < rows; ++m) {
        const float* xr = &xf[m * K];
        float total = 0.f;
        for (int64_t kb = 0; kb < kb_n; ++kb) {
          const int64_t k0 = kb * 128, k1 = std::min<int64_t>(k0 + 128, K);
          float acc[16] = {0};
          for (int64_t k = k0; k < k1; k += 16)
            for (int j = 0; j < 16; ++j) acc[j] += xr[k + j] * wf[k + j]; /* K is a multiple of 16 */
          total += (sx_row[kb] * swn[kb]) * tree16(acc);
        }
        y[(m0 + m) * ldy + n] = tobf(total);
      }
    }
  }
}

} /* namespace */

extern "C" {

/* ------------------------------------------------------------------ GEMM */

/*
 * Grouped block-scaled GEMM.  Rows of X are grouped in segments seg_off[n_groups+1]; group g multiplies
 * by W8 + g*N*K (row-major [N][K]) with scales sw + g*ceil(N/128)*ceil(K/128).  Activation scale rows are
 * indexed by the running 128-row block number (blocks restart at each segment start).  n_groups == 1 with
 * seg_off = {0, M} is the dense case.  K must be a multiple of 16.
 */
void orc_gemm_fp8_grouped(const uint8_t* x8, const float* sx, const int32_t* seg_off, int32_t n_groups,
                          const uint8_t* w8, const float* sw, int64_t N, int64_t K, uint16_t* y) {
  const int64_t kb_n = cdiv(K, 128), nb_n = cdiv(N, 128);
  int64_t blk = 0;
  for (int32_t g = 0; g < n_groups; ++g) {
    const int64_t lo = seg_off[g], hi = seg_off[g + 1];
    for (int64_t r0 = lo; r0 < hi; r0 += 128, ++blk) {
      const int64_t r1 = std::min<int64_t>(r0 + 128, hi);
      gemm_rows(x8, sx + blk * kb_n, w8 + (int64_t)g * N * K, sw + (int64_t)g * nb_n * kb_n, r0, r1, N, K, y, N);
    }
  }
}

void orc_gemm_fp8_block(const uint8_t* x8, const float* sx, const uint8_t* w8, const float* sw, int64_t M, int64_t N,
                        int64_t K, uint16_t* y) {
  int32_t seg[2] = {0, (int32_t)M};
  orc_gemm_fp8_grouped(x8, sx, seg, 1, w8, sw, N, K, y);
}

/* ------------------------------------------------------------ KV cache */

/*
 * Cache layout of one layer: [num_pages][2 (K,V)][n_kv][page_size][head_dim] bf16.
 * Token at absolute position p of sequence slot s lives in page block_tables[s*bt_stride + p/page_size],
 * slot p % page_size.  k_new/v_new: [T][n_kv][head_dim] with a row stride (elements) so the K and V
 * slices of a fused QKV buffer can be passed directly.
 */
void orc_kv_append(uint16_t* cache, int32_t n_kv, int32_t head_dim, int32_t page_size, const uint16_t* k_new,
                   const uint16_t* v_new, int64_t row_stride, const int32_t* block_tables, int32_t bt_stride,
                   const int32_t* tok_seq, const int32_t* positions, int32_t T) {
  const int64_t head_sz = (int64_t)page_size * head_dim;
  const int64_t page_sz = 2 * n_kv * head_sz;
  for (int32_t t = 0; t < T; ++t) {
    const int32_t s = tok_seq[t], p = positions[t];
    const int64_t page = block_tables[(int64_t)s * bt_stride + p / page_size];
    const int32_t slot = p % page_size;
    for (int32_t h = 0; h < n_kv; ++h) {
      uint16_t* kd = cache + page * page_sz + (int64_t)h * head_sz + (int64_t)slot * head_dim;
      uint16_t* vd = cache + page * page_sz + (int64_t)(n_kv + h) * head_sz + (int64_t)slot * head_dim;
      memcpy(kd, k_new + t * row_stride + (int64_t)h * head_dim, 2 * head_dim);
      memcpy(vd, v_new + t * row_stride + (int64_t)h * head_dim, 2 * head_dim);
    }
  }
}

/* ----------------------------------------------------------- attention */

/*
 * Paged sink attention for a ragged batch.
 *   q, out : [T][n_q][head_dim] bf16 with row strides; tokens of sequence i are rows q_off[i] .. q_off[i+1]-1
 *   ctx_lens[i] counts every token of the sequence already in the cache, the q_len new ones included;
 *   query j of sequence i sits at absolute position p = ctx_lens[i] - q_len + j.
 *   visible keys: t <= p, and t > p - window when window > 0.
 *   s_t = (q . k_t) * scale;  m = max(sink_h, max_t s_t);
 *   out = sum_t exp(s_t - m) v_t / ( exp(sink_h - m) + sum_t exp(s_t - m) )
 */
void orc_attn_paged_sink(const uint16_t* q, int64_t q_stride, const uint16_t* cache, const int32_t* block_tables,
                         int32_t bt_stride, const int32_t* seq_slots, const int32_t* q_off, const int32_t* ctx_lens,
                         int32_t n_seqs, const float* sinks, int32_t window, int32_t n_q, int32_t n_kv,
                         int32_t head_dim, int32_t page_size, float scale, uint16_t* out, int64_t out_stride) {
  const int64_t head_sz = (int64_t)page_size * head_dim;
  const int64_t page_sz = 2 * n_kv * head_sz;
  const int32_t group = n_q / n_kv;
#pragma omp parallel for schedule(dynamic) collapse(2)
  for (int32_t i = 0; i < n_seqs; ++i) {
    for (int32_t h = 0; h < n_q; ++h) {
      const int32_t slot_id = seq_slots[i];
      const int32_t q_len = q_off[i + 1] - q_off[i];
      const int32_t L = ctx_lens[i];
      const int32_t hk = h / group;
      std::vector<float> s((size_t)L);
      for (int32_t j = 0; j < q_len; ++j) {
        const int32_t p = L - q_len + j;
        const int32_t t_lo = (window > 0) ? std::max(0, p - window + 1) : 0;
        const uint16_t* qr = q + (int64_t)(q_off[i] + j) * q_stride + (int64_t)h * head_dim;
        float m = sinks[h];
        for (int32_t t = t_lo; t <= p; ++t) {
          const int64_t page = block_tables[(int64_t)slot_id * bt_stride + t / page_size];
          const uint16_t* kr = cache + page * page_sz + (int64_t)hk * head_sz + (int64_t)(t % page_size) * head_dim;
          float d = 0.f;
          for (int32_t c = 0; c < head_dim; ++c) d += bf(qr[c]) * bf(kr[c]);
          s[t] = d * scale;
          m = std::max(m, s[t]);
        }
        double denom = exp((double)sinks[h] - (double)m);
        std::vector<double> acc((size_t)head_dim, 0.0);
        for (int32_t t = t_lo; t <= p; ++t) {
          const int64_t page = block_tables[(int64_t)slot_id * bt_stride + t / page_size];
          const uint16_t* vr =
              cache + page * page_sz + (int64_t)(n_kv + hk) * head_sz + (int64_t)(t % page_size) * head_dim;
          const double e = exp((double)s[t] - (double)m);
          denom += e;
          for (int32_t c = 0; c < head_dim; ++c) acc[c] += e * (double)bf(vr[c]);
        }
        uint16_t* orow = out + (int64_t)(q_off[i] + j) * out_stride + (int64_t)h * head_dim;
        for (int32_t c = 0; c < head_dim; ++c) orow[c] = tobf((float)(acc[c] / denom));
      }
    }
  }
}

/* ---------------------------------------------------------------- glue */

/* y = bf16( (x * r) * g ), r = 1 / sqrt(ss / H + eps), fp32 arithmetic with every operation rounded once.
 * The sum of squares ss follows a fixed order, the one a 256-thread row kernel uses: partial sum t of 256 takes the
 * 8-column chunks t, t + 256, ... in ascending column order with fused multiply-adds; each group of 32 partial sums
 * is combined by an xor butterfly (offsets 16, 8, 4, 2, 1), and the 8 group sums are added in ascending order. */
void orc_rmsnorm(const uint16_t* x, const float* g, int64_t T, int64_t H, float eps, uint16_t* y) {
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < T; ++t) {
    float part[256];
    for (int p = 0; p < 256; ++p) {
      float ss = 0.f;
      for (int64_t c0 = (int64_t)p * 8; c0 < H; c0 += 256 * 8)
        for (int64_t c = c0; c < std::min(c0 + 8, H); ++c) {
          const float v = bf(x[t * H + c]);
          ss = fmaf(v, v, ss);
        }
      part[p] = ss;
    }
    float total = 0.f;
    for (int w = 0; w < 8; ++w) {
      float a[32], b[32];
      for (int l = 0; l < 32; ++l) a[l] = part[w * 32 + l];
      for (int o = 16; o; o >>= 1) {
        for (int l = 0; l < 32; ++l) b[l] = a[l] + a[l ^ o];
        for (int l = 0; l < 32; ++l) a[l] = b[l];
      }
      total += a[0];
    }
    const float r = 1.0f / sqrtf(total / (float)H + eps);
    for (int64_t c = 0; c < H; ++c) y[t * H + c] = tobf((bf(x[t * H + c]) * r) * g[c]);
  }
}

/* cos/sin table [max_pos][head_dim/2]: angle = pos * theta^(-2i/head_dim), evaluated in double. */
void orc_rope_table(int32_t max_pos, int32_t head_dim, double theta, float* cos_t, float* sin_t) {
  const int32_t half = head_dim / 2;
#pragma omp parallel for schedule(static)
  for (int32_t p = 0; p < max_pos; ++p)
    for (int32_t i = 0; i < half; ++i) {
      const double inv = pow(theta, -2.0 * (double)i / (double)head_dim);
      const double a = (double)p * inv;
      cos_t[(int64_t)p * half + i] = (float)cos(a);
      sin_t[(int64_t)p * half + i] = (float)sin(a);
    }
}

/*
 * In-place rotary embedding of n_heads heads starting at x (row stride in elements):
 *   (a, b) = (x[i], x[i + D/2]);  x[i] = a*cos - b*sin;  x[i + D/2] = b*cos + a*sin;  bf16 rounding of each.
 */
void orc_rope(uint16_t* x, int64_t row_stride, int32_t n_heads, int32_t head_dim, const int32_t* positions, int32_t T,
              const float* cos_t, const float* sin_t) {
  const int32_t half = head_dim / 2;
  for (int32_t t = 0; t < T; ++t)
    for (int32_t h = 0; h < n_heads; ++h) {
      uint16_t* r = x + (int64_t)t * row_stride + (int64_t)h * head_dim;
      for (int32_t i = 0; i < half; ++i) {
        const float c = cos_t[(int64_t)positions[t] * half + i], s = sin_t[(int64_t)positions[t] * half + i];
        const float a = bf(r[i]), b = bf(r[i + half]);
        r[i] = tobf(a * c - b * s);
        r[i + half] = tobf(b * c + a * s);
      }
    }
}

/* x = bf16(x + y) */
void orc_residual_add(uint16_t* x, const uint16_t* y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) x[i] = tobf(bf(x[i]) + bf(y[i]));
}

void orc_embed(const uint16_t* table, int64_t H, const int32_t* tokens, int32_t T, uint16_t* x) {
  for (int32_t t = 0; t < T; ++t) memcpy(x + (int64_t)t * H, table + (int64_t)tokens[t] * H, 2 * H);
}

/* ----------------------------------------------------------------- MoE */

/*
 * Router.  logit[t][e] = sum_k x[t][k]*wr[e][k] in fp32 with this exact order: the row is cut in groups of 8
 * consecutive elements; lane l (0..31) owns groups l, l+32, l+64, ... and adds their products in ascending k with
 * fmaf (each product of two bf16 is exact in fp32); then the 32 lane sums are combined by a butterfly:
 * for off in 16,8,4,2,1: a[l] += a[l ^ off].  top_k by value, ties to the lower expert index; weights = softmax
 * over the selected logits.  H must be a multiple of 8.
 */
void orc_router_topk(const uint16_t* x, const uint16_t* wr, int32_t T, int32_t E, int32_t H, int32_t top_k,
                     int32_t* idx, float* wts, float* logits_out) {
#pragma omp parallel for schedule(static)
  for (int32_t t = 0; t < T; ++t) {
    std::vector<float> lg((size_t)E);
    for (int32_t e = 0; e < E; ++e) {
      float a[32];
      for (int l = 0; l < 32; ++l) {
        float acc = 0.f;
        for (int32_t g = l; g < H / 8; g += 32)
          for (int32_t k = 8 * g; k < 8 * g + 8; ++k) acc = fmaf(bf(x[(int64_t)t * H + k]), bf(wr[(int64_t)e * H + k]), acc);
        a[l] = acc;
      }
      for (int off = 16; off >= 1; off >>= 1) {
        float b[32];
        for (int l = 0; l < 32; ++l) b[l] = a[l] + a[l ^ off];
        memcpy(a, b, sizeof(a));
      }
      lg[e] = a[0];
      if (logits_out) logits_out[(int64_t)t * E + e] = a[0];
    }
    std::vector<char> used((size_t)E, 0);
    float sel[64];
    for (int32_t j = 0; j < top_k; ++j) {
      int32_t best = -1;
      for (int32_t e = 0; e < E; ++e)
        if (!used[e] && (best < 0 || lg[e] > lg[best])) best = e;
      used[best] = 1;
      idx[(int64_t)t * top_k + j] = best;
      sel[j] = lg[best];
    }
    float den = 0.f, ex[64];
    for (int32_t j = 0; j < top_k; ++j) {
      ex[j] = expf(sel[j] - sel[0]);
      den += ex[j];
    }
    for (int32_t j = 0; j < top_k; ++j) wts[(int64_t)t * top_k + j] = ex[j] / den;
  }
}

/*
 * Token -> expert permutation.  Slots (t, j) are ordered by (expert, t, j).  seg_off[E+1] are the expert
 * segment bounds in the permuted row space, perm_row[t*top_k + j] the permuted row of slot (t, j).
 */
void orc_moe_permute(const int32_t* idx, int32_t T, int32_t top_k, int32_t E, int32_t* seg_off, int32_t* perm_row) {
  std::vector<int32_t> cnt((size_t)E + 1, 0);
  for (int64_t i = 0; i < (int64_t)T * top_k; ++i) cnt[idx[i] + 1]++;
  for (int32_t e = 0; e < E; ++e) cnt[e + 1] += cnt[e];
  for (int32_t e = 0; e <= E; ++e) seg_off[e] = cnt[e];
  std::vector<int32_t> cur(cnt.begin(), cnt.end() - 1);
  for (int64_t i = 0; i < (int64_t)T * top_k; ++i) perm_row[i] = cur[idx[i]]++;
}

/*
 * Mixture of experts on normalised activations h [T][H] bf16:
 *   rows gathered by perm -> quantise (blocks per expert segment) -> gate_up = GEMM(W1[e]) [2I]
 *   -> act = bf16(silu(gate) * up) -> quantise -> y = GEMM(W2[e]) [H]
 *   -> out[t] = bf16( sum_j w[t][j] * y[perm(t,j)] ) accumulated in fp32 for j = 0..top_k-1 in order.
 */
void orc_quant_act_block128(const uint16_t* x, int64_t cols, const int32_t* seg_off, int32_t n_seg, uint8_t* codes,
                            float* scales);

void orc_moe_forward(const uint16_t* h, int32_t T, int32_t H, int32_t I, int32_t E, int32_t top_k, const int32_t* idx,
                     const float* wts, const uint8_t* w1, const float* s1, const uint8_t* w2, const float* s2,
                     uint16_t* out) {
  const int64_t R = (int64_t)T * top_k;
  std::vector<int32_t> seg((size_t)E + 1), perm((size_t)R);
  orc_moe_permute(idx, T, top_k, E, seg.data(), perm.data());
  int64_t n_blk = 0;
  for (int32_t e = 0; e < E; ++e) n_blk += cdiv(seg[e + 1] - seg[e], 128);
  const int64_t kbH = cdiv(H, 128), kbI = cdiv(I, 128);
  std::vector<uint16_t> xp((size_t)R * H);
  for (int32_t t = 0; t < T; ++t)
    for (int32_t j = 0; j < top_k; ++j)
      memcpy(&xp[(int64_t)perm[(int64_t)t * top_k + j] * H], h + (int64_t)t * H, 2 * (size_t)H);
  std::vector<uint8_t> x8((size_t)R * H);
  std::vector<float> sx((size_t)std::max<int64_t>(n_blk, 1) * kbH);
  orc_quant_act_block128(xp.data(), H, seg.data(), E, x8.data(), sx.data());
  std::vector<uint16_t> gu((size_t)R * 2 * I);
  orc_gemm_fp8_grouped(x8.data(), sx.data(), seg.data(), E, w1, s1, 2 * (int64_t)I, H, gu.data());
  std::vector<uint16_t> act((size_t)R * I);
  for (int64_t r = 0; r < R; ++r)
    for (int32_t c = 0; c < I; ++c) {
      const float g = bf(gu[r * 2 * I + c]), u = bf(gu[r * 2 * I + I + c]);
      act[r * I + c] = tobf(g / (1.0f + expf(-g)) * u);
    }
  std::vector<uint8_t> a8((size_t)R * I);
  std::vector<float> sa((size_t)std::max<int64_t>(n_blk, 1) * kbI);
  orc_quant_act_block128(act.data(), I, seg.data(), E, a8.data(), sa.data());
  std::vector<uint16_t> y((size_t)R * H);
  orc_gemm_fp8_grouped(a8.data(), sa.data(), seg.data(), E, w2, s2, H, I, y.data());
  for (int32_t t = 0; t < T; ++t)
    for (int32_t c = 0; c < H; ++c) {
      float acc = 0.f;
      for (int32_t j = 0; j < top_k; ++j)
        acc = fmaf(wts[(int64_t)t * top_k + j], bf(y[(int64_t)perm[(int64_t)t * top_k + j] * H + c]), acc);
      out[(int64_t)t * H + c] = tobf(acc);
    }
}

/* greedy argmax over bf16 logits, ties to the lower id; margin = top1 - top2 (fp32 of the bf16 values).
 * NaN logits are never chosen; a row without any value above -inf yields token 0. */
void orc_argmax(const uint16_t* logits, int32_t T, int64_t V, int32_t* tok, float* margin) {
#pragma omp parallel for schedule(static)
  for (int32_t t = 0; t < T; ++t) {
    const uint16_t* r = logits + (int64_t)t * V;
    int64_t b = 0;
    float bv = -INFINITY, sv = -INFINITY;
    for (int64_t v = 0; v < V; ++v) {
      const float x = bf(r[v]);
      if (x > bv) {
        sv = bv;
        bv = x;
        b = v;
      } else if (x > sv) {
        sv = x;
      }
    }
    tok[t] = (int32_t)b;
    if (margin) margin[t] = bv - sv;
  }
}

} /* extern "C" */

/*
 * TEST INFRASTRUCTURE -- not part of the product (see oracle.cpp's header; parity unpinned: the reference project
 * contains no decoder).
 *
 * A whole decoder on the CPU, assembled from the oracle's operators: random-init weights regenerated from
 * (shape, seed) with the generator of include/eb_synth.h, a paged KV cache, and one ragged decode / verify step
 *   embed -> [ rmsnorm -> e4m3 -> QKV -> rotary -> KV append -> paged sink attention -> e4m3 -> O -> residual
 *              -> rmsnorm -> router top-k -> experts (W1, silu*up, W2) -> combine -> residual ] x layers
 *         -> rmsnorm -> e4m3 -> LM head -> greedy argmax (+ top-2 margin).
 * Even layers use the sliding window, odd layers attend to everything.  Block tables come from the caller.
 */
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <vector>

#include "../include/eb_synth.h"
#include "../include/eidola_b200.h"

extern "C" {
void orc_synth_normal_f32(uint64_t, uint64_t, uint64_t, int64_t, float, float*);
void orc_synth_normal_bf16(uint64_t, uint64_t, uint64_t, int64_t, float, uint16_t*);
void orc_synth_weight_fp8(uint64_t, uint64_t, int64_t, int64_t, int64_t, int64_t, float, uint8_t*, float*);
void orc_quant_act_block128(const uint16_t*, int64_t, const int32_t*, int32_t, uint8_t*, float*);
void orc_gemm_fp8_block(const uint8_t*, const float*, const uint8_t*, const float*, int64_t, int64_t, int64_t, uint16_t*);
void orc_kv_append(uint16_t*, int32_t, int32_t, int32_t, const uint16_t*, const uint16_t*, int64_t, const int32_t*, int32_t,
                   const int32_t*, const int32_t*, int32_t);
void orc_attn_paged_sink(const uint16_t*, int64_t, const uint16_t*, const int32_t*, int32_t, const int32_t*, const int32_t*,
                         const int32_t*, int32_t, const float*, int32_t, int32_t, int32_t, int32_t, int32_t, float, uint16_t*,
                         int64_t);
void orc_rmsnorm(const uint16_t*, const float*, int64_t, int64_t, float, uint16_t*);
void orc_rope_table(int32_t, int32_t, double, float*, float*);
void orc_rope(uint16_t*, int64_t, int32_t, int32_t, const int32_t*, int32_t, const float*, const float*);
void orc_residual_add(uint16_t*, const uint16_t*, int64_t);
void orc_embed(const uint16_t*, int64_t, const int32_t*, int32_t, uint16_t*);
void orc_router_topk(const uint16_t*, const uint16_t*, int32_t, int32_t, int32_t, int32_t, int32_t*, float*, float*);
void orc_moe_forward(const uint16_t*, int32_t, int32_t, int32_t, int32_t, int32_t, const int32_t*, const float*,
                     const uint8_t*, const float*, const uint8_t*, const float*, uint16_t*);
void orc_argmax(const uint16_t*, int32_t, int64_t, int32_t*, float*);
}

namespace {

inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline uint64_t sid(int layer, int kind, int expert) {
  return ((uint64_t)(layer + 1) << 20) | ((uint64_t)kind << 12) | (uint64_t)expert;
}

struct W8 {
  std::vector<uint8_t> codes;
  std::vector<float> scales;
  void gen(uint64_t seed, uint64_t stream, int64_t rows, int64_t cols, float std, int64_t group = 0, int64_t groups = 1) {
    if (codes.empty()) {
      codes.resize((size_t)(groups * rows * cols));
      scales.resize((size_t)(groups * cdiv(rows, 128) * cdiv(cols, 128)));
    }
    orc_synth_weight_fp8(seed, stream, rows, cols, 0, rows, std, codes.data() + group * rows * cols,
                         scales.data() + group * cdiv(rows, 128) * cdiv(cols, 128));
  }
};

struct LayerW {
  W8 wqkv, wo, w1, w2;
  std::vector<uint16_t> wr;
  std::vector<float> sinks, g_attn, g_mlp;
  std::vector<uint16_t> cache;
};

}  // namespace

struct orc_model {
  eb_config c;
  int nqkv, hqd;
  std::vector<LayerW> layers;
  std::vector<uint16_t> embed;
  W8 lm;
  std::vector<float> g_final, rope_cos, rope_sin;
  /* intermediates of the last layer of the last step: rotated q | k | v rows, attention output, O projection */
  std::vector<uint16_t> last_qkv, last_att, last_o;
};

extern "C" {

orc_model* orc_model_create(const eb_config* cfg) {
  orc_model* m = new orc_model;
  m->c = *cfg;
  const eb_config& c = m->c;
  const int H = c.hidden, I = c.inter, E = c.n_experts;
  m->hqd = c.n_q_heads * c.head_dim;
  m->nqkv = (c.n_q_heads + 2 * c.n_kv_heads) * c.head_dim;
  m->layers.resize((size_t)c.n_layers);
  for (int l = 0; l < c.n_layers; ++l) {
    LayerW& L = m->layers[(size_t)l];
    L.wqkv.gen(c.seed, sid(l, 1, 0), m->nqkv, H, c.init_std);
    L.wo.gen(c.seed, sid(l, 2, 0), H, m->hqd, c.init_std);
    for (int e = 0; e < E; ++e) {
      L.w1.gen(c.seed, sid(l, 4, e), 2 * I, H, c.init_std, e, E);
      L.w2.gen(c.seed, sid(l, 5, e), H, I, c.init_std, e, E);
    }
    L.wr.resize((size_t)E * H);
    orc_synth_normal_bf16(c.seed, sid(l, 3, 0), 0, (int64_t)E * H, c.init_std, L.wr.data());
    L.sinks.resize((size_t)c.n_q_heads);
    orc_synth_normal_f32(c.seed, sid(l, 6, 0), 0, c.n_q_heads, 1.0f, L.sinks.data());
    L.g_attn.assign((size_t)H, 1.0f);
    L.g_mlp.assign((size_t)H, 1.0f);
    L.cache.assign((size_t)c.num_pages * 2 * c.n_kv_heads * c.page_size * c.head_dim, 0);
  }
  m->embed.resize((size_t)c.vocab * H);
  orc_synth_normal_bf16(c.seed, sid(-1, 1, 0), 0, (int64_t)c.vocab * H, c.init_std, m->embed.data());
  m->lm.gen(c.seed, sid(-1, 2, 0), c.vocab, H, c.init_std);
  m->g_final.assign((size_t)H, 1.0f);
  const int max_pos = c.max_pages_per_seq * c.page_size;
  m->rope_cos.resize((size_t)max_pos * (c.head_dim / 2));
  m->rope_sin.resize((size_t)max_pos * (c.head_dim / 2));
  orc_rope_table(max_pos, c.head_dim, (double)c.rope_theta, m->rope_cos.data(), m->rope_sin.data());
  return m;
}

void orc_model_destroy(orc_model* m) { delete m; }

/* Same stand-in for prefill as the engine's: layer l, element i = eb_normal(seed, 20000 + l, i). */
void orc_model_kv_fill_synth(orc_model* m) {
  for (int l = 0; l < m->c.n_layers; ++l) {
    auto& cache = m->layers[(size_t)l].cache;
    orc_synth_normal_bf16(m->c.seed, 20000 + (uint64_t)l, 0, (int64_t)cache.size(), 1.0f, cache.data());
  }
}

/* Intermediates of the last layer the last step ran (which: 0 = [q | k | v] rows after the rotary embedding,
 * 1 = attention output, 2 = O projection output); returns the element count. */
int64_t orc_model_last(orc_model* m, int32_t which, const uint16_t** p) {
  const std::vector<uint16_t>& v = which == 0 ? m->last_qkv : which == 1 ? m->last_att : m->last_o;
  *p = v.data();
  return (int64_t)v.size();
}

uint16_t* orc_model_cache(orc_model* m, int32_t layer) { return m->layers[(size_t)layer].cache.data(); }
/* Embedding table [vocab][hidden] bf16 (tests perturb one entry by one ulp to measure the decoder's own sensitivity). */
uint16_t* orc_model_embed(orc_model* m) { return m->embed.data(); }

/*
 * One step.  Packing arrays as eb_sched_pack writes them; block_tables [max_seqs][bt_stride].
 * Outputs (each may be NULL): next[T], margin[T], logits [T][vocab] bf16, route_idx [layers][T][top_k],
 * route_logits [layers][T][E] fp32, hidden [layers+1][T][hidden] bf16 (index 0 = embeddings).
 * n_layers_run < n_layers stops early (for timing one layer); logits then come from that depth.
 */
void orc_model_step(orc_model* m, int32_t T, int32_t n_seqs, const int32_t* tokens, const int32_t* tok_slot,
                    const int32_t* positions, const int32_t* slots, const int32_t* q_off, const int32_t* ctx_lens,
                    const int32_t* block_tables, int32_t bt_stride, int32_t n_layers_run, int32_t* next, float* margin,
                    uint16_t* logits_out, int32_t* route_idx, float* route_logits, uint16_t* hidden) {
  const eb_config& c = m->c;
  const int H = c.hidden, I = c.inter, E = c.n_experts, K = c.top_k;
  std::vector<uint16_t> x((size_t)T * H), h((size_t)T * H), qkv((size_t)T * m->nqkv), att((size_t)T * m->hqd),
      o((size_t)T * H), moe((size_t)T * H);
  std::vector<uint8_t> h8((size_t)T * H), a8((size_t)T * m->hqd);
  std::vector<float> sh((size_t)(cdiv(T, 128) * cdiv(H, 128))), sa((size_t)(cdiv(T, 128) * cdiv(m->hqd, 128)));
  std::vector<int32_t> idx((size_t)T * K);
  std::vector<float> wts((size_t)T * K), rl((size_t)T * E);
  const int32_t seg[2] = {0, T};
  orc_embed(m->embed.data(), H, tokens, T, x.data());
  if (hidden) memcpy(hidden, x.data(), x.size() * 2);
  const int nl = std::min(n_layers_run, c.n_layers);
  for (int l = 0; l < nl; ++l) {
    LayerW& L = m->layers[(size_t)l];
    orc_rmsnorm(x.data(), L.g_attn.data(), T, H, c.rms_eps, h.data());
    orc_quant_act_block128(h.data(), H, seg, 1, h8.data(), sh.data());
    orc_gemm_fp8_block(h8.data(), sh.data(), L.wqkv.codes.data(), L.wqkv.scales.data(), T, m->nqkv, H, qkv.data());
    orc_rope(qkv.data(), m->nqkv, c.n_q_heads + c.n_kv_heads, c.head_dim, positions, T, m->rope_cos.data(), m->rope_sin.data());
    orc_kv_append(L.cache.data(), c.n_kv_heads, c.head_dim, c.page_size, qkv.data() + m->hqd,
                  qkv.data() + m->hqd + c.n_kv_heads * c.head_dim, m->nqkv, block_tables, bt_stride, tok_slot, positions, T);
    const int window = (l % 2 == 0) ? c.window : 0;
    orc_attn_paged_sink(qkv.data(), m->nqkv, L.cache.data(), block_tables, bt_stride, slots, q_off, ctx_lens, n_seqs,
                        L.sinks.data(), window, c.n_q_heads, c.n_kv_heads, c.head_dim, c.page_size, 0.125f, att.data(), m->hqd);
    orc_quant_act_block128(att.data(), m->hqd, seg, 1, a8.data(), sa.data());
    orc_gemm_fp8_block(a8.data(), sa.data(), L.wo.codes.data(), L.wo.scales.data(), T, H, m->hqd, o.data());
    if (l + 1 == nl) {
      m->last_qkv = qkv;
      m->last_att = att;
      m->last_o = o;
    }
    orc_residual_add(x.data(), o.data(), (int64_t)T * H);
    orc_rmsnorm(x.data(), L.g_mlp.data(), T, H, c.rms_eps, h.data());
    orc_router_topk(h.data(), L.wr.data(), T, E, H, K, idx.data(), wts.data(), rl.data());
    if (route_idx) memcpy(route_idx + (size_t)l * T * K, idx.data(), idx.size() * 4);
    if (route_logits) memcpy(route_logits + (size_t)l * T * E, rl.data(), rl.size() * 4);
    orc_moe_forward(h.data(), T, H, I, E, K, idx.data(), wts.data(), L.w1.codes.data(), L.w1.scales.data(),
                    L.w2.codes.data(), L.w2.scales.data(), moe.data());
    orc_residual_add(x.data(), moe.data(), (int64_t)T * H);
    if (hidden) memcpy(hidden + (size_t)(l + 1) * T * H, x.data(), x.size() * 2);
  }
  if (!next && !logits_out) return;
  orc_rmsnorm(x.data(), m->g_final.data(), T, H, c.rms_eps, h.data());
  orc_quant_act_block128(h.data(), H, seg, 1, h8.data(), sh.data());
  std::vector<uint16_t> logits((size_t)T * c.vocab);
  orc_gemm_fp8_block(h8.data(), sh.data(), m->lm.codes.data(), m->lm.scales.data(), T, c.vocab, H, logits.data());
  if (logits_out) memcpy(logits_out, logits.data(), logits.size() * 2);
  if (next) {
    std::vector<float> mg((size_t)T);
    orc_argmax(logits.data(), T, c.vocab, next, mg.data());
    if (margin) memcpy(margin, mg.data(), mg.size() * 4);
  }
}

} /* extern "C" */

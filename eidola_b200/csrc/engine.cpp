// The decode engine: owns weights (random-init from a seed, generated on the device), the paged KV cache of
// every layer, the page scheduler and the step workspaces, and runs one ragged decode / verify step through the
// library's own kernels.  Host code only; every kernel is reached through the operator entry points.
//
// Layer (l even: sliding window, l odd: full attention):
//   h = rmsnorm(x) -> e4m3 -> QKV GEMM -> rotary(q, k) -> KV append -> paged sink attention -> e4m3 -> O GEMM
//   -> x += o -> h = rmsnorm(x) -> router top-k -> permute -> gather+e4m3 -> W1 grouped GEMM -> silu(gate)*up
//   -> e4m3 -> W2 grouped GEMM -> x += combine.   After the last layer: rmsnorm -> e4m3 -> LM head -> argmax.
//
// Per step the host builds ONE pinned staging block (token ids, packing arrays, block-table patches, the two
// attention plans) and copies it with one transfer; results come back in one transfer.
//
// What would sit above this in the reference: the loopback HTTP client of a local engine
// (crates/eidola-app-core/src/lib.rs:7155-7163) or a `ChatBackend` (crates/eidola-server/src/backend.rs:87-108).
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <new>
#include <utility>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include "common.h"
#include "loader.h"

namespace {

// Tensor parallel, steps of at most this many token rows: every rank sends its WHOLE partial [T, H] to every peer and
// sums all rows itself, so residual, norm, routing and quantisation run replicated and a layer needs two exchanges
// instead of four.  Larger steps deal the rows to the ranks in slices (fewer bytes, more exchanges).
constexpr int kWholeBatchTokens = 512;

inline uint64_t sid(int layer, int kind, int expert) {
  return ((uint64_t)(layer + 1) << 20) | ((uint64_t)kind << 12) | (uint64_t)expert;
}
enum { K_WQKV = 1, K_WO = 2, K_ROUTER = 3, K_W1 = 4, K_W2 = 5, K_SINK = 6, K_EMBED = 1, K_LMHEAD = 2 };

struct Fp8Weight {
  uint8_t* codes = nullptr;
  float* scales = nullptr;
};

struct Layer {
  Fp8Weight wqkv, wo, w1, w2;
  uint16_t* wr = nullptr;
  float* sinks = nullptr;
  float *g_attn = nullptr, *g_mlp = nullptr;
  uint16_t* cache = nullptr;
};

struct Plan {
  std::vector<eb_attn_item> items;
  std::vector<int32_t> seq_part;
  int32_t n_items = 0, n_parts = 0;
};

}  // namespace

struct eb_engine {
  eb_config c;
  int sm_count = 0;
  // tensor / expert parallelism: this rank holds query heads [rank*hq_l, +hq_l), KV heads [rank*hkv_l, +hkv_l) and
  // experts [e0, e0 + e_l); hqd and nqkv below are the LOCAL widths
  int tp_rank = 0, tp_size = 1;
  eb_comm* comm = nullptr;
  int hq_l = 0, hkv_l = 0, e_l = 0, e0 = 0;
  int v0 = 0, v1 = 0;      // vocabulary rows [v0, v1) of the LM head live on this rank (whole 128-row scale blocks)
  float* cand = nullptr;   // argmax candidates of every rank's vocabulary slice: [tp_size][max_tokens][4]
  int kv_band = 0, k_col0 = 0, v_col0 = 0;  // the K and V bands of the local QKV row start on 128-row scale blocks
  float* ar_buf = nullptr;                   // fp32 [max_tokens][hidden] summed across ranks
  // peer-memory collectives (tensor parallel): the buffers that cross ranks live in one symmetric arena
  eb_symm* symm = nullptr;
  uint8_t* arena = nullptr;                  // this rank's arena
  size_t arena_used = 0;
  uint8_t* planes = nullptr;                 // [tp_size][chunk rows][hidden] fp32 or bf16: the ranks' partial rows of my slice
  // expert parallelism as dispatch / return of rows (the all-to-all pair) instead of gather-everything + reduce-scatter
  bool slices_forced = false;
  // Tensor-parallel O projection on the GATHERED attention output: every rank keeps the full W_o, quantises its heads'
  // columns straight into the other ranks' copies of the operand, and multiplies full-K rows itself (all rows of a small
  // step, its token slice of a large one).  One byte per (token, head column) crosses the links instead of a partial
  // [T, H] per rank, and the sum over K is the single-GPU one.  Default from four ranks on (EIDOLA_B200_TP_OGATHER=1 / 0 forces it on / off);
  // otherwise, and with NCCL transport, the ranks keep their column band of W_o and exchange partial results.
  bool o_gather = false;
  int o_cols = 0;           // columns of the W_o this rank holds: all head columns (o_gather) or its own heads'
  uint8_t* a8g = nullptr;   // [Tc][n_q_heads * head_dim] e4m3 gathered operand (arena)
  float* sag = nullptr;     // its block scales
  bool a2a = false, a2a_forced = false;  // forced: EIDOLA_B200_EP_A2A=1 (tests): row dispatch whatever the step's size
  uint16_t* xp16 = nullptr;                  // [tokens * top_k][hidden] bf16: rows dispatched to this rank's experts (global row numbering)
  int32_t* r_idx_local = nullptr;
  float* sinks_all = nullptr;
  int nqkv = 0, hqd = 0, kbH = 0, kbI = 0, kbA = 0;
  std::vector<Layer> layers;
  uint16_t* embed = nullptr;
  Fp8Weight lm;
  float* g_final = nullptr;
  float *rope_cos = nullptr, *rope_sin = nullptr;
  eb_sched* sched = nullptr;
  std::vector<int32_t> uploaded_pages;  // block-table entries of each slot already on the device
  int32_t* d_bt = nullptr;
  int32_t* d_bt_ring = nullptr;  // window_ring: [max_seqs][max_pages_per_seq], logical page p -> slot*ring + p % ring
  int ring = 0;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  std::vector<void*> allocs;
  uint8_t* w_scratch = nullptr;  // row-major staging while the weights are generated
  int64_t weight_bytes = 0, kv_bytes = 0, work_bytes = 0;

  // step workspaces
  uint16_t *x = nullptr, *h = nullptr, *qkv = nullptr, *attn = nullptr, *o = nullptr, *gu = nullptr, *y = nullptr,
           *logits = nullptr;
  uint8_t *h8 = nullptr, *a8 = nullptr, *xp8 = nullptr, *act8 = nullptr;
  float *sh = nullptr, *sa = nullptr, *sxp = nullptr, *sact = nullptr;
  int32_t *r_idx = nullptr, *seg_off = nullptr, *perm_row = nullptr, *row_token = nullptr;
  float* r_wts = nullptr;
  void *gemm_ws = nullptr, *group_ws = nullptr;
  size_t gemm_ws_bytes = 0, group_ws_bytes = 0;
  float *part_acc = nullptr, *part_ml = nullptr;
  int32_t* d_next = nullptr;
  float* d_margin = nullptr;
  int32_t *h_stage = nullptr, *d_stage = nullptr;
  size_t stage_words = 0;
  int32_t* h_result = nullptr;  // pinned: next[T] then margin[T]
  int32_t cap_items = 0;
  // prefill: the LM head runs only over the 128-row blocks that hold these rows (the last prompt token of a sequence that
  // finishes in the step); the other rows of the step's results are then undefined
  bool head_rows_on = false;
  std::vector<int32_t> head_rows;
  // per slot: log2(e) / temperature (0: greedy), top_p in units of 2^-24, seed of the counter-based random numbers
  std::vector<int32_t> high_len;  // per slot: the largest length the sequence has had (what its page rings were written up to)
  std::vector<float> samp_scale;
  std::vector<uint32_t> samp_q24;
  std::vector<uint64_t> samp_seed;
  const int32_t* d_samp = nullptr;  // this step's per-row {scale, top_p, rand32} [3][T] in the staging block, or null
  int32_t chunk_cap = 0;  // most new tokens one sequence may bring to a step (a prefill chunk); see eb_engine_chunk_tokens
  int32_t cap_ent = 0;    // most attention entries of a step: a sequence's new tokens in runs of at most max_q_len
  // debug
  int32_t* dbg_route = nullptr;
  uint16_t* dbg_hidden = nullptr;
  uint16_t* dbg_force = nullptr;       // [n_layers+1][max_tokens][hidden]: residual stream to impose before a layer
  std::vector<int32_t> force_rows;     // rows imposed before each layer (0 = none)

  // per-category device time of the last step (debug & 2): 0 attention full, 1 attention windowed, 2 dense GEMMs,
  // 3 expert GEMMs, 4 LM head
  std::vector<cudaEvent_t> prof_ev;
  std::vector<int> prof_cat;
  float prof_ms[8] = {0};

  // state of the step in flight
  int32_t cur_T = 0;
  bool in_flight = false;
  int32_t launches = 0;
  float last_ms = 0.f;
  int64_t tick = 0;                      // steps launched so far: the clock of least-recently-used admission
  int64_t h2d_bytes = 0, d2h_bytes = 0;  // bytes the last step copied host -> device (staging block) and back (results)
};

namespace {

#define EB_TRY(expr)            \
  do {                          \
    int32_t _rc = (expr);       \
    if (_rc != EB_OK) return _rc; \
  } while (0)

// Pages of layer l's cache: sliding-window layers keep a ring per sequence when the engine was asked to.
inline bool layer_windowed(const eb_engine* e, int l) { return l % 2 == 0 && e->c.window > 0; }
inline int32_t layer_pages(const eb_engine* e, int l) {
  return (e->ring && layer_windowed(e, l)) ? e->c.max_seqs * e->ring : e->c.num_pages;
}

template <typename T>
int32_t dev_alloc(eb_engine* e, T** p, size_t count, int64_t* tally) {
  void* q = nullptr;
  const size_t bytes = std::max<size_t>(count * sizeof(T), 16);
  cudaError_t err = cudaMalloc(&q, bytes);
  if (err != cudaSuccess) return eb::fail((int32_t)err, "engine: cudaMalloc of %zu bytes: %s", bytes, cudaGetErrorString(err));
  e->allocs.push_back(q);
  *p = (T*)q;
  *tally += (int64_t)bytes;
  return EB_OK;
}

// Weights live in HBM as 16 KiB tiles (eb_weight_tile_fp8): a GEMM stage is then one contiguous read.
int32_t alloc_fp8(eb_engine* e, Fp8Weight* w, int64_t groups, int64_t rows, int64_t cols) {
  size_t tiled = 0;
  EB_TRY(eb_weight_tiled_bytes((int32_t)groups, (int32_t)rows, (int32_t)cols, &tiled));
  EB_TRY(dev_alloc(e, &w->codes, tiled, &e->weight_bytes));
  EB_TRY(dev_alloc(e, &w->scales, (size_t)(groups * eb::cdiv(rows, 128) * eb::cdiv(cols, 128)), &e->weight_bytes));
  return EB_OK;
}

int32_t fill_ones(eb_engine* e, float* d, int n) {
  std::vector<float> ones((size_t)n, 1.0f);
  EB_CUDA(cudaMemcpyAsync(d, ones.data(), (size_t)n * sizeof(float), cudaMemcpyHostToDevice, e->stream));
  EB_CUDA(cudaStreamSynchronize(e->stream));
  return EB_OK;
}

// Generate rows [src_row0, +nrows) of a seeded [rows_total x cols] weight (row-major, into the scratch buffer) and store
// them as tiles at weight-row block dst_row0 / 128 of `w` (group `group` of a tensor whose groups have rows_per_group
// rows).  Bands start on 128-row boundaries, so their tiles are whole and consecutive.
int32_t synth_band_tiled(eb_engine* e, Fp8Weight* w, int64_t group, int64_t rows_per_group, int64_t dst_row0, float* scales_dst,
                         int64_t rows_total, int64_t cols, int64_t src_row0, int64_t nrows, uint64_t stream_id) {
  const eb_config& c = e->c;
  const int64_t KB = eb::cdiv(cols, 128), NB = eb::cdiv(rows_per_group, 128);
  const int64_t band = 65536;  // rows generated per pass: bounds the scratch buffer (an LM head has 200k rows)
  for (int64_t r = 0; r < nrows; r += band) {
    const int64_t n = std::min(band, nrows - r);
    EB_TRY(eb_synth_weight_fp8(e->w_scratch, scales_dst + ((r) / 128) * KB, rows_total, cols, src_row0 + r, n, c.seed, stream_id,
                               c.init_std, e->stream));
    uint8_t* dst = w->codes + ((group * NB + (dst_row0 + r) / 128) * KB) * (int64_t)(128 * 128);
    EB_TRY(eb_weight_tile_fp8(e->w_scratch, 1, (int32_t)n, (int32_t)cols, dst, e->stream));
  }
  return EB_OK;
}

int32_t init_weights(eb_engine* e) {
  const eb_config& c = e->c;
  const int H = c.hidden, I = c.inter, E = e->e_l;  // E: experts held by this rank
  void* st = e->stream;
  const int hqd_g = c.n_q_heads * c.head_dim, hkd_g = c.n_kv_heads * c.head_dim, nqkv_g = hqd_g + 2 * hkd_g;
  {  // row-major staging for one band of one weight tensor; released when the weights are in place
    const int64_t widest = std::max<int64_t>(std::max(H, I), e->o_cols);
    EB_CUDA(cudaMalloc((void**)&e->w_scratch, (size_t)(65536 * widest)));
  }
  const int kv_row0 = (e->tp_rank * e->hkv_l * c.head_dim) / 128 * 128;  // start of this rank's K (and V) band
  for (int l = 0; l < c.n_layers; ++l) {
    Layer& L = e->layers[(size_t)l];
    EB_TRY(alloc_fp8(e, &L.wqkv, 1, e->nqkv, H));
    EB_TRY(alloc_fp8(e, &L.wo, 1, H, e->o_cols));
    EB_TRY(alloc_fp8(e, &L.w1, E, 2 * I, H));
    EB_TRY(alloc_fp8(e, &L.w2, E, H, I));
    EB_TRY(dev_alloc(e, &L.wr, (size_t)c.n_experts * H, &e->weight_bytes));
    EB_TRY(dev_alloc(e, &L.sinks, (size_t)c.n_q_heads, &e->weight_bytes));
    EB_TRY(dev_alloc(e, &L.g_attn, (size_t)H, &e->weight_bytes));
    EB_TRY(dev_alloc(e, &L.g_mlp, (size_t)H, &e->weight_bytes));
    // local QKV rows = [q heads | K band | V band], each a row band of the global [q | k | v] tensor
    const int64_t band_rows[3] = {e->hqd, e->kv_band, e->kv_band};
    const int64_t band_src[3] = {(int64_t)e->tp_rank * e->hqd, hqd_g + kv_row0, hqd_g + hkd_g + kv_row0};
    int64_t dst_row = 0;
    for (int b = 0; b < 3; ++b) {
      EB_TRY(synth_band_tiled(e, &L.wqkv, 0, e->nqkv, dst_row, L.wqkv.scales + (dst_row / 128) * e->kbH, nqkv_g, H, band_src[b],
                              band_rows[b], sid(l, K_WQKV, 0)));
      dst_row += band_rows[b];
    }
    EB_TRY(eb_synth_weight_fp8_slice(e->w_scratch, L.wo.scales, H, hqd_g, 0, H, e->o_gather ? 0 : (int64_t)e->tp_rank * e->hqd,
                                     e->o_cols, c.seed, sid(l, K_WO, 0), c.init_std, st));
    EB_TRY(eb_weight_tile_fp8(e->w_scratch, 1, H, e->o_cols, L.wo.codes, st));
    const int64_t s1 = eb::cdiv(2 * I, 128) * e->kbH, s2 = eb::cdiv(H, 128) * e->kbI;
    for (int x = 0; x < E; ++x) {
      EB_TRY(synth_band_tiled(e, &L.w1, x, 2 * I, 0, L.w1.scales + x * s1, 2 * I, H, 0, 2 * I, sid(l, K_W1, e->e0 + x)));
      EB_TRY(synth_band_tiled(e, &L.w2, x, H, 0, L.w2.scales + x * s2, H, I, 0, H, sid(l, K_W2, e->e0 + x)));
    }
    EB_TRY(eb_synth_normal_bf16(L.wr, (int64_t)c.n_experts * H, c.seed, sid(l, K_ROUTER, 0), 0, c.init_std, st));
    EB_TRY(eb_synth_normal_f32(L.sinks, c.n_q_heads, c.seed, sid(l, K_SINK, 0), 0, 1.0f, st));
    EB_TRY(fill_ones(e, L.g_attn, H));
    EB_TRY(fill_ones(e, L.g_mlp, H));
  }
  EB_TRY(dev_alloc(e, &e->embed, (size_t)c.vocab * H, &e->weight_bytes));
  EB_TRY(eb_synth_normal_bf16(e->embed, (int64_t)c.vocab * H, c.seed, sid(-1, K_EMBED, 0), 0, c.init_std, st));
  EB_TRY(alloc_fp8(e, &e->lm, 1, e->v1 - e->v0, H));
  EB_TRY(synth_band_tiled(e, &e->lm, 0, e->v1 - e->v0, 0, e->lm.scales, c.vocab, H, e->v0, e->v1 - e->v0, sid(-1, K_LMHEAD, 0)));
  EB_TRY(dev_alloc(e, &e->g_final, (size_t)H, &e->weight_bytes));
  EB_TRY(fill_ones(e, e->g_final, H));
  // rotary table
  const int max_pos = c.max_pages_per_seq * c.page_size;
  const size_t n = (size_t)max_pos * (c.head_dim / 2);
  std::vector<float> hc(n), hs(n);
  EB_TRY(eb_rope_table(max_pos, c.head_dim, (double)c.rope_theta, hc.data(), hs.data()));
  EB_TRY(dev_alloc(e, &e->rope_cos, n, &e->weight_bytes));
  EB_TRY(dev_alloc(e, &e->rope_sin, n, &e->weight_bytes));
  EB_CUDA(cudaMemcpyAsync(e->rope_cos, hc.data(), n * sizeof(float), cudaMemcpyHostToDevice, e->stream));
  EB_CUDA(cudaMemcpyAsync(e->rope_sin, hs.data(), n * sizeof(float), cudaMemcpyHostToDevice, e->stream));
  EB_CUDA(cudaStreamSynchronize(e->stream));
  cudaFree(e->w_scratch);
  e->w_scratch = nullptr;
  return EB_OK;
}

int32_t init_work(eb_engine* e) {
  const eb_config& c = e->c;
  const int H = c.hidden, I = c.inter, E = e->e_l, T = c.max_tokens;
  const int64_t R = (int64_t)T * c.top_k;
  int64_t* w = &e->work_bytes;
  // under tensor parallelism rows are dealt to ranks in tp_size equal chunks for the in-place collectives: slack rows
  const size_t Tc = (size_t)T + (e->tp_size > 1 ? (size_t)e->tp_size * 128 : 0);  // slices are whole 128-row scale blocks
  const int64_t tb0 = eb::cdiv((int64_t)Tc, 128);
  const size_t r_cap0 = (size_t)R + (e->tp_size > 1 ? (size_t)e->tp_size * 128 * c.top_k : 0);
  const bool want_symm = e->tp_size > 1 && !(getenv("EIDOLA_B200_TP_NCCL") && getenv("EIDOLA_B200_TP_NCCL")[0] == '1');
  if (want_symm) {
    // everything another rank writes into, or that is pushed from, sits in the arena
    auto a256 = [](size_t v) { return (v + 255) & ~(size_t)255; };
    const size_t sz_rows2 = a256(Tc * H * 2), sz_rows1 = a256(Tc * H), sz_rows4 = a256(Tc * H * 4);
    // small steps exchange whole [T, H] partials (one plane per rank, every rank sums all rows): room for tp_size planes
    const size_t sz_planes = std::max(sz_rows4, a256((size_t)e->tp_size * std::min(T, kWholeBatchTokens) * H * 4));
    const size_t sz_sh = a256((size_t)(tb0 * e->kbH) * 4), sz_r = a256(r_cap0 * 4), sz_cand = a256((size_t)e->tp_size * T * 4 * 4);
    {
      const char* v = getenv("EIDOLA_B200_EP_A2A");
      e->a2a = v ? v[0] == '1' : e->tp_size >= 4;  // the row exchange moves fewer bytes from four ranks on (large steps)
      e->a2a_forced = v && v[0] == '1';
      const char* w = getenv("EIDOLA_B200_TP_WHOLE");  // =0 (tests, A/B timing): token slices even for small steps
      e->slices_forced = w && w[0] == '0';
    }
    const size_t sz_routed = e->a2a ? a256((size_t)R * H * 2) : 0;
    const size_t sz_a8g = e->o_gather ? a256(Tc * (size_t)e->o_cols) : 0, sz_sag = e->o_gather ? a256((size_t)tb0 * (e->o_cols / 128) * 4) : 0;
    const size_t total = 3 * sz_rows2 + sz_rows1 + sz_rows4 + sz_planes + sz_sh + 2 * sz_r + sz_cand + 2 * sz_routed + sz_a8g + sz_sag;
    EB_TRY(eb_symm_create(e->comm, total, &e->symm));
    void* base = nullptr;
    EB_TRY(eb_symm_ptr(e->symm, e->tp_rank, &base, nullptr));
    e->arena = (uint8_t*)base;
    size_t o = 0;
    auto carve = [&](size_t bytes) {
      uint8_t* p = e->arena + o;
      o += bytes;
      return p;
    };
    e->x = (uint16_t*)carve(sz_rows2);
    e->h = (uint16_t*)carve(sz_rows2);
    e->o = (uint16_t*)carve(sz_rows2);
    e->h8 = carve(sz_rows1);
    e->ar_buf = (float*)carve(sz_rows4);
    e->planes = carve(sz_planes);
    e->sh = (float*)carve(sz_sh);
    e->r_idx = (int32_t*)carve(sz_r);
    e->r_wts = (float*)carve(sz_r);
    e->cand = (float*)carve(sz_cand);
    if (e->a2a) {
      e->xp16 = (uint16_t*)carve(sz_routed);
      e->y = (uint16_t*)carve(sz_routed);
    }
    if (e->o_gather) {
      e->a8g = carve(sz_a8g);
      e->sag = (float*)carve(sz_sag);
    }
    e->arena_used = o;
    *w += (int64_t)total;
  }
  if (!e->x) EB_TRY(dev_alloc(e, &e->x, Tc * H, w));
  if (!e->h) EB_TRY(dev_alloc(e, &e->h, Tc * H, w));
  EB_TRY(dev_alloc(e, &e->qkv, (size_t)T * e->nqkv, w));
  EB_TRY(dev_alloc(e, &e->attn, (size_t)T * e->hqd, w));
  if (!e->o) EB_TRY(dev_alloc(e, &e->o, Tc * H, w));  // also the bf16 operand of the tensor-parallel reduce-scatters
  EB_TRY(dev_alloc(e, &e->gu, (size_t)R * 2 * I, w));
  if (!e->y) EB_TRY(dev_alloc(e, &e->y, (size_t)R * H, w));
  EB_TRY(dev_alloc(e, &e->logits, (size_t)T * c.vocab, w));
  if (!e->h8) EB_TRY(dev_alloc(e, &e->h8, Tc * H, w));
  EB_TRY(dev_alloc(e, &e->a8, (size_t)T * e->hqd, w));
  EB_TRY(dev_alloc(e, &e->xp8, (size_t)R * H, w));
  EB_TRY(dev_alloc(e, &e->act8, (size_t)R * I, w));
  const int64_t tb = eb::cdiv((int64_t)Tc, 128), rb = R / 128 + E;
  if (!e->sh) EB_TRY(dev_alloc(e, &e->sh, (size_t)(tb * e->kbH), w));
  EB_TRY(dev_alloc(e, &e->sa, (size_t)(tb * e->kbA), w));
  EB_TRY(dev_alloc(e, &e->sxp, (size_t)(rb * e->kbH), w));
  EB_TRY(dev_alloc(e, &e->sact, (size_t)(rb * e->kbI), w));
  // routing is computed on a token slice per rank and all-gathered in place: room for tp_size equal chunks
  const size_t r_cap = (size_t)R + (e->tp_size > 1 ? (size_t)e->tp_size * 128 * c.top_k : 0);
  if (!e->r_idx) EB_TRY(dev_alloc(e, &e->r_idx, r_cap, w));
  EB_TRY(dev_alloc(e, &e->r_idx_local, (size_t)R, w));
  if (e->tp_size > 1 && !e->symm) {
    EB_TRY(dev_alloc(e, &e->ar_buf, Tc * H, w));
    EB_TRY(dev_alloc(e, &e->cand, (size_t)e->tp_size * T * 4, w));
  }
  if (!e->r_wts) EB_TRY(dev_alloc(e, &e->r_wts, r_cap, w));
  EB_TRY(dev_alloc(e, &e->seg_off, (size_t)c.n_experts + 1, w));  // all experts' segments under row dispatch, the local ones otherwise
  EB_TRY(dev_alloc(e, &e->perm_row, (size_t)R, w));
  EB_TRY(dev_alloc(e, &e->row_token, (size_t)R, w));
  size_t ws = 0, ws2 = 0;
  const int nmax = std::max(std::max(e->nqkv, H), 1);
  EB_TRY(eb_gemm_workspace(T, nmax, 1, &ws));
  uint8_t* p8 = nullptr;
  EB_TRY(dev_alloc(e, &p8, ws, w));
  e->gemm_ws = p8;
  e->gemm_ws_bytes = ws;
  EB_TRY(eb_gemm_workspace((int32_t)R, 2 * I, std::max(E, 2), &ws2));
  EB_TRY(dev_alloc(e, &p8, ws2, w));
  e->group_ws = p8;
  e->group_ws_bytes = ws2;
  // work items of one attention launch: ~4 per SM from the planner, one per sequence at least, and enough for a pool
  // whose every page is in use at the largest run the kernel accepts (512 pages per item)
  e->cap_ent = c.max_seqs + c.max_tokens / c.max_q_len;
  e->cap_items = 4 * e->sm_count + e->cap_ent + 16 + c.num_pages / 512;
  const int ppi = 8 / e->hkv_l;
  size_t acc_b = 0, ml_b = 0;
  EB_TRY(eb_attn_workspace(e->cap_items * ppi, c.max_q_len, e->hq_l, c.head_dim, &acc_b, &ml_b));
  EB_TRY(dev_alloc(e, &e->part_acc, acc_b / sizeof(float), w));
  EB_TRY(dev_alloc(e, &e->part_ml, ml_b / sizeof(float), w));
  EB_TRY(dev_alloc(e, &e->d_next, (size_t)T, w));
  EB_TRY(dev_alloc(e, &e->d_margin, (size_t)T, w));
  EB_TRY(dev_alloc(e, &e->d_bt, (size_t)c.max_seqs * c.max_pages_per_seq, w));
  EB_CUDA(cudaMemsetAsync(e->d_bt, 0xFF, (size_t)c.max_seqs * c.max_pages_per_seq * sizeof(int32_t), e->stream));
  // staging: tokens, tok_slot, positions, and the sampler's scale, top_p, random number [T each]; slots, ctx_lens [N], q_off [N+1] of the N attention entries; patches
  // 3*P (P <= all pages of newly admitted sequences: bounded by max_seqs*max_pages); two plans (items 4 words each +
  // seq_part)
  const size_t S = (size_t)c.max_seqs, N = (size_t)e->cap_ent;
  e->stage_words = 6 * (size_t)T + 3 * N + 1 + 3 * S * (size_t)c.max_pages_per_seq + 2 * (4 * (size_t)e->cap_items + N + 1) + 64;
  EB_CUDA(cudaMallocHost((void**)&e->h_stage, e->stage_words * sizeof(int32_t)));
  EB_TRY(dev_alloc(e, &e->d_stage, e->stage_words, w));
  EB_CUDA(cudaMallocHost((void**)&e->h_result, 2 * (size_t)T * sizeof(int32_t)));
  if (c.debug & 1) {
    EB_TRY(dev_alloc(e, &e->dbg_route, (size_t)c.n_layers * R, w));
    EB_TRY(dev_alloc(e, &e->dbg_hidden, (size_t)(c.n_layers + 1) * T * H, w));
    EB_TRY(dev_alloc(e, &e->dbg_force, (size_t)(c.n_layers + 1) * T * H, w));
    e->force_rows.assign((size_t)c.n_layers + 1, 0);
  }
  return EB_OK;
}

__global__ void bt_patch_kernel(int32_t* bt, int stride, const int32_t* patches, int n) {
  eb::pdl_wait();  // programmatic dependent launch: the predecessor in the stream has completed
  eb::pdl_trigger();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) bt[(int64_t)patches[3 * i] * stride + patches[3 * i + 1]] = patches[3 * i + 2];
}

int32_t validate(const eb_config* c) {
  EB_REQUIRE(c, EB_ERR_ARG, "eb_engine_create: null config");
  EB_REQUIRE(c->n_layers >= 1 && c->hidden >= 128 && c->hidden % 16 == 0, EB_ERR_ARG, "config: hidden %d", c->hidden);
  EB_REQUIRE(c->head_dim == 64 && c->page_size == 16, EB_ERR_UNSUPPORTED, "config: head_dim %d / page_size %d (64 / 16)",
             c->head_dim, c->page_size);
  EB_REQUIRE(c->n_kv_heads == 1 || c->n_kv_heads == 2 || c->n_kv_heads == 4 || c->n_kv_heads == 8, EB_ERR_UNSUPPORTED,
             "config: n_kv_heads %d not in {1,2,4,8}", c->n_kv_heads);
  EB_REQUIRE(c->n_q_heads == 8 * c->n_kv_heads || c->n_q_heads == 4 * c->n_kv_heads, EB_ERR_UNSUPPORTED,
             "config: %d query heads over %d KV heads (groups of 8 or 4)", c->n_q_heads, c->n_kv_heads);
  EB_REQUIRE(c->n_experts >= 1 && c->n_experts <= 256 && c->top_k >= 1 && c->top_k <= 8 && c->top_k <= c->n_experts,
             EB_ERR_UNSUPPORTED, "config: experts %d, top_k %d", c->n_experts, c->top_k);
  EB_REQUIRE(c->inter >= 128 && c->inter % 16 == 0 && c->vocab >= 2, EB_ERR_ARG, "config: inter %d / vocab %d", c->inter,
             c->vocab);
  EB_REQUIRE(c->num_pages >= 1 && c->max_seqs >= 1 && c->max_pages_per_seq >= 1 && c->max_tokens >= 1 && c->max_q_len >= 1,
             EB_ERR_ARG, "config: non-positive capacity");
  EB_REQUIRE(c->max_q_len * (c->n_q_heads / c->n_kv_heads) <= 48, EB_ERR_UNSUPPORTED, "config: max_q_len %d", c->max_q_len);
  EB_REQUIRE(c->window >= 0 && c->rope_theta > 0 && c->rms_eps > 0 && c->init_std > 0, EB_ERR_ARG, "config: bad scalar");
  return EB_OK;
}

int32_t run_layers(eb_engine* e, int T, int n_seqs, const int32_t* d_tokens, const int32_t* d_tok_slot,
                   const int32_t* d_positions, const int32_t* d_slots, const int32_t* d_q_off, const int32_t* d_ctx,
                   const eb_attn_item* d_items[2], const int32_t* d_seq_part[2], const Plan plans[2], int max_q_len) {
  const eb_config& c = e->c;
  const int H = c.hidden, I = c.inter, E = e->e_l, R = T * c.top_k;  // E: local experts; R: upper bound of local rows
  const bool tp = e->tp_size > 1;
  // token slice of this rank for the reduce-scatter / all-gather pairs: tp_size equal chunks of whole 128-row scale
  // blocks (so that a slice can be quantised by its owner), the last ones may be short or empty
  const int chunk = ((T + e->tp_size - 1) / e->tp_size + 127) / 128 * 128;
  const int t0 = std::min(T, e->tp_rank * chunk), nt = std::min(T, t0 + chunk) - t0;
  void* st = e->stream;
  const int max_pos = c.max_pages_per_seq * c.page_size;
  int& n = e->launches;
  n = 0;
  // ---- collectives over the symmetric arena (peer stores + flags) when the engine has one, NCCL otherwise
  const bool symm = e->symm != nullptr;
  bool first_exchange = true;
  auto aoff = [&](const void* p) { return (int64_t)((const uint8_t*)p - e->arena); };
  // in-place all-gather of buffers whose per-rank slices are per_rank[i] bytes apart; this rank's slice holds valid[i] bytes
  auto gather = [&](int nb, void* const* bufs, const int64_t* per_rank, const int64_t* valid) -> int32_t {
    if (!symm) return eb_comm_allgather(e->comm, nb, bufs, per_rank, st);
    int64_t so[4], zero[4] = {0, 0, 0, 0}, by[4];
    for (int i = 0; i < nb; ++i) {
      so[i] = aoff(bufs[i]) + (int64_t)e->tp_rank * per_rank[i];
      by[i] = std::min(per_rank[i], (valid[i] + 15) / 16 * 16);
      if (per_rank[i] % 16) by[i] = std::min(per_rank[i], (valid[i] + 3) / 4 * 4);
    }
    int32_t seq = 0;
    EB_TRY(eb_symm_push(e->symm, nb, so, zero, so, zero, by, nullptr, 0, &seq, st));
    n += 1;
    return eb_symm_wait(e->symm, seq, 1, st);
  };
  // the WHOLE [T][H] partial to every rank (this rank's copy included), side by side as planes of T rows
  // (the consumer, eb_planes_residual_rmsnorm_after, waits for the peers' flags itself: no wait launch)
  auto share_planes = [&](const void* src, int esz, int32_t* seq, int32_t* patience) -> int32_t {
    const int64_t so = aoff(src), zero = 0, dof = aoff(e->planes), step = (int64_t)T * H * esz;
    EB_TRY(eb_symm_push(e->symm, 1, &so, &zero, &dof, &step, &step, nullptr, 1, seq, st));
    n += 1;
    *patience = first_exchange ? 32 : 1;  // the first exchange of a step also absorbs the skew between the ranks' host loops
    first_exchange = false;
    return EB_OK;
  };
  // the ranks' slices of a [T][H] partial (esz bytes per element, in the arena) to their owners, side by side as planes
  // and the owner's residual + norm over the planes of its slice; its CTAs wait for the peers' flags themselves (a rank
  // whose slice is empty still waits, with a launch of its own: every rank meets every exchange)
  auto scatter_planes_norm = [&](const void* src, int esz, const float* gain) -> int32_t {
    const int64_t so = aoff(src), step = (int64_t)chunk * H * esz, dof = aoff(e->planes), valid = (int64_t)T * H * esz;
    int32_t seq = 0;
    EB_TRY(eb_symm_push(e->symm, 1, &so, &step, &dof, &step, &step, &valid, 1, &seq, st));
    n += 1;
    // the first exchange of a step also absorbs the skew between the ranks' host loops
    const int patience = first_exchange ? 32 : 1;
    first_exchange = false;
    if (nt == 0) return eb_symm_wait(e->symm, seq, patience, st);
    return eb_planes_residual_rmsnorm_after(e->symm, seq, patience, e->planes, esz == 2, e->tp_size, (int64_t)chunk * H,
                                            e->x + (size_t)t0 * H, gain, nt, H, c.rms_eps, e->h + (size_t)t0 * H, st);
  };

  const bool prof = (c.debug & 2) != 0;
  size_t prof_used = 0;
  e->prof_cat.clear();
  // EIDOLA_B200_NVTX=1: the same intervals as named NVTX ranges (no-ops unless a tool that reads them is attached)
  static const bool nvtx_on = [] {
    const char* v = getenv("EIDOLA_B200_NVTX");
    return v && v[0] == '1';
  }();
  static const char* const kCatName[8] = {"attn_full", "attn_window", "dense_gemm", "expert_gemm", "lm_head", "collectives", "router", "quantisers"};
  auto mark = [&](int cat) {  // one event before and one after a call; cat < 0 closes the open interval
    if (nvtx_on) {
      if (cat >= 0 && cat < 8)
        nvtxRangePushA(kCatName[cat]);
      else
        nvtxRangePop();
    }
    if (!prof) return;
    if (prof_used == e->prof_ev.size()) {
      cudaEvent_t ev;
      if (cudaEventCreate(&ev) != cudaSuccess) return;
      e->prof_ev.push_back(ev);
    }
    cudaEventRecord(e->prof_ev[prof_used++], e->stream);
    e->prof_cat.push_back(cat);
  };
  // Dense GEMM; when `splits` is given the split-K partials are left in gemm_ws for a fused consumer.
  auto dense = [&](const uint8_t* x8, const float* sx, const Fp8Weight& w, int N, int K, uint16_t* yout,
                   int32_t* splits, int64_t ldy = 0, int want_splits = 0, int rows = -1) -> int32_t {
    if (rows < 0) rows = T;
    eb_gemm_args g = {};
    g.d_x8 = x8;
    g.d_sx = sx;
    g.d_w8 = w.codes;
    g.d_sw = w.scales;
    g.d_y = yout;
    g.ldy = ldy ? ldy : N;
    g.rows = rows;
    g.N = N;
    g.K = K;
    g.n_groups = 1;
    g.w_tiled = 1;
    g.splits = want_splits;
    g.d_work = (rows <= 512 && N <= std::max(e->nqkv, H)) ? e->gemm_ws : nullptr;
    g.work_bytes = g.d_work ? e->gemm_ws_bytes : 0;
    n += 1;
    return splits ? eb_gemm_fp8_block_partial(&g, splits, st) : eb_gemm_fp8_block(&g, st);
  };
  const int avg2 = std::min(128, 2 * ((R / e->tp_size + E - 1) / E));
  const int group_tn = avg2 <= 16 ? 16 : avg2 <= 32 ? 32 : avg2 <= 64 ? 64 : 128;
  // under row dispatch the segment table covers all experts (global row numbering) and this rank works on its own part
  // small steps: whole-batch planes (see kWholeBatchTokens); large steps: token slices, with the experts by row
  // dispatch from four ranks on
  const bool whole = tp && e->symm != nullptr && T <= kWholeBatchTokens && !e->a2a_forced && !e->slices_forced;
  const bool a2a = tp && e->a2a && !whole && (e->a2a_forced || T >= 1024);
  const int32_t* seg = a2a ? e->seg_off + e->e0 : e->seg_off;
  auto grouped = [&](const uint8_t* x8, const float* sx, const Fp8Weight& w, int N, int K, uint16_t* yout) -> int32_t {
    eb_gemm_args g = {};
    g.d_x8 = x8;
    g.d_sx = sx;
    g.d_w8 = w.codes;
    g.d_sw = w.scales;
    g.d_y = yout;
    g.ldy = N;
    g.rows = R;
    g.N = N;
    g.K = K;
    g.n_groups = E;
    g.d_seg_off = seg;
    g.d_work = e->group_ws;
    g.work_bytes = e->group_ws_bytes;
    g.tile_tokens = group_tn;
    g.tiles_ready = 1;
    g.w_tiled = 1;
    n += 1;
    return eb_gemm_fp8_grouped(&g, st);
  };

  EB_TRY(eb_embed(e->embed, c.vocab, H, d_tokens, T, e->x, st));
  n += 1;
  if (c.debug & 1)
    EB_CUDA(cudaMemcpyAsync(e->dbg_hidden, e->x, (size_t)T * H * 2, cudaMemcpyDeviceToDevice, e->stream));

  auto impose = [&](int l) -> int32_t {  // debug: replace the residual stream before layer l (n_layers = before the head)
    if ((c.debug & 1) && e->force_rows[(size_t)l] == T)
      EB_CUDA(cudaMemcpyAsync(e->x, e->dbg_force + (size_t)l * c.max_tokens * H, (size_t)T * H * 2,
                              cudaMemcpyDeviceToDevice, e->stream));
    return EB_OK;
  };
  // h = rmsnorm(x) of the first layer; later layers get it from the fused combine of the layer before
  bool h8_ready = false;  // tensor parallel: the e4m3 rows and scales of h were gathered, no rank quantises all of h
  EB_TRY(eb_rmsnorm(e->x, e->layers[0].g_attn, T, H, c.rms_eps, e->h, st));
  n += 1;
  for (int l = 0; l < c.n_layers; ++l) {
    const Layer& L = e->layers[(size_t)l];
    const int pi = (l % 2 == 0 && c.window > 0) ? 1 : 0;  // plan 1 = windowed
    const int32_t* bt = (pi && e->ring) ? e->d_bt_ring : e->d_bt;
    const int32_t n_pages = layer_pages(e, l);
    if ((c.debug & 1) && e->force_rows[(size_t)l] == T) {
      EB_TRY(impose(l));
      EB_TRY(eb_rmsnorm(e->x, L.g_attn, T, H, c.rms_eps, e->h, st));
      h8_ready = false;
    }
    int32_t splits = 1;
    if (!h8_ready) {
      mark(7);
      EB_TRY(eb_quant_act_block128(e->h, H, T, H, nullptr, 1, e->h8, e->sh, st));
      mark(-1);
    }
    h8_ready = false;
    mark(2);
    EB_TRY(dense(e->h8, e->sh, L.wqkv, e->nqkv, H, e->qkv, &splits));
    mark(-1);
    EB_TRY(eb_qkv_rope_append_ex((const float*)e->gemm_ws, splits, e->qkv, e->nqkv, e->k_col0, e->v_col0, T, e->hq_l,
                                 e->hkv_l, c.head_dim, d_positions, e->rope_cos, e->rope_sin, max_pos, L.cache,
                                 n_pages, c.page_size, bt, c.max_pages_per_seq, d_tok_slot, st));
    eb_attn_args a = {};
    a.d_q = e->qkv;
    a.q_stride = e->nqkv;
    a.d_out = e->attn;
    a.out_stride = e->hqd;
    a.d_cache = L.cache;
    a.num_pages = n_pages;
    a.d_block_tables = bt;
    a.bt_stride = c.max_pages_per_seq;
    a.d_seq_slots = d_slots;
    a.d_q_off = d_q_off;
    a.d_ctx_lens = d_ctx;
    a.n_seqs = n_seqs;
    a.max_q_len = max_q_len;
    a.d_sinks = L.sinks + e->tp_rank * e->hq_l;
    a.window = pi ? c.window : 0;
    a.n_q = e->hq_l;
    a.n_kv = e->hkv_l;
    a.head_dim = c.head_dim;
    a.page_size = c.page_size;
    a.scale = 0.125f;
    a.d_items = d_items[pi];
    a.n_items = plans[pi].n_items;
    a.d_seq_part = d_seq_part[pi];
    a.n_parts = plans[pi].n_parts;
    a.d_part_acc = e->part_acc;
    a.d_part_ml = e->part_ml;
    mark(pi ? 1 : 0);
    EB_TRY(eb_attn_paged_sink(&a, st));
    mark(-1);
    if (tp && e->o_gather && symm) {
      // C1 on the gathered operand: my heads' columns go, quantised, into every rank's operand (small steps) or into the
      // operand of the rank that owns the rows (large steps); then full-K rows of the projection, the residual and the
      // norm exactly as on one GPU.
      int32_t seq = 0;
      mark(5);
      EB_TRY(eb_quant_act_block128_to_peers(e->symm, e->attn, e->hqd, T, e->hqd, aoff(e->a8g), e->o_cols, aoff(e->sag), e->o_cols / 128,
                                            whole ? 0 : chunk, &seq, st));
      EB_TRY(eb_symm_wait(e->symm, seq, first_exchange ? 32 : 1, st));
      first_exchange = false;
      mark(-1);
      const int r0 = whole ? 0 : t0, nr = whole ? T : nt;
      if (nr > 0) {
        mark(2);
        EB_TRY(dense(e->a8g + (size_t)r0 * e->o_cols, e->sag + (size_t)(r0 / 128) * (e->o_cols / 128), L.wo, H, e->o_cols,
                     e->o + (size_t)r0 * H, &splits, 0, 0, nr));
        mark(-1);
        EB_TRY(eb_oproj_residual_rmsnorm(splits > 1 ? (const float*)e->gemm_ws : nullptr, splits, e->o + (size_t)r0 * H,
                                         e->x + (size_t)r0 * H, L.g_mlp, nr, H, c.rms_eps, e->h + (size_t)r0 * H, st));
      }
      n += 3;
    } else {
    mark(7);
    EB_TRY(eb_quant_act_block128(e->attn, e->hqd, T, e->hqd, nullptr, 1, e->a8, e->sa, st));
    mark(-1);
    mark(2);
    {
      // Decode-sized tensor-parallel steps add the ranks' partials in fp32 (whatever the transport): the projection must
      // then leave fp32 (split-K) planes, not a bf16 result rounded per rank.  The GEMM splits K by itself only while the
      // tiles do not fill the GPU and every split keeps four K blocks; otherwise (8 ranks: K = 512; steps above 256
      // tokens) two splits are asked for.
      const int kb_o = (e->hqd + 127) / 128;
      const int o_splits = (tp && T <= kWholeBatchTokens && !(kb_o >= 8 && T <= 256) && kb_o >= 2) ? 2 : 0;
      EB_TRY(dense(e->a8, e->sa, L.wo, H, e->hqd, e->o, &splits, 0, o_splits));
    }
    mark(-1);
    if (!tp) {
      EB_TRY(eb_oproj_residual_rmsnorm(splits > 1 ? (const float*)e->gemm_ws : nullptr, splits, e->o, e->x, L.g_mlp, T, H,
                                       c.rms_eps, e->h, st));
    } else {
      // C1: this rank's heads contributed a partial [T, H].  Reduce-scatter the partials over token slices; the owner
      // of a slice adds the residual, rounds once and normalises; the normalised rows are gathered below.  Prefill-
      // sized steps have the partial in bf16 already (the GEMM's output) and scatter it as such, half the bytes;
      // decode-sized steps sum their split-K planes in fp32 and scatter fp32.
      if (whole) {
        // every rank gets every rank's partial and adds them itself, in rank order: residual, norm and routing then run
        // on all rows everywhere with identical bits, and nothing has to be gathered
        const int esz = splits == 1 ? 2 : 4;
        int32_t seq = 0, patience = 1;
        mark(5);
        if (splits > 1) {  // the sum of the split-K planes goes straight into every rank's plane
          EB_TRY(eb_sum_planes_f32_to_peers(e->symm, aoff(e->planes), (int64_t)T * H * 4, (const float*)e->gemm_ws, splits, (int64_t)T * H,
                                            &seq, st));
          patience = first_exchange ? 32 : 1;
          first_exchange = false;
        } else {
          EB_TRY(share_planes(e->o, esz, &seq, &patience));
        }
        EB_TRY(eb_planes_residual_rmsnorm_after(e->symm, seq, patience, e->planes, esz == 2, e->tp_size, (int64_t)T * H, e->x, L.g_mlp, T,
                                                H, c.rms_eps, e->h, st));
        mark(-1);
        n += 2;
      } else if (splits == 1) {
        mark(5);
        if (symm) {  // the ranks' bf16 planes of my slice, added in rank order in fp32, rounded once
          EB_TRY(scatter_planes_norm(e->o, 2, L.g_mlp));
          mark(-1);
        } else {
          EB_TRY(eb_comm_reduce_scatter_bf16(e->comm, e->o, (int64_t)chunk * H, st));
          mark(-1);
          EB_TRY(eb_oproj_residual_rmsnorm(nullptr, 1, e->o + (size_t)t0 * H, e->x + (size_t)t0 * H, L.g_mlp, nt, H, c.rms_eps,
                                           e->h + (size_t)t0 * H, st));
        }
        n += 1;
      } else {
        EB_TRY(eb_sum_planes_f32((const float*)e->gemm_ws, splits, e->o, (int64_t)T * H, e->ar_buf, st));
        mark(5);
        if (symm) {
          EB_TRY(scatter_planes_norm(e->ar_buf, 4, L.g_mlp));
          mark(-1);
        } else {
          EB_TRY(eb_comm_reduce_scatter_f32(e->comm, e->ar_buf, (int64_t)chunk * H, st));
          mark(-1);
          EB_TRY(eb_oproj_residual_rmsnorm(e->ar_buf + (size_t)t0 * H, 1, nullptr, e->x + (size_t)t0 * H, L.g_mlp, nt, H, c.rms_eps,
                                           e->h + (size_t)t0 * H, st));
        }
        n += 2;
      }
    }
    }
    mark(6);
    if (!tp || whole) {
      EB_TRY(eb_moe_route(e->h, L.wr, T, c.n_experts, H, c.top_k, e->r_idx, e->r_wts, nullptr, st));
      mark(-1);
    } else {
      // every rank routes its slice of the tokens, then normalised rows and routing are gathered in one group: the
      // same bits as doing all tokens everywhere, at 1/tp_size of the work
      if (nt > 0)
        EB_TRY(eb_moe_route(e->h + (size_t)t0 * H, L.wr, nt, c.n_experts, H, c.top_k, e->r_idx + (size_t)t0 * c.top_k,
                            e->r_wts + (size_t)t0 * c.top_k, nullptr, st));
      mark(-1);
      // row dispatch needs only the routing everywhere; the normalised rows travel to their experts' ranks below
      void* bufs[3] = {e->r_idx, e->r_wts, e->h};
      const int64_t sizes[3] = {(int64_t)chunk * c.top_k * 4, (int64_t)chunk * c.top_k * 4, (int64_t)chunk * H * 2};
      const int64_t valid[3] = {(int64_t)nt * c.top_k * 4, (int64_t)nt * c.top_k * 4, (int64_t)nt * H * 2};
      mark(5);
      EB_TRY(gather(a2a ? 2 : 3, bufs, sizes, valid));
      mark(-1);
      n += 1;
    }
    if (!tp) {
      EB_TRY(eb_moe_permute_tiles(e->r_idx, T, c.top_k, E, e->seg_off, e->perm_row, e->row_token, group_tn, e->group_ws, st));
      mark(7);
      EB_TRY(eb_quant_gather_block128(e->h, H, T, e->row_token, R, H, e->seg_off, E, e->xp8, e->sxp, st));
      mark(-1);
    } else if (a2a) {
      // C2 as a row exchange: every rank sorts ALL routed slots by expert (the routing is the same everywhere), so a
      // slot's row number is known to sender and receiver alike; the owner of a token stores its normalised row into
      // the arena of each of its experts' ranks at that row, and the outputs come back the same way
      EB_TRY(eb_moe_permute(e->r_idx, T, c.top_k, c.n_experts, e->seg_off, e->perm_row, e->row_token, st));
      EB_TRY(eb_gemm_group_tiles(seg, E, R, group_tn, e->group_ws, st));
      int32_t seq = 0;
      mark(5);
      EB_TRY(eb_symm_dispatch_rows(e->symm, aoff(e->h), aoff(e->xp16), H * 2, e->r_idx, e->perm_row, t0, nt, c.top_k, E, c.n_experts, R,
                                   &seq, st));
      EB_TRY(eb_symm_wait(e->symm, seq, 1, st));
      mark(-1);
      mark(7);
      EB_TRY(eb_quant_act_block128(e->xp16, H, R, H, seg, E, e->xp8, e->sxp, st));
      mark(-1);
      n += 3;
    } else {
      // routing is replicated; keep the slots of this rank's experts only
      EB_TRY(eb_moe_localize(e->r_idx, T * c.top_k, e->e0, E, e->r_idx_local, st));
      EB_TRY(eb_moe_permute_tiles_local(e->r_idx_local, T, c.top_k, E, e->seg_off, e->perm_row, e->row_token, group_tn,
                                        e->group_ws, st));
      n += 1;
      mark(7);
      EB_TRY(eb_quant_gather_block128(e->h, H, T, e->row_token, R, H, e->seg_off, E, e->xp8, e->sxp, st));
      mark(-1);
    }
    mark(3);
    EB_TRY(grouped(e->xp8, e->sxp, L.w1, 2 * I, H, e->gu));
    mark(-1);
    mark(7);
    EB_TRY(eb_quant_silu_mul_block128(e->gu, 2 * I, R, I, seg, E, e->act8, e->sact, st));
    mark(-1);
    mark(3);
    EB_TRY(grouped(e->act8, e->sact, L.w2, H, I, e->y));
    mark(-1);
    const float* g_next = (l + 1 < c.n_layers) ? e->layers[(size_t)l + 1].g_attn : e->g_final;
    if (!tp) {
      EB_TRY(eb_moe_combine_rmsnorm(e->y, e->perm_row, e->r_wts, T, c.top_k, H, e->x, g_next, c.rms_eps, e->h, st));
    } else {
      if (a2a) {
        // the expert outputs return to their tokens' owners, who mix the four rows of a token exactly as one GPU would
        int32_t seq = 0;
        mark(5);
        EB_TRY(eb_symm_return_rows(e->symm, aoff(e->y), aoff(e->y), H * 2, e->row_token, e->seg_off, e->e0, E, chunk, R, &seq, st));
        EB_TRY(eb_symm_wait(e->symm, seq, 1, st));
        mark(-1);
        EB_TRY(eb_moe_combine_rmsnorm_ex(e->y, e->perm_row + (size_t)t0 * c.top_k, e->r_wts + (size_t)t0 * c.top_k, nt, c.top_k, H, R,
                                         e->x + (size_t)t0 * H, g_next, c.rms_eps, e->h + (size_t)t0 * H, st));
      } else {
        // C2 without an exchange of rows: every rank holds every token, mixes its own experts' outputs into a partial
        // [T, H] and the partials are summed over token slices
        if (whole) {
          // this rank's experts' mix of every token goes straight into every rank's plane
          int32_t seq = 0, patience = first_exchange ? 32 : 1;
          first_exchange = false;
          mark(5);
          EB_TRY(eb_moe_combine_bf16_to_peers(e->symm, aoff(e->planes), (int64_t)T * H * 2, e->y, e->perm_row, e->r_wts, T, c.top_k, H, &seq,
                                              st));
          EB_TRY(eb_planes_residual_rmsnorm_after(e->symm, seq, patience, e->planes, 1, e->tp_size, (int64_t)T * H, e->x, g_next, T, H,
                                                  c.rms_eps, e->h, st));
          mark(-1);
          n += 2;
          goto layer_done;  // every rank holds every normalised row: the next consumer quantises them itself
        }
        EB_TRY(eb_moe_combine_bf16(e->y, e->perm_row, e->r_wts, T, c.top_k, H, e->o, st));
        mark(5);
        if (symm) {
          EB_TRY(scatter_planes_norm(e->o, 2, g_next));
          mark(-1);
        } else {
          EB_TRY(eb_comm_reduce_scatter_bf16(e->comm, e->o, (int64_t)chunk * H, st));
          mark(-1);
          EB_TRY(eb_oproj_residual_rmsnorm(nullptr, 1, e->o + (size_t)t0 * H, e->x + (size_t)t0 * H, g_next, nt, H, c.rms_eps,
                                           e->h + (size_t)t0 * H, st));
        }
      }
      // the next consumer (QKV projection of the next layer, or the LM head) needs every token's normalised row as
      // e4m3 with block scales: the slice's owner quantises its rows and the codes and scales are gathered (half the
      // bytes of the bf16 rows, and no rank quantises the whole batch).  The residual stream itself stays sliced,
      // except when the debug taps want it whole (then the bf16 rows travel too).
      mark(7);
      EB_TRY(eb_quant_act_block128(e->h + (size_t)t0 * H, H, nt, H, nullptr, 1, e->h8 + (size_t)t0 * H,
                                   e->sh + (size_t)(t0 / 128) * e->kbH, st));
      mark(-1);
      void* bufs[3] = {e->h8, e->sh, e->x};
      const int64_t sizes[3] = {(int64_t)chunk * H, (int64_t)(chunk / 128) * e->kbH * 4, (int64_t)chunk * H * 2};
      const int64_t valid[3] = {(int64_t)nt * H, (int64_t)((nt + 127) / 128) * e->kbH * 4, (int64_t)nt * H * 2};
      mark(5);
      EB_TRY(gather((c.debug & 1) ? 3 : 2, bufs, sizes, valid));
      mark(-1);
      h8_ready = true;
      n += 3;
    }
  layer_done:
    n += 9 + (plans[pi].n_parts > n_seqs ? 1 : 0);
    if (c.debug & 1) {
      EB_CUDA(cudaMemcpyAsync(e->dbg_route + (size_t)l * c.max_tokens * c.top_k, e->r_idx, (size_t)R * sizeof(int32_t),
                              cudaMemcpyDeviceToDevice, e->stream));
      EB_CUDA(cudaMemcpyAsync(e->dbg_hidden + (size_t)(l + 1) * c.max_tokens * H, e->x, (size_t)T * H * 2,
                              cudaMemcpyDeviceToDevice, e->stream));
    }
  }
  if ((c.debug & 1) && e->force_rows[(size_t)c.n_layers] == T) {
    EB_TRY(impose(c.n_layers));
    EB_TRY(eb_rmsnorm(e->x, e->g_final, T, H, c.rms_eps, e->h, st));
    h8_ready = false;
  }
  if (!h8_ready) EB_TRY(eb_quant_act_block128(e->h, H, T, H, nullptr, 1, e->h8, e->sh, st));
  // rows the head runs over: all of them, or (prefill) the 128-row scale blocks that hold a wanted row, as ranges
  std::vector<std::pair<int, int>> ranges;  // (first row, rows)
  if (!e->head_rows_on) {
    ranges.emplace_back(0, T);
  } else {
    std::vector<int32_t> rows = e->head_rows;
    std::sort(rows.begin(), rows.end());
    for (int32_t r : rows) {
      if (r < 0 || r >= T) continue;
      const int b0 = r / 128 * 128, b1 = std::min(T, b0 + 128);
      if (!ranges.empty() && ranges.back().first + ranges.back().second >= b0)
        ranges.back().second = std::max(ranges.back().second, b1 - ranges.back().first);
      else
        ranges.emplace_back(b0, b1 - b0);
    }
  }
  mark(4);
  if (!tp) {
    for (const auto& rg : ranges) {
      EB_TRY(dense(e->h8 + (size_t)rg.first * H, e->sh + (size_t)(rg.first / 128) * e->kbH, e->lm, c.vocab, H,
                   e->logits + (size_t)rg.first * c.vocab, nullptr, 0, 0, rg.second));
      EB_TRY(eb_argmax(e->logits + (size_t)rg.first * c.vocab, rg.second, c.vocab, c.vocab, e->d_next + rg.first, e->d_margin + rg.first, st));
      if (e->d_samp)  // rows of sequences with a temperature: the drawn token replaces the greedy one
        EB_TRY(eb_sample_top_p(e->logits + (size_t)rg.first * c.vocab, rg.second, c.vocab, c.vocab,
                               reinterpret_cast<const float*>(e->d_samp) + rg.first,
                               reinterpret_cast<const uint32_t*>(e->d_samp) + T + rg.first,
                               reinterpret_cast<const uint32_t*>(e->d_samp) + 2 * (size_t)T + rg.first, e->d_next + rg.first, st));
    }
    mark(-1);
  } else {
    // vocabulary-parallel head: logits of this rank's rows only, one candidate per token and rank, merged everywhere
    const int64_t cap = c.max_tokens;
    for (const auto& rg : ranges) {
      EB_TRY(dense(e->h8 + (size_t)rg.first * H, e->sh + (size_t)(rg.first / 128) * e->kbH, e->lm, e->v1 - e->v0, H,
                   e->logits + (size_t)rg.first * c.vocab + e->v0, nullptr, c.vocab, 0, rg.second));
      EB_TRY(eb_argmax_partial(e->logits + (size_t)rg.first * c.vocab + e->v0, rg.second, e->v1 - e->v0, c.vocab, e->v0,
                               e->cand + ((size_t)e->tp_rank * cap + rg.first) * 4, st));
    }
    mark(-1);
    if (!ranges.empty()) {  // every rank has the same ranges: all of them meet the exchange or none does
      void* cb[1] = {e->cand};
      const int64_t csz[1] = {cap * 4 * (int64_t)sizeof(float)};
      const int64_t cvalid[1] = {(int64_t)T * 4 * (int64_t)sizeof(float)};
      mark(5);
      EB_TRY(gather(1, cb, csz, cvalid));
      mark(-1);
      EB_TRY(eb_argmax_merge(e->cand, e->tp_size, cap, T, e->d_next, e->d_margin, st));
    }
    n += 2;
  }
  n += 3;
  return EB_OK;
}

int32_t step_launch_body(eb_engine* e, const int32_t* h_slots, const int32_t* h_q_lens, int32_t n_seqs,
                         const int32_t* h_tokens, int T, int max_q);

}  // namespace

extern "C" {

int32_t eb_engine_create(const eb_config* cfg, eb_engine** out) { return eb_engine_create_tp(cfg, 0, 1, nullptr, out); }

int32_t eb_engine_create_tp(const eb_config* cfg, int32_t tp_rank, int32_t tp_size, eb_comm* comm, eb_engine** out) {
  EB_REQUIRE(out, EB_ERR_ARG, "eb_engine_create: null out");
  EB_TRY(validate(cfg));
  EB_REQUIRE(tp_size >= 1 && tp_rank >= 0 && tp_rank < tp_size, EB_ERR_ARG, "eb_engine_create_tp: rank %d of %d", tp_rank, tp_size);
  EB_REQUIRE(tp_size == 1 || comm, EB_ERR_ARG, "eb_engine_create_tp: %d ranks need a communicator", tp_size);
  EB_REQUIRE(cfg->n_kv_heads % tp_size == 0 && cfg->n_experts % tp_size == 0, EB_ERR_UNSUPPORTED,
             "eb_engine_create_tp: %d KV heads / %d experts do not divide over %d ranks", cfg->n_kv_heads, cfg->n_experts, tp_size);
  EB_REQUIRE(tp_size == 1 || cfg->n_q_heads == 8 * cfg->n_kv_heads, EB_ERR_UNSUPPORTED,
             "eb_engine_create_tp: tensor parallelism is built for groups of 8 query heads per KV head");
  EB_REQUIRE(tp_size == 1 || ((cfg->n_q_heads / tp_size) * cfg->head_dim) % 128 == 0, EB_ERR_UNSUPPORTED,
             "eb_engine_create_tp: the query heads of a rank must fill whole 128-row scale blocks");
  eb_engine* e = new (std::nothrow) eb_engine;
  EB_REQUIRE(e, EB_ERR_NOMEM, "eb_engine_create: host allocation failed");
  e->c = *cfg;
  const eb_config& c = e->c;
  int dev = 0;
  cudaDeviceProp prop;
  cudaError_t err = cudaGetDevice(&dev);
  if (err == cudaSuccess) err = cudaGetDeviceProperties(&prop, dev);
  if (err != cudaSuccess) {
    delete e;
    return eb::fail(EB_ERR_NODEVICE, "eb_engine_create: %s", cudaGetErrorString(err));
  }
  if (prop.major != 10) {
    delete e;
    return eb::fail(EB_ERR_NODEVICE, "eb_engine_create: compute capability %d.%d (built for sm_100a only)", prop.major,
                    prop.minor);
  }
  e->sm_count = prop.multiProcessorCount;
  e->tp_rank = tp_rank;
  e->tp_size = tp_size;
  e->comm = comm;
  e->hq_l = c.n_q_heads / tp_size;
  e->hkv_l = c.n_kv_heads / tp_size;
  e->e_l = c.n_experts / tp_size;
  e->e0 = tp_rank * e->e_l;
  {
    const int blocks = (c.vocab + 127) / 128, per = (blocks + tp_size - 1) / tp_size;
    e->v0 = std::min(c.vocab, tp_rank * per * 128);
    e->v1 = std::min(c.vocab, (tp_rank + 1) * per * 128);
    if (e->v1 <= e->v0) {
      delete e;
      return eb::fail(EB_ERR_UNSUPPORTED, "eb_engine_create_tp: vocabulary %d has fewer 128-row blocks than %d ranks can share",
                      c.vocab, tp_size);
    }
  }
  e->hqd = e->hq_l * c.head_dim;
  if (tp_size == 1) {
    e->kv_band = e->hkv_l * c.head_dim;  // the fused [q | k | v] row as it is
    e->k_col0 = e->hqd;
    e->v_col0 = e->hqd + e->kv_band;
  } else {
    e->kv_band = (int)eb::cdiv(e->hkv_l * c.head_dim, 128) * 128;
    const int koff = (tp_rank * e->hkv_l * c.head_dim) % 128;  // this rank's heads inside a shared 128-row block
    e->k_col0 = e->hqd + koff;
    e->v_col0 = e->hqd + e->kv_band + koff;
  }
  e->nqkv = e->hqd + 2 * e->kv_band;
  e->kbH = (int)eb::cdiv(c.hidden, 128);
  e->kbI = (int)eb::cdiv(c.inter, 128);
  e->kbA = (int)eb::cdiv(e->hqd, 128);
  // a ring of window pages has to hold a whole chunk besides the window: chunks stay short when rings are asked for
  e->chunk_cap = std::max(c.max_q_len, (c.window_ring && c.window > 0) ? std::min(c.max_tokens, 256) : c.max_tokens);
  {
    const char* nccl = getenv("EIDOLA_B200_TP_NCCL");
    const char* og = getenv("EIDOLA_B200_TP_OGATHER");
    // measured: 2 % slower than the partial planes on 2 ranks (bytes do not matter there), 2 % faster on 4
    e->o_gather = tp_size > 1 && !(nccl && nccl[0] == '1') && (og ? og[0] == '1' : tp_size >= 4);
    e->o_cols = e->o_gather ? c.n_q_heads * c.head_dim : e->hqd;
  }
  e->layers.resize((size_t)c.n_layers);
  e->uploaded_pages.assign((size_t)c.max_seqs, 0);
  e->high_len.assign((size_t)c.max_seqs, 0);
  e->samp_scale.assign((size_t)c.max_seqs, 0.f);
  e->samp_q24.assign((size_t)c.max_seqs, 1u << 24);
  e->samp_seed.assign((size_t)c.max_seqs, 0);
  int32_t rc = EB_OK;
  do {
    if (cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreate(&e->ev0) != cudaSuccess || cudaEventCreate(&e->ev1) != cudaSuccess) {
      rc = eb::fail(EB_ERR_NODEVICE, "eb_engine_create: stream/event creation failed");
      break;
    }
    if ((rc = eb_sched_create(c.num_pages, c.page_size, c.max_seqs, c.max_pages_per_seq, c.seed, &e->sched)) != EB_OK) break;
    if ((rc = init_weights(e)) != EB_OK) break;
    e->ring = (c.window_ring && c.window > 0) ? (c.window + e->chunk_cap + c.page_size - 1) / c.page_size + 1 : 0;
    for (int l = 0; l < c.n_layers && rc == EB_OK; ++l) {
      const size_t cache_elems = (size_t)layer_pages(e, l) * 2 * e->hkv_l * c.page_size * c.head_dim;
      rc = dev_alloc(e, &e->layers[(size_t)l].cache, cache_elems, &e->kv_bytes);
      if (rc == EB_OK && cudaMemsetAsync(e->layers[(size_t)l].cache, 0, cache_elems * 2, e->stream) != cudaSuccess)
        rc = eb::fail(EB_ERR_NODEVICE, "eb_engine_create: cache memset failed");
    }
    if (rc == EB_OK && e->ring) {
      std::vector<int32_t> t((size_t)c.max_seqs * c.max_pages_per_seq);
      for (int s_ = 0; s_ < c.max_seqs; ++s_)
        for (int p_ = 0; p_ < c.max_pages_per_seq; ++p_) t[(size_t)s_ * c.max_pages_per_seq + p_] = s_ * e->ring + p_ % e->ring;
      rc = dev_alloc(e, &e->d_bt_ring, t.size(), &e->work_bytes);
      if (rc == EB_OK && cudaMemcpy(e->d_bt_ring, t.data(), t.size() * sizeof(int32_t), cudaMemcpyHostToDevice) != cudaSuccess)
        rc = eb::fail(EB_ERR_NODEVICE, "eb_engine_create: ring table upload failed");
    }
    if (rc != EB_OK) break;
    if ((rc = init_work(e)) != EB_OK) break;
    if (cudaStreamSynchronize(e->stream) != cudaSuccess) rc = eb::fail(EB_ERR_NODEVICE, "eb_engine_create: sync failed");
  } while (0);
  if (rc != EB_OK) {
    eb_engine_destroy(e);
    return rc;
  }
  *out = e;
  return EB_OK;
}

int32_t eb_engine_destroy(eb_engine* e) {
  if (!e) return EB_OK;
  if (e->stream) cudaStreamSynchronize(e->stream);
  for (void* p : e->allocs) cudaFree(p);
  if (e->w_scratch) cudaFree(e->w_scratch);
  if (e->symm) eb_symm_destroy(e->symm);
  for (cudaEvent_t ev : e->prof_ev) cudaEventDestroy(ev);
  if (e->h_stage) cudaFreeHost(e->h_stage);
  if (e->h_result) cudaFreeHost(e->h_result);
  if (e->ev0) cudaEventDestroy(e->ev0);
  if (e->ev1) cudaEventDestroy(e->ev1);
  if (e->stream) cudaStreamDestroy(e->stream);
  if (e->sched) eb_sched_destroy(e->sched);
  delete e;
  return EB_OK;
}

int32_t eb_engine_memory(const eb_engine* e, int64_t* weight_bytes, int64_t* kv_bytes, int64_t* work_bytes) {
  EB_REQUIRE(e, EB_ERR_ARG, "eb_engine_memory: null engine");
  if (weight_bytes) *weight_bytes = e->weight_bytes;
  if (kv_bytes) *kv_bytes = e->kv_bytes;
  if (work_bytes) *work_bytes = e->work_bytes;
  return EB_OK;
}

namespace {

struct LoadCtx {
  eb::GgufFile gg;
  std::vector<float> host;   // one band of rows as fp32
  float* d_f32 = nullptr;    // the same on the device
  uint8_t* d_codes = nullptr;  // its e4m3 codes, row-major, before tiling
  int64_t band_rows = 8192, max_cols = 0;
  ~LoadCtx() {
    if (d_f32) cudaFree(d_f32);
    if (d_codes) cudaFree(d_codes);
  }
};

// Tensor `name` must exist with `cols` columns and rows_total * groups rows (GGUF extents are innermost first).
int32_t find_tensor(LoadCtx& L, const std::string& name, int64_t groups, int64_t rows_total, int64_t cols, const eb::GgufTensor** out) {
  const eb::GgufTensor* t = L.gg.find(name);
  EB_REQUIRE(t, EB_ERR_ARG, "eb_engine_load_gguf: tensor %s is missing", name.c_str());
  EB_REQUIRE(t->ne[0] == cols && t->elements() == groups * rows_total * cols, EB_ERR_ARG,
             "eb_engine_load_gguf: tensor %s has %lld elements in rows of %lld, the configuration needs %lld x %lld x %lld", name.c_str(),
             (long long)t->elements(), (long long)t->ne[0], (long long)groups, (long long)rows_total, (long long)cols);
  *out = t;
  return EB_OK;
}

// rows [src_row0, +nrows) of group `src_group` of tensor t, fp32 on the device (d_f32, row pitch = cols_total)
int32_t stage_rows(eb_engine* e, LoadCtx& L, const eb::GgufTensor& t, int64_t rows_total, int64_t cols_total, int64_t src_group,
                   int64_t src_row0, int64_t nrows) {
  EB_TRY(L.gg.read_f32(t, (src_group * rows_total + src_row0) * cols_total, nrows * cols_total, L.host.data()));
  EB_CUDA(cudaMemcpyAsync(L.d_f32, L.host.data(), (size_t)(nrows * cols_total) * sizeof(float), cudaMemcpyHostToDevice, e->stream));
  EB_CUDA(cudaStreamSynchronize(e->stream));  // the host band is reused by the next read
  return EB_OK;
}

// A linear layer's rows [src_row0, +nrows) x columns [col0, +ncols) -> e4m3 + block scales -> tiles at weight-row block
// dst_row0 / 128 of group dst_group of w (whose groups have rows_per_group rows).  Bands start on 128-row boundaries.
int32_t load_linear(eb_engine* e, LoadCtx& L, const eb::GgufTensor& t, int64_t rows_total, int64_t cols_total, int64_t src_group,
                    int64_t src_row0, int64_t nrows, int64_t col0, int64_t ncols, Fp8Weight* w, int64_t dst_group,
                    int64_t rows_per_group, int64_t dst_row0, float* scales_dst) {
  const int64_t KB = eb::cdiv(ncols, 128), NB = eb::cdiv(rows_per_group, 128);
  for (int64_t r = 0; r < nrows; r += L.band_rows) {
    const int64_t n = std::min(L.band_rows, nrows - r);
    EB_TRY(stage_rows(e, L, t, rows_total, cols_total, src_group, src_row0 + r, n));
    EB_TRY(eb_quant_weight_f32(L.d_f32 + col0, cols_total, n, ncols, L.d_codes, scales_dst + (r / 128) * KB, e->stream));
    uint8_t* dst = w->codes + ((dst_group * NB + (dst_row0 + r) / 128) * KB) * (int64_t)(128 * 128);
    EB_TRY(eb_weight_tile_fp8(L.d_codes, 1, (int32_t)n, (int32_t)ncols, dst, e->stream));
  }
  return EB_OK;
}

// A small tensor kept as it is: fp32 (to_bf16 = false) or bf16.
int32_t load_plain(eb_engine* e, LoadCtx& L, const eb::GgufTensor& t, int64_t rows, int64_t cols, void* d_dst, bool to_bf16) {
  for (int64_t r = 0; r < rows; r += L.band_rows) {
    const int64_t n = std::min(L.band_rows, rows - r);
    EB_TRY(stage_rows(e, L, t, rows, cols, 0, r, n));
    if (to_bf16)
      EB_TRY(eb_f32_to_bf16(L.d_f32, (uint16_t*)d_dst + r * cols, n * cols, e->stream));
    else
      EB_CUDA(cudaMemcpyAsync((float*)d_dst + r * cols, L.d_f32, (size_t)(n * cols) * sizeof(float), cudaMemcpyDeviceToDevice, e->stream));
  }
  return EB_OK;
}

}  // namespace

int32_t eb_engine_load_gguf(eb_engine* e, const char* path) {
  EB_REQUIRE(e && path, EB_ERR_ARG, "eb_engine_load_gguf: null");
  EB_REQUIRE(!e->in_flight, EB_ERR_STATE, "eb_engine_load_gguf: a step is in flight");
  const eb_config& c = e->c;
  const int64_t H = c.hidden, I = c.inter, E = e->e_l, D = c.head_dim;
  const int64_t hqd_g = (int64_t)c.n_q_heads * D, hkd_g = (int64_t)c.n_kv_heads * D, nqkv_g = hqd_g + 2 * hkd_g;
  LoadCtx L;
  EB_TRY(L.gg.open(path));
  L.max_cols = std::max(std::max(H, I), hqd_g);
  L.host.resize((size_t)(L.band_rows * L.max_cols));
  EB_CUDA(cudaMalloc((void**)&L.d_f32, (size_t)(L.band_rows * L.max_cols) * sizeof(float)));
  EB_CUDA(cudaMalloc((void**)&L.d_codes, (size_t)(L.band_rows * L.max_cols)));
  const eb::GgufTensor* t = nullptr;
  const int64_t kv_row0 = ((int64_t)e->tp_rank * e->hkv_l * D) / 128 * 128;
  char name[128];
  for (int l = 0; l < c.n_layers; ++l) {
    Layer& Ly = e->layers[(size_t)l];
    snprintf(name, sizeof(name), "blk.%d.attn_qkv.weight", l);
    EB_TRY(find_tensor(L, name, 1, nqkv_g, H, &t));
    const int64_t band_rows[3] = {e->hqd, e->kv_band, e->kv_band};
    const int64_t band_src[3] = {(int64_t)e->tp_rank * e->hqd, hqd_g + kv_row0, hqd_g + hkd_g + kv_row0};
    int64_t dst_row = 0;
    for (int b = 0; b < 3; ++b) {
      EB_TRY(load_linear(e, L, *t, nqkv_g, H, 0, band_src[b], band_rows[b], 0, H, &Ly.wqkv, 0, e->nqkv, dst_row,
                         Ly.wqkv.scales + (dst_row / 128) * e->kbH));
      dst_row += band_rows[b];
    }
    snprintf(name, sizeof(name), "blk.%d.attn_output.weight", l);
    EB_TRY(find_tensor(L, name, 1, H, hqd_g, &t));
    EB_TRY(load_linear(e, L, *t, H, hqd_g, 0, 0, H, e->o_gather ? 0 : (int64_t)e->tp_rank * e->hqd, e->o_cols, &Ly.wo, 0, H, 0,
                       Ly.wo.scales));
    snprintf(name, sizeof(name), "blk.%d.ffn_gate_up_exps.weight", l);
    EB_TRY(find_tensor(L, name, c.n_experts, 2 * I, H, &t));
    const eb::GgufTensor* td = nullptr;
    snprintf(name, sizeof(name), "blk.%d.ffn_down_exps.weight", l);
    EB_TRY(find_tensor(L, name, c.n_experts, H, I, &td));
    const int64_t s1 = eb::cdiv(2 * I, 128) * e->kbH, s2 = eb::cdiv(H, 128) * e->kbI;
    for (int64_t x = 0; x < E; ++x) {
      EB_TRY(load_linear(e, L, *t, 2 * I, H, e->e0 + x, 0, 2 * I, 0, H, &Ly.w1, x, 2 * I, 0, Ly.w1.scales + x * s1));
      EB_TRY(load_linear(e, L, *td, H, I, e->e0 + x, 0, H, 0, I, &Ly.w2, x, H, 0, Ly.w2.scales + x * s2));
    }
    snprintf(name, sizeof(name), "blk.%d.ffn_gate_inp.weight", l);
    EB_TRY(find_tensor(L, name, 1, c.n_experts, H, &t));
    EB_TRY(load_plain(e, L, *t, c.n_experts, H, Ly.wr, true));
    snprintf(name, sizeof(name), "blk.%d.attn_sinks.weight", l);
    EB_TRY(find_tensor(L, name, 1, 1, c.n_q_heads, &t));
    EB_TRY(load_plain(e, L, *t, 1, c.n_q_heads, Ly.sinks, false));
    snprintf(name, sizeof(name), "blk.%d.attn_norm.weight", l);
    EB_TRY(find_tensor(L, name, 1, 1, H, &t));
    EB_TRY(load_plain(e, L, *t, 1, H, Ly.g_attn, false));
    snprintf(name, sizeof(name), "blk.%d.ffn_norm.weight", l);
    EB_TRY(find_tensor(L, name, 1, 1, H, &t));
    EB_TRY(load_plain(e, L, *t, 1, H, Ly.g_mlp, false));
  }
  EB_TRY(find_tensor(L, "token_embd.weight", 1, c.vocab, H, &t));
  EB_TRY(load_plain(e, L, *t, c.vocab, H, e->embed, true));
  EB_TRY(find_tensor(L, "output.weight", 1, c.vocab, H, &t));
  EB_TRY(load_linear(e, L, *t, c.vocab, H, 0, e->v0, e->v1 - e->v0, 0, H, &e->lm, 0, e->v1 - e->v0, 0, e->lm.scales));
  EB_TRY(find_tensor(L, "output_norm.weight", 1, 1, H, &t));
  EB_TRY(load_plain(e, L, *t, 1, H, e->g_final, false));
  EB_CUDA(cudaStreamSynchronize(e->stream));
  return EB_OK;
}

int32_t eb_engine_kv_fill_synth(eb_engine* e) {
  EB_REQUIRE(e, EB_ERR_ARG, "eb_engine_kv_fill_synth: null engine");
  const eb_config& c = e->c;
  for (int l = 0; l < c.n_layers; ++l)
    EB_TRY(eb_synth_kv_heads_bf16(e->layers[(size_t)l].cache, layer_pages(e, l), c.n_kv_heads, e->tp_rank * e->hkv_l, e->hkv_l,
                                  c.page_size, c.head_dim, c.seed, 20000 + (uint64_t)l, e->stream));
  EB_CUDA(cudaStreamSynchronize(e->stream));
  return EB_OK;
}

int32_t eb_engine_seq_admit(eb_engine* e, int32_t context_len, int32_t* slot) {
  EB_REQUIRE(e && slot, EB_ERR_ARG, "eb_engine_seq_admit: null");
  EB_REQUIRE(!e->in_flight, EB_ERR_STATE, "eb_engine_seq_admit: a step is in flight");
  EB_TRY(eb_sched_admit(e->sched, context_len, slot));
  e->uploaded_pages[(size_t)*slot] = 0;
  e->high_len[(size_t)*slot] = context_len;
  e->samp_scale[(size_t)*slot] = 0.f;  // a new sequence decodes greedily until eb_engine_seq_sampling says otherwise
  return EB_OK;
}

int32_t eb_engine_seq_admit_evicting(eb_engine* e, int32_t context_len, int32_t* slot, int32_t* h_evicted, int32_t cap,
                                     int32_t* n_evicted) {
  EB_REQUIRE(e && slot && n_evicted, EB_ERR_ARG, "eb_engine_seq_admit_evicting: null");
  EB_REQUIRE(!e->in_flight, EB_ERR_STATE, "eb_engine_seq_admit_evicting: a step is in flight");
  EB_TRY(eb_sched_admit_evicting(e->sched, context_len, e->tick, slot, h_evicted, cap, n_evicted));
  for (int32_t i = 0; i < *n_evicted; ++i) e->uploaded_pages[(size_t)h_evicted[i]] = 0;
  e->uploaded_pages[(size_t)*slot] = 0;
  e->high_len[(size_t)*slot] = context_len;
  e->samp_scale[(size_t)*slot] = 0.f;
  return EB_OK;
}

int32_t eb_engine_seq_pin(eb_engine* e, int32_t slot, int32_t pinned) {
  EB_REQUIRE(e, EB_ERR_ARG, "eb_engine_seq_pin: null");
  return eb_sched_set_flags(e->sched, slot, pinned ? 1 : 0, -1);
}

int32_t eb_engine_seq_sampling(eb_engine* e, int32_t slot, float temperature, float top_p, uint64_t seed) {
  EB_REQUIRE(e, EB_ERR_ARG, "eb_engine_seq_sampling: null");
  EB_REQUIRE(!e->in_flight, EB_ERR_STATE, "eb_engine_seq_sampling: a step is in flight");
  EB_REQUIRE(e->tp_size == 1 || !(temperature > 0.f), EB_ERR_UNSUPPORTED,
             "eb_engine_seq_sampling: the sampler needs whole logit rows; under tensor parallelism the LM head is split over the vocabulary");
  int32_t len = 0;
  EB_TRY(eb_sched_seq_len(e->sched, slot, &len));  // refuses a slot that is not live
  EB_REQUIRE(!(temperature > 0.f) || (temperature >= 1e-3f && temperature <= 100.f), EB_ERR_ARG,
             "eb_engine_seq_sampling: temperature %g outside [0.001, 100]", (double)temperature);
  EB_REQUIRE(top_p == top_p, EB_ERR_ARG, "eb_engine_seq_sampling: top_p is NaN");
  e->samp_scale[(size_t)slot] = temperature > 0.f ? 1.4426950408889634f / temperature : 0.f;
  const float p = top_p < 0.f ? 0.f : top_p > 1.f ? 1.f : top_p;
  e->samp_q24[(size_t)slot] = (uint32_t)((double)p * 16777216.0);
  e->samp_seed[(size_t)slot] = seed;
  return EB_OK;
}

int32_t eb_engine_seq_release(eb_engine* e, int32_t slot) {
  EB_REQUIRE(e, EB_ERR_ARG, "eb_engine_seq_release: null");
  EB_REQUIRE(!e->in_flight, EB_ERR_STATE, "eb_engine_seq_release: a step is in flight");
  EB_TRY(eb_sched_release(e->sched, slot));
  e->uploaded_pages[(size_t)slot] = 0;
  return EB_OK;
}

int32_t eb_engine_seq_truncate(eb_engine* e, int32_t slot, int32_t new_len) {
  EB_REQUIRE(e, EB_ERR_ARG, "eb_engine_seq_truncate: null");
  EB_REQUIRE(!e->in_flight, EB_ERR_STATE, "eb_engine_seq_truncate: a step is in flight");
  if (e->ring && slot >= 0 && slot < e->c.max_seqs && new_len >= 0) {
    // Sliding-window layers keep a ring of pages: logical page p shares its ring page with p + ring.  The window before
    // the cut is still there only while no page written later has taken the place of its first page.
    const int32_t P = e->c.page_size, high = e->high_len[(size_t)slot];
    const int32_t first_needed = std::max(0, new_len - e->c.window - 1) / P, last_written = std::max(0, high - 1) / P;
    EB_REQUIRE(first_needed + e->ring > last_written, EB_ERR_UNSUPPORTED,
               "eb_engine_seq_truncate: the page rings of slot %d were written up to token %d and no longer hold the window before %d",
               slot, high, new_len);
  }
  EB_TRY(eb_sched_truncate(e->sched, slot, new_len));
  const int32_t pages = (new_len + e->c.page_size - 1) / e->c.page_size;
  e->uploaded_pages[(size_t)slot] = std::min(e->uploaded_pages[(size_t)slot], pages);
  return EB_OK;
}

int32_t eb_engine_seq_truncate_many(eb_engine* e, const int32_t* h_slots, const int32_t* h_new_lens, int32_t n) {
  EB_REQUIRE(e && h_slots && h_new_lens && n >= 0, EB_ERR_ARG, "eb_engine_seq_truncate_many: bad argument");
  for (int i = 0; i < n; ++i) EB_TRY(eb_engine_seq_truncate(e, h_slots[i], h_new_lens[i]));
  return EB_OK;
}

int32_t eb_engine_seq_len(const eb_engine* e, int32_t slot, int32_t* len) {
  EB_REQUIRE(e, EB_ERR_ARG, "eb_engine_seq_len: null");
  return eb_sched_seq_len(e->sched, slot, len);
}

int32_t eb_engine_sched(eb_engine* e, eb_sched** sched) {
  EB_REQUIRE(e && sched, EB_ERR_ARG, "eb_engine_sched: null");
  *sched = e->sched;
  return EB_OK;
}

int32_t eb_engine_step_launch(eb_engine* e, const int32_t* h_slots, const int32_t* h_q_lens, int32_t n_seqs,
                              const int32_t* h_tokens) {
  EB_REQUIRE(e && h_slots && h_q_lens && h_tokens, EB_ERR_ARG, "eb_engine_step: null pointer");
  EB_REQUIRE(!e->in_flight, EB_ERR_STATE, "eb_engine_step: the previous step has not been waited for");
  const eb_config& c = e->c;
  EB_REQUIRE(n_seqs >= 1 && n_seqs <= c.max_seqs, EB_ERR_ARG, "eb_engine_step: n_seqs %d outside 1..%d", n_seqs, c.max_seqs);
  int64_t T64 = 0;
  int max_q = 1;
  for (int i = 0; i < n_seqs; ++i) {
    EB_REQUIRE(h_q_lens[i] >= 1 && h_q_lens[i] <= e->chunk_cap, EB_ERR_ARG, "eb_engine_step: q_len %d of sequence %d outside 1..%d",
               h_q_lens[i], i, e->chunk_cap);
    for (int j = 0; j < i; ++j)
      EB_REQUIRE(h_slots[j] != h_slots[i], EB_ERR_ARG, "eb_engine_step: slot %d appears twice", h_slots[i]);
    T64 += h_q_lens[i];
    max_q = std::max(max_q, std::min(h_q_lens[i], c.max_q_len));  // longer runs are cut into attention entries of max_q_len
  }
  EB_REQUIRE(T64 <= c.max_tokens, EB_ERR_ARG, "eb_engine_step: %lld token rows exceed max_tokens %d", (long long)T64, c.max_tokens);
  const int T = (int)T64;
  for (int t = 0; t < T; ++t)
    EB_REQUIRE(h_tokens[t] >= 0 && h_tokens[t] < c.vocab, EB_ERR_ARG, "eb_engine_step: token id %d of row %d outside the vocabulary",
               h_tokens[t], t);

  // grow every sequence; on ANY failure before the step is in flight undo the growth (lengths, pages and the record
  // of which block-table entries the device holds), so a refused step leaves no trace
  std::vector<int32_t> old_len((size_t)n_seqs), old_uploaded((size_t)n_seqs);
  int grown = 0;
  auto rollback = [&](int32_t rc) -> int32_t {
    for (int j = 0; j < grown; ++j) {
      eb_sched_truncate(e->sched, h_slots[j], old_len[(size_t)j]);
      e->uploaded_pages[(size_t)h_slots[j]] = old_uploaded[(size_t)j];
    }
    return rc;
  };
  for (int i = 0; i < n_seqs; ++i) {
    int32_t rc = eb_sched_seq_len(e->sched, h_slots[i], &old_len[(size_t)i]);
    if (rc == EB_OK) {
      old_uploaded[(size_t)i] = e->uploaded_pages[(size_t)h_slots[i]];
      rc = eb_sched_extend(e->sched, h_slots[i], old_len[(size_t)i] + h_q_lens[i]);
    }
    if (rc != EB_OK) return rollback(rc);
    grown = i + 1;
  }
  for (int i = 0; i < n_seqs; ++i)  // (kept when the step is refused below: only ever too cautious)
    e->high_len[(size_t)h_slots[i]] = std::max(e->high_len[(size_t)h_slots[i]], old_len[(size_t)i] + h_q_lens[i]);
  static const bool nvtx_step = [] {
    const char* v = getenv("EIDOLA_B200_NVTX");
    return v && v[0] == '1';
  }();
  if (nvtx_step) nvtxRangePushA("eb_engine_step_launch");
  const int32_t rc_body = step_launch_body(e, h_slots, h_q_lens, n_seqs, h_tokens, T, max_q);
  if (nvtx_step) nvtxRangePop();
  if (rc_body != EB_OK) return rollback(rc_body);
  ++e->tick;
  for (int i = 0; i < n_seqs; ++i) eb_sched_touch(e->sched, h_slots[i], e->tick);
  e->cur_T = T;
  e->in_flight = true;
  return EB_OK;
}

}  // extern "C"

namespace {

// Everything of a step after the sequences have grown: staging block, copies, kernels.  Any non-zero return leaves
// nothing in flight; the caller undoes the growth.
int32_t step_launch_body(eb_engine* e, const int32_t* h_slots, const int32_t* h_q_lens, int32_t n_seqs,
                         const int32_t* h_tokens, int T, int max_q) {
  const eb_config& c = e->c;
  // ---- one staging block
  int32_t* hs = e->h_stage;
  size_t off = 0;
  auto take = [&](size_t n) {
    int32_t* p = hs + off;
    off += n;
    return p;
  };
  int32_t* s_tokens = take((size_t)T);
  int32_t* s_tok_slot = take((size_t)T);
  int32_t* s_pos = take((size_t)T);
  bool sampling = false;
  for (int i = 0; i < n_seqs; ++i) sampling = sampling || e->samp_scale[(size_t)h_slots[i]] > 0.f;
  int32_t* s_samp = sampling ? take(3 * (size_t)T) : nullptr;
  memcpy(s_tokens, h_tokens, (size_t)T * sizeof(int32_t));
  std::vector<int32_t> tok_seq((size_t)T), seq_ctx((size_t)n_seqs), seq_qoff((size_t)n_seqs + 1);
  int32_t nt = 0;
  EB_TRY(eb_sched_pack(e->sched, h_slots, h_q_lens, n_seqs, seq_qoff.data(), seq_ctx.data(), tok_seq.data(), s_tok_slot, s_pos, &nt));
  // the sampler's per-row arguments, when a sequence of the step is not greedy: the random number of a row is a function
  // of the sequence's seed and the absolute position of the token drawn, whatever else shares the step
  if (sampling) {
    for (int t = 0; t < T; ++t) {
      const size_t slot = (size_t)s_tok_slot[t];
      memcpy(&s_samp[t], &e->samp_scale[slot], sizeof(float));
      s_samp[(size_t)T + t] = (int32_t)e->samp_q24[slot];
      s_samp[2 * (size_t)T + t] = (int32_t)eb_sample_rand32(e->samp_seed[slot], (uint64_t)s_pos[t] + 1);
    }
  }
  e->d_samp = sampling ? e->d_stage + (s_samp - hs) : nullptr;
  // Attention entries: a sequence's new tokens in runs of at most max_q_len.  Decode and verify steps have one entry per
  // sequence; a prefill chunk has several on the same block-table row, entry j seeing the context up to its own last
  // token (every K and V of the step is in the cache before any attention kernel of a layer runs).
  int n_ent = 0;
  for (int i = 0; i < n_seqs; ++i) n_ent += (h_q_lens[i] + c.max_q_len - 1) / c.max_q_len;
  EB_REQUIRE(n_ent <= e->cap_ent, EB_ERR_NOMEM, "eb_engine_step: %d attention entries exceed the %d planned for", n_ent, e->cap_ent);
  int32_t* s_slots = take((size_t)n_ent);
  int32_t* s_ctx = take((size_t)n_ent);
  int32_t* s_qoff = take((size_t)n_ent + 1);
  std::vector<int32_t> ent_q((size_t)n_ent);
  {
    int k = 0;
    for (int i = 0; i < n_seqs; ++i)
      for (int b = 0; b < h_q_lens[i]; b += c.max_q_len, ++k) {
        const int len = std::min(c.max_q_len, h_q_lens[i] - b);
        s_slots[k] = h_slots[i];
        s_qoff[k] = seq_qoff[(size_t)i] + b;
        s_ctx[k] = seq_ctx[(size_t)i] - h_q_lens[i] + b + len;
        ent_q[(size_t)k] = len;
      }
    s_qoff[n_ent] = T;
  }
  // block-table patches
  const int32_t* tables = nullptr;
  int32_t stride = 0;
  EB_TRY(eb_sched_block_tables(e->sched, &tables, &stride));
  int32_t* s_patch = hs + off;
  int n_patch = 0;
  for (int i = 0; i < n_seqs; ++i) {
    const int slot = h_slots[i];
    const int pages = (seq_ctx[(size_t)i] + c.page_size - 1) / c.page_size;
    for (int p = e->uploaded_pages[(size_t)slot]; p < pages; ++p) {
      s_patch[3 * n_patch] = slot;
      s_patch[3 * n_patch + 1] = p;
      s_patch[3 * n_patch + 2] = tables[(size_t)slot * stride + p];
      ++n_patch;
    }
    e->uploaded_pages[(size_t)slot] = pages;
  }
  off += 3 * (size_t)n_patch;
  // attention plans: [0] full, [1] windowed
  Plan plans[2];
  size_t items_off[2], part_off[2];
  const int ppi = 8 / e->hkv_l;
  for (int k = 0; k < 2; ++k) {
    if (k == 1 && c.window == 0) {
      items_off[1] = items_off[0];
      part_off[1] = part_off[0];
      plans[1] = plans[0];
      break;
    }
    items_off[k] = off;
    eb_attn_item* it = reinterpret_cast<eb_attn_item*>(hs + off);
    off += 4 * (size_t)e->cap_items;
    part_off[k] = off;
    int32_t* sp = take((size_t)n_ent + 1);
    // the chunk size follows the kernel the attention entry point picks for this step's shapes
    const int32_t plan_sms = eb_attn_plan_sm_count(e->sm_count, max_q, e->hq_l, e->hkv_l, k ? c.window : 0);
    EB_TRY(eb_attn_plan(s_ctx, ent_q.data(), n_ent, c.page_size, k ? c.window : 0, plan_sms, 0, ppi, it, e->cap_items,
                        &plans[k].n_items, sp, &plans[k].n_parts));
  }
  EB_REQUIRE(off <= e->stage_words, EB_ERR_NOMEM, "eb_engine_step: staging block overflow (%zu > %zu words)", off, e->stage_words);

  EB_CUDA(cudaEventRecord(e->ev0, e->stream));
  EB_CUDA(cudaMemcpyAsync(e->d_stage, hs, off * sizeof(int32_t), cudaMemcpyHostToDevice, e->stream));
  const int32_t* ds = e->d_stage;
  if (n_patch > 0) {
    EB_CUDA(eb::launch(bt_patch_kernel, dim3((unsigned)eb::cdiv(n_patch, 256)), dim3(256), 0, e->stream, e->d_bt, c.max_pages_per_seq,
                                                                            ds + (s_patch - hs), n_patch));
    EB_LAUNCH_CHECK();
  }
  const eb_attn_item* d_items[2] = {reinterpret_cast<const eb_attn_item*>(ds + items_off[0]),
                                    reinterpret_cast<const eb_attn_item*>(ds + items_off[1])};
  const int32_t* d_seq_part[2] = {ds + part_off[0], ds + part_off[1]};
  int32_t rc = run_layers(e, T, n_ent, ds + (s_tokens - hs), ds + (s_tok_slot - hs), ds + (s_pos - hs), ds + (s_slots - hs),
                          ds + (s_qoff - hs), ds + (s_ctx - hs), d_items, d_seq_part, plans, max_q);
  if (rc != EB_OK) return rc;
  e->launches += (n_patch > 0 ? 1 : 0);
  EB_CUDA(cudaMemcpyAsync(e->h_result, e->d_next, (size_t)T * sizeof(int32_t), cudaMemcpyDeviceToHost, e->stream));
  EB_CUDA(cudaMemcpyAsync(e->h_result + T, e->d_margin, (size_t)T * sizeof(float), cudaMemcpyDeviceToHost, e->stream));
  EB_CUDA(cudaEventRecord(e->ev1, e->stream));
  e->h2d_bytes = (int64_t)(off * sizeof(int32_t));
  e->d2h_bytes = (int64_t)T * (int64_t)(sizeof(int32_t) + sizeof(float));
  return EB_OK;
}

}  // namespace

extern "C" {

int32_t eb_engine_step_wait(eb_engine* e, int32_t* h_next, float* h_margin) {
  EB_REQUIRE(e && h_next, EB_ERR_ARG, "eb_engine_step_wait: null pointer");
  EB_REQUIRE(e->in_flight, EB_ERR_STATE, "eb_engine_step_wait: no step in flight");
  e->in_flight = false;
  EB_CUDA(cudaEventSynchronize(e->ev1));
  EB_CUDA(cudaEventElapsedTime(&e->last_ms, e->ev0, e->ev1));
  for (float& v : e->prof_ms) v = 0.f;
  for (size_t i = 0; i + 1 < e->prof_cat.size(); i += 2) {
    float ms = 0.f;
    if (e->prof_cat[i] >= 0 && cudaEventElapsedTime(&ms, e->prof_ev[i], e->prof_ev[i + 1]) == cudaSuccess)
      e->prof_ms[e->prof_cat[i]] += ms;
  }
  memcpy(h_next, e->h_result, (size_t)e->cur_T * sizeof(int32_t));
  if (h_margin) memcpy(h_margin, e->h_result + e->cur_T, (size_t)e->cur_T * sizeof(float));
  return EB_OK;
}

int32_t eb_engine_step(eb_engine* e, const int32_t* h_slots, const int32_t* h_q_lens, int32_t n_seqs,
                       const int32_t* h_tokens, int32_t* h_next, float* h_margin) {
  EB_TRY(eb_engine_step_launch(e, h_slots, h_q_lens, n_seqs, h_tokens));
  return eb_engine_step_wait(e, h_next, h_margin);
}

int32_t eb_engine_prefill(eb_engine* e, const int32_t* h_slots, const int32_t* h_n_tokens, int32_t n_seqs, const int32_t* h_tokens,
                          int32_t* h_next, float* h_margin, int32_t* steps_run, float* device_ms) {
  EB_REQUIRE(e && h_slots && h_n_tokens && h_tokens && h_next, EB_ERR_ARG, "eb_engine_prefill: null pointer");
  const eb_config& c = e->c;
  EB_REQUIRE(n_seqs >= 1 && n_seqs <= c.max_seqs, EB_ERR_ARG, "eb_engine_prefill: n_seqs %d outside 1..%d", n_seqs, c.max_seqs);
  std::vector<int64_t> off((size_t)n_seqs + 1, 0);
  for (int i = 0; i < n_seqs; ++i) {
    EB_REQUIRE(h_n_tokens[i] >= 1, EB_ERR_ARG, "eb_engine_prefill: sequence %d has %d prompt tokens", i, h_n_tokens[i]);
    off[(size_t)i + 1] = off[(size_t)i] + h_n_tokens[i];
  }
  std::vector<int32_t> done((size_t)n_seqs, 0), b_slots, b_q, b_tok, b_seq;
  std::vector<int32_t> next((size_t)c.max_tokens);
  std::vector<float> margin((size_t)c.max_tokens);
  int32_t steps = 0;
  float ms = 0.f;
  int64_t left = off[(size_t)n_seqs];
  int start = 0;  // rotate the first sequence considered, so that a batch too wide for max_tokens starves nobody
  while (left > 0) {
    b_slots.clear();
    b_q.clear();
    b_tok.clear();
    b_seq.clear();
    int32_t rows = 0;
    bool skipped = false;
    for (int k = 0; k < n_seqs; ++k) {
      const int i = (start + k) % n_seqs;
      const int32_t rem = h_n_tokens[i] - done[(size_t)i];
      if (rem <= 0) continue;
      const int32_t q = std::min(std::min(rem, e->chunk_cap), c.max_tokens - rows);  // what is left of the step, if short
      if (q < rem && q < std::min(rem, c.max_q_len)) {  // less room than one attention entry: the next step
        skipped = true;
        continue;
      }
      b_slots.push_back(h_slots[i]);
      b_q.push_back(q);
      b_seq.push_back(i);
      for (int32_t j = 0; j < q; ++j) b_tok.push_back(h_tokens[off[(size_t)i] + done[(size_t)i] + j]);
      rows += q;
    }
    EB_REQUIRE(rows > 0, EB_ERR_STATE, "eb_engine_prefill: no sequence fits a step of %d token rows", c.max_tokens);
    // only the row after a prompt's last token is read below: the LM head skips the 128-row blocks that hold none
    e->head_rows.clear();
    {
      int32_t row = 0;
      for (size_t k = 0; k < b_seq.size(); ++k) {
        row += b_q[k];
        if (done[(size_t)b_seq[k]] + b_q[k] == h_n_tokens[b_seq[k]]) e->head_rows.push_back(row - 1);
      }
    }
    e->head_rows_on = true;
    const int32_t rc_step = eb_engine_step(e, b_slots.data(), b_q.data(), (int32_t)b_slots.size(), b_tok.data(), next.data(), margin.data());
    e->head_rows_on = false;
    if (rc_step != EB_OK) return rc_step;
    ms += e->last_ms;
    ++steps;
    int32_t row = 0;
    for (size_t k = 0; k < b_seq.size(); ++k) {
      const int i = b_seq[k];
      row += b_q[k];
      done[(size_t)i] += b_q[k];
      left -= b_q[k];
      if (done[(size_t)i] == h_n_tokens[i]) {  // the row of the prompt's last token predicts the first generated token
        h_next[i] = next[(size_t)row - 1];
        if (h_margin) h_margin[i] = margin[(size_t)row - 1];
      }
    }
    if (skipped) start = (start + 1) % n_seqs;  // only a batch too wide for one step changes the order of the sequences
  }
  if (steps_run) *steps_run = steps;
  if (device_ms) *device_ms = ms;
  return EB_OK;
}

int32_t eb_engine_chunk_tokens(const eb_engine* e, int32_t* tokens) {
  EB_REQUIRE(e && tokens, EB_ERR_ARG, "eb_engine_chunk_tokens: null");
  *tokens = e->chunk_cap;
  return EB_OK;
}

int32_t eb_engine_last_step_stats(const eb_engine* e, float* device_ms, int32_t* kernel_launches) {
  EB_REQUIRE(e, EB_ERR_ARG, "eb_engine_last_step_stats: null engine");
  if (device_ms) *device_ms = e->last_ms;
  if (kernel_launches) *kernel_launches = e->launches;
  return EB_OK;
}

int32_t eb_engine_last_step_copies(const eb_engine* e, int64_t* h2d_bytes, int64_t* d2h_bytes) {
  EB_REQUIRE(e, EB_ERR_ARG, "eb_engine_last_step_copies: null engine");
  if (h2d_bytes) *h2d_bytes = e->h2d_bytes;
  if (d2h_bytes) *d2h_bytes = e->d2h_bytes;
  return EB_OK;
}

int32_t eb_engine_profile(eb_engine* e, int32_t on) {
  EB_REQUIRE(e, EB_ERR_ARG, "eb_engine_profile: null engine");
  EB_REQUIRE(!e->in_flight, EB_ERR_STATE, "eb_engine_profile: a step is in flight");
  e->c.debug = on ? (e->c.debug | 2) : (e->c.debug & ~2);
  return EB_OK;
}

int32_t eb_engine_last_step_breakdown(const eb_engine* e, float* ms8) {
  EB_REQUIRE(e && ms8, EB_ERR_ARG, "eb_engine_last_step_breakdown: null");
  EB_REQUIRE(e->c.debug & 2, EB_ERR_STATE, "eb_engine_last_step_breakdown: engine was not created with debug & 2");
  for (int i = 0; i < 8; ++i) ms8[i] = e->prof_ms[i];
  return EB_OK;
}

int32_t eb_engine_stream(eb_engine* e, void** stream) {
  EB_REQUIRE(e && stream, EB_ERR_ARG, "eb_engine_stream: null");
  *stream = e->stream;
  return EB_OK;
}

int32_t eb_engine_read_logits(eb_engine* e, void* h_logits, int64_t bytes) {
  EB_REQUIRE(e && h_logits, EB_ERR_ARG, "eb_engine_read_logits: null");
  EB_REQUIRE(!e->in_flight, EB_ERR_STATE, "eb_engine_read_logits: a step is in flight");
  EB_REQUIRE(bytes == (int64_t)e->cur_T * e->c.vocab * 2, EB_ERR_ARG, "eb_engine_read_logits: expected %lld bytes",
             (long long)e->cur_T * e->c.vocab * 2);
  EB_CUDA(cudaMemcpy(h_logits, e->logits, (size_t)bytes, cudaMemcpyDeviceToHost));
  return EB_OK;
}

int32_t eb_engine_read_routing(eb_engine* e, int32_t layer, int32_t* h_idx, int64_t bytes) {
  EB_REQUIRE(e && h_idx, EB_ERR_ARG, "eb_engine_read_routing: null");
  EB_REQUIRE(e->c.debug && e->dbg_route, EB_ERR_STATE, "eb_engine_read_routing: engine was not created with debug = 1");
  EB_REQUIRE(layer >= 0 && layer < e->c.n_layers, EB_ERR_ARG, "eb_engine_read_routing: layer %d", layer);
  EB_REQUIRE(bytes == (int64_t)e->cur_T * e->c.top_k * 4, EB_ERR_ARG, "eb_engine_read_routing: expected %lld bytes",
             (long long)e->cur_T * e->c.top_k * 4);
  EB_CUDA(cudaMemcpy(h_idx, e->dbg_route + (size_t)layer * e->c.max_tokens * e->c.top_k, (size_t)bytes, cudaMemcpyDeviceToHost));
  return EB_OK;
}

int32_t eb_engine_read_hidden(eb_engine* e, int32_t layer, void* h_x, int64_t bytes) {
  EB_REQUIRE(e && h_x, EB_ERR_ARG, "eb_engine_read_hidden: null");
  EB_REQUIRE(e->c.debug && e->dbg_hidden, EB_ERR_STATE, "eb_engine_read_hidden: engine was not created with debug = 1");
  EB_REQUIRE(layer >= -1 && layer < e->c.n_layers, EB_ERR_ARG, "eb_engine_read_hidden: layer %d", layer);
  EB_REQUIRE(bytes == (int64_t)e->cur_T * e->c.hidden * 2, EB_ERR_ARG, "eb_engine_read_hidden: expected %lld bytes",
             (long long)e->cur_T * e->c.hidden * 2);
  EB_CUDA(cudaMemcpy(h_x, e->dbg_hidden + (size_t)(layer + 1) * e->c.max_tokens * e->c.hidden, (size_t)bytes, cudaMemcpyDeviceToHost));
  return EB_OK;
}


int32_t eb_engine_debug_read_last(eb_engine* e, int32_t which, void* h_out, int64_t bytes) {
  EB_REQUIRE(e && h_out, EB_ERR_ARG, "eb_engine_debug_read_last: null");
  EB_REQUIRE(e->c.debug & 1, EB_ERR_STATE, "eb_engine_debug_read_last: engine was not created with debug = 1");
  EB_REQUIRE(!e->in_flight, EB_ERR_STATE, "eb_engine_debug_read_last: a step is in flight");
  EB_REQUIRE(which == 0 || which == 1, EB_ERR_ARG, "eb_engine_debug_read_last: which %d (0 = q rows, 1 = attention output)", which);
  const void* src = which == 0 ? (const void*)e->qkv : (const void*)e->attn;
  const int64_t width = which == 0 ? e->nqkv : e->hqd;
  EB_REQUIRE(bytes == (int64_t)e->cur_T * width * 2, EB_ERR_ARG, "eb_engine_debug_read_last: expected %lld bytes",
             (long long)e->cur_T * width * 2);
  EB_CUDA(cudaMemcpy(h_out, src, (size_t)bytes, cudaMemcpyDeviceToHost));
  return EB_OK;
}

int32_t eb_engine_debug_force_hidden(eb_engine* e, int32_t layer, const void* h_x, int32_t rows) {
  EB_REQUIRE(e, EB_ERR_ARG, "eb_engine_debug_force_hidden: null engine");
  EB_REQUIRE(e->c.debug && e->dbg_force, EB_ERR_STATE, "eb_engine_debug_force_hidden: engine was not created with debug = 1");
  EB_REQUIRE(!e->in_flight, EB_ERR_STATE, "eb_engine_debug_force_hidden: a step is in flight");
  EB_REQUIRE(layer >= 0 && layer <= e->c.n_layers, EB_ERR_ARG, "eb_engine_debug_force_hidden: layer %d", layer);
  EB_REQUIRE(rows >= 0 && rows <= e->c.max_tokens, EB_ERR_ARG, "eb_engine_debug_force_hidden: rows %d", rows);
  if (!h_x || rows == 0) {
    e->force_rows[(size_t)layer] = 0;
    return EB_OK;
  }
  EB_CUDA(cudaMemcpy(e->dbg_force + (size_t)layer * e->c.max_tokens * e->c.hidden, h_x, (size_t)rows * e->c.hidden * 2,
                     cudaMemcpyHostToDevice));
  e->force_rows[(size_t)layer] = rows;
  return EB_OK;
}

}  // extern "C"

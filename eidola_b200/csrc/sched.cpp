// Continuous-batching scheduler of libeidola_b200: page pool, block tables, ragged packing and the
// split-K attention plan.  Host only -- nothing here calls CUDA, so it runs on a machine without a GPU.
//
// Nearest reference analogue: the admission planner for whole engines,
// crates/eidola-app-core/src/local_models.rs:441-485 (`reserve_engine`: plan and reserve in one critical
// section) and :653-701 (`plan_evictions`: refuse without side effects when the budget cannot hold the
// request).  The same two properties hold here at page granularity.
#include <algorithm>
#include <new>
#include <vector>

#include "../../include/eb_synth.h"
#include "common.h"

struct eb_sched {
  int32_t num_pages, page_size, max_seqs, max_pages;
  std::vector<int32_t> free_list;  // allocation pops from the back
  std::vector<int32_t> tables;     // [max_seqs][max_pages]
  std::vector<int32_t> len;        // tokens held, -1 = slot free
  // admission with eviction (the reference's engine pool, one level down): when a sequence was last used, whether
  // its owner pinned it, whether a step that includes it is in flight
  std::vector<int64_t> last_used;
  std::vector<uint8_t> pinned, in_flight;
};

namespace {
inline int32_t pages_for(const eb_sched* s, int32_t len) { return (len + s->page_size - 1) / s->page_size; }
inline bool live(const eb_sched* s, int32_t slot) { return slot >= 0 && slot < s->max_seqs && s->len[slot] >= 0; }
}  // namespace

extern "C" {

int32_t eb_sched_create(int32_t num_pages, int32_t page_size, int32_t max_seqs, int32_t max_pages_per_seq,
                        uint64_t seed, eb_sched** out) {
  EB_REQUIRE(out, EB_ERR_ARG, "eb_sched_create: null out");
  EB_REQUIRE(num_pages > 0 && page_size > 0 && max_seqs > 0 && max_pages_per_seq > 0, EB_ERR_ARG,
             "eb_sched_create: non-positive size (pages %d, page_size %d, seqs %d, pages/seq %d)", num_pages,
             page_size, max_seqs, max_pages_per_seq);
  eb_sched* s = new (std::nothrow) eb_sched;
  EB_REQUIRE(s, EB_ERR_NOMEM, "eb_sched_create: host allocation failed");
  s->num_pages = num_pages;
  s->page_size = page_size;
  s->max_seqs = max_seqs;
  s->max_pages = max_pages_per_seq;
  s->free_list.resize((size_t)num_pages);
  for (int32_t i = 0; i < num_pages; ++i) s->free_list[(size_t)i] = i;
  // Seeded Fisher-Yates: page ids are handed out in shuffled order so that no kernel can rely on
  // physically consecutive pages.
  for (int32_t i = num_pages - 1; i >= 1; --i) {
    const uint64_t j = eb_hash(seed, 0x5EEDull, (uint64_t)i) % (uint64_t)(i + 1);
    std::swap(s->free_list[(size_t)i], s->free_list[(size_t)j]);
  }
  s->tables.assign((size_t)max_seqs * max_pages_per_seq, -1);
  s->len.assign((size_t)max_seqs, -1);
  s->last_used.assign((size_t)max_seqs, 0);
  s->pinned.assign((size_t)max_seqs, 0);
  s->in_flight.assign((size_t)max_seqs, 0);
  *out = s;
  return EB_OK;
}

int32_t eb_sched_destroy(eb_sched* s) {
  delete s;
  return EB_OK;
}

int32_t eb_sched_admit(eb_sched* s, int32_t context_len, int32_t* slot) {
  EB_REQUIRE(s && slot, EB_ERR_ARG, "eb_sched_admit: null");
  EB_REQUIRE(context_len >= 0, EB_ERR_ARG, "eb_sched_admit: negative length %d", context_len);
  const int32_t need = pages_for(s, context_len);
  EB_REQUIRE(need <= s->max_pages, EB_ERR_NOMEM, "eb_sched_admit: %d tokens need %d pages, a sequence may hold %d",
             context_len, need, s->max_pages);
  EB_REQUIRE(need <= (int32_t)s->free_list.size(), EB_ERR_NOMEM, "eb_sched_admit: need %d pages, %d free", need,
             (int32_t)s->free_list.size());
  int32_t found = -1;
  for (int32_t i = 0; i < s->max_seqs; ++i)
    if (s->len[(size_t)i] < 0) {
      found = i;
      break;
    }
  EB_REQUIRE(found >= 0, EB_ERR_NOMEM, "eb_sched_admit: all %d sequence slots in use", s->max_seqs);
  for (int32_t p = 0; p < need; ++p) {
    s->tables[(size_t)found * s->max_pages + p] = s->free_list.back();
    s->free_list.pop_back();
  }
  s->len[(size_t)found] = context_len;
  s->pinned[(size_t)found] = s->in_flight[(size_t)found] = 0;
  s->last_used[(size_t)found] = 0;
  *slot = found;
  return EB_OK;
}

int32_t eb_sched_extend(eb_sched* s, int32_t slot, int32_t new_len) {
  EB_REQUIRE(s, EB_ERR_ARG, "eb_sched_extend: null");
  EB_REQUIRE(live(s, slot), EB_ERR_STATE, "eb_sched_extend: slot %d is not live", slot);
  const int32_t cur = s->len[(size_t)slot];
  EB_REQUIRE(new_len >= cur, EB_ERR_ARG, "eb_sched_extend: slot %d holds %d tokens, asked for %d", slot, cur, new_len);
  const int32_t have = pages_for(s, cur), need = pages_for(s, new_len);
  EB_REQUIRE(need <= s->max_pages, EB_ERR_NOMEM, "eb_sched_extend: %d tokens need %d pages, a sequence may hold %d",
             new_len, need, s->max_pages);
  EB_REQUIRE(need - have <= (int32_t)s->free_list.size(), EB_ERR_NOMEM, "eb_sched_extend: need %d more pages, %d free",
             need - have, (int32_t)s->free_list.size());
  for (int32_t p = have; p < need; ++p) {
    s->tables[(size_t)slot * s->max_pages + p] = s->free_list.back();
    s->free_list.pop_back();
  }
  s->len[(size_t)slot] = new_len;
  return EB_OK;
}

int32_t eb_sched_truncate(eb_sched* s, int32_t slot, int32_t new_len) {
  EB_REQUIRE(s, EB_ERR_ARG, "eb_sched_truncate: null");
  EB_REQUIRE(live(s, slot), EB_ERR_STATE, "eb_sched_truncate: slot %d is not live", slot);
  const int32_t cur = s->len[(size_t)slot];
  EB_REQUIRE(new_len >= 0 && new_len <= cur, EB_ERR_ARG, "eb_sched_truncate: slot %d holds %d tokens, asked for %d",
             slot, cur, new_len);
  const int32_t have = pages_for(s, cur), need = pages_for(s, new_len);
  for (int32_t p = have - 1; p >= need; --p) {
    int32_t& e = s->tables[(size_t)slot * s->max_pages + p];
    s->free_list.push_back(e);
    e = -1;
  }
  s->len[(size_t)slot] = new_len;
  return EB_OK;
}

int32_t eb_sched_release(eb_sched* s, int32_t slot) {
  EB_REQUIRE(s, EB_ERR_ARG, "eb_sched_release: null");
  EB_REQUIRE(live(s, slot), EB_ERR_STATE, "eb_sched_release: slot %d is not live", slot);
  int32_t rc = eb_sched_truncate(s, slot, 0);
  if (rc != EB_OK) return rc;
  s->len[(size_t)slot] = -1;
  return EB_OK;
}

int32_t eb_sched_touch(eb_sched* s, int32_t slot, int64_t now) {
  EB_REQUIRE(s, EB_ERR_ARG, "eb_sched_touch: null");
  EB_REQUIRE(live(s, slot), EB_ERR_STATE, "eb_sched_touch: slot %d is not live", slot);
  s->last_used[(size_t)slot] = now;
  return EB_OK;
}

int32_t eb_sched_set_flags(eb_sched* s, int32_t slot, int32_t pinned, int32_t in_flight) {
  EB_REQUIRE(s, EB_ERR_ARG, "eb_sched_set_flags: null");
  EB_REQUIRE(live(s, slot), EB_ERR_STATE, "eb_sched_set_flags: slot %d is not live", slot);
  if (pinned >= 0) s->pinned[(size_t)slot] = pinned ? 1 : 0;
  if (in_flight >= 0) s->in_flight[(size_t)slot] = in_flight ? 1 : 0;
  return EB_OK;
}

// The reference's plan_evictions (crates/eidola-app-core/src/local_models.rs:653-701) with pages for bytes and sequences
// for engines: nothing to do when the request fits; otherwise least recently used first, but only sequences that are
// neither pinned nor part of a step in flight, and only as many as needed; when even that cannot make room, refuse and
// change nothing (message: what is holding the pages).
int32_t eb_sched_plan_evictions(const eb_sched* s, int32_t context_len, int32_t* evict_slots, int32_t cap, int32_t* n_evict) {
  EB_REQUIRE(s && n_evict && (evict_slots || cap == 0) && cap >= 0, EB_ERR_ARG, "eb_sched_plan_evictions: bad argument");
  EB_REQUIRE(context_len >= 0, EB_ERR_ARG, "eb_sched_plan_evictions: negative length %d", context_len);
  *n_evict = 0;
  const int32_t required = pages_for(s, context_len);
  EB_REQUIRE(required <= s->max_pages && required <= s->num_pages, EB_ERR_NOMEM,
             "eb_sched_plan_evictions: the sequence needs %d pages but the budget is %d (a sequence may hold %d)", required,
             s->num_pages, s->max_pages);
  int64_t free_pages = (int64_t)s->free_list.size();
  bool slot_free = false;
  for (int32_t i = 0; i < s->max_seqs; ++i) slot_free |= s->len[(size_t)i] < 0;
  if (free_pages >= required && slot_free) return EB_OK;
  std::vector<int32_t> cand;
  int64_t held = 0;
  for (int32_t i = 0; i < s->max_seqs; ++i) {
    if (s->len[(size_t)i] < 0) continue;
    if (s->pinned[(size_t)i] || s->in_flight[(size_t)i])
      held += pages_for(s, s->len[(size_t)i]);
    else
      cand.push_back(i);
  }
  std::stable_sort(cand.begin(), cand.end(), [&](int32_t a, int32_t b) { return s->last_used[(size_t)a] < s->last_used[(size_t)b]; });
  int32_t n = 0;
  for (int32_t slot : cand) {
    if (free_pages >= required && (slot_free || n > 0)) break;
    free_pages += pages_for(s, s->len[(size_t)slot]);
    if (n < cap) evict_slots[n] = slot;
    ++n;
  }
  if (!(free_pages >= required && (slot_free || n > 0)))
    return eb::fail(EB_ERR_NOMEM, "eb_sched_plan_evictions: the sequence needs %d pages, but %lld pages are held by pinned or in-use "
                    "sequences", required, (long long)held);
  EB_REQUIRE(n <= cap, EB_ERR_ARG, "eb_sched_plan_evictions: %d evictions needed, room for %d", n, cap);
  *n_evict = n;
  return EB_OK;
}

// Plan and reserve in one call (the reference does both inside one critical section, local_models.rs:441-485): the
// victims are released and the new sequence admitted, or nothing changes.
int32_t eb_sched_admit_evicting(eb_sched* s, int32_t context_len, int64_t now, int32_t* slot, int32_t* evict_slots, int32_t cap,
                                int32_t* n_evict) {
  EB_REQUIRE(s && slot && n_evict, EB_ERR_ARG, "eb_sched_admit_evicting: null");
  int32_t rc = eb_sched_plan_evictions(s, context_len, evict_slots, cap, n_evict);
  if (rc != EB_OK) return rc;
  for (int32_t i = 0; i < *n_evict; ++i) {
    rc = eb_sched_release(s, evict_slots[i]);
    if (rc != EB_OK) return rc;
  }
  rc = eb_sched_admit(s, context_len, slot);
  if (rc == EB_OK) s->last_used[(size_t)*slot] = now;
  return rc;
}

int32_t eb_sched_free_pages(const eb_sched* s, int32_t* n) {
  EB_REQUIRE(s && n, EB_ERR_ARG, "eb_sched_free_pages: null");
  *n = (int32_t)s->free_list.size();
  return EB_OK;
}

int32_t eb_sched_seq_len(const eb_sched* s, int32_t slot, int32_t* len) {
  EB_REQUIRE(s && len, EB_ERR_ARG, "eb_sched_seq_len: null");
  EB_REQUIRE(live(s, slot), EB_ERR_STATE, "eb_sched_seq_len: slot %d is not live", slot);
  *len = s->len[(size_t)slot];
  return EB_OK;
}

int32_t eb_sched_block_tables(const eb_sched* s, const int32_t** h_tables, int32_t* stride) {
  EB_REQUIRE(s && h_tables && stride, EB_ERR_ARG, "eb_sched_block_tables: null");
  *h_tables = s->tables.data();
  *stride = s->max_pages;
  return EB_OK;
}

int32_t eb_sched_pack(const eb_sched* s, const int32_t* slots, const int32_t* q_lens, int32_t n_seqs, int32_t* q_off,
                      int32_t* ctx_lens, int32_t* tok_seq, int32_t* tok_slot, int32_t* positions, int32_t* n_tokens) {
  EB_REQUIRE(s && slots && q_lens && q_off && ctx_lens && tok_seq && tok_slot && positions && n_tokens, EB_ERR_ARG,
             "eb_sched_pack: null");
  EB_REQUIRE(n_seqs >= 0, EB_ERR_ARG, "eb_sched_pack: negative n_seqs");
  for (int32_t i = 0; i < n_seqs; ++i) {
    EB_REQUIRE(live(s, slots[i]), EB_ERR_STATE, "eb_sched_pack: sequence %d names slot %d, which is not live", i,
               slots[i]);
    EB_REQUIRE(q_lens[i] >= 1 && q_lens[i] <= s->len[(size_t)slots[i]], EB_ERR_ARG,
               "eb_sched_pack: sequence %d has q_len %d but holds %d tokens", i, q_lens[i], s->len[(size_t)slots[i]]);
  }
  int32_t t = 0;
  for (int32_t i = 0; i < n_seqs; ++i) {
    const int32_t L = s->len[(size_t)slots[i]];
    q_off[i] = t;
    ctx_lens[i] = L;
    for (int32_t j = 0; j < q_lens[i]; ++j, ++t) {
      tok_seq[t] = i;
      tok_slot[t] = slots[i];
      positions[t] = L - q_lens[i] + j;
    }
  }
  q_off[n_seqs] = t;
  *n_tokens = t;
  return EB_OK;
}

int32_t eb_attn_plan_sm_count(int32_t sm_count, int32_t max_q_len, int32_t n_q, int32_t n_kv, int32_t window) {
  if (sm_count < 1 || max_q_len < 1 || n_q < 1 || n_kv < 1) return sm_count < 1 ? 1 : sm_count;
  const int32_t rows = max_q_len * (n_q / n_kv);
  // decode shapes, and verify shapes on short windows: one CTA per item works on all KV heads of the rank
  if (rows <= 16 || (window > 0 && window < 2048)) return sm_count;
  // verify shapes on long items: one CTA per (item, KV head), two per SM
  return std::max(1, 2 * sm_count / n_kv);
}

int32_t eb_attn_plan(const int32_t* ctx_lens, const int32_t* q_lens, int32_t n_seqs, int32_t page_size,
                     int32_t window, int32_t sm_count, int32_t chunk_pages, int32_t parts_per_item,
                     eb_attn_item* items, int32_t cap_items, int32_t* n_items, int32_t* seq_part, int32_t* n_parts) {
  EB_REQUIRE(ctx_lens && q_lens && items && n_items && seq_part && n_parts, EB_ERR_ARG, "eb_attn_plan: null");
  EB_REQUIRE(n_seqs >= 0 && page_size > 0 && window >= 0 && sm_count > 0 && chunk_pages >= 0 && parts_per_item >= 1,
             EB_ERR_ARG, "eb_attn_plan: bad scalar argument");
  struct Range {
    int32_t pb, pe;
  };
  std::vector<Range> rg((size_t)n_seqs);
  int64_t total = 0;
  int32_t max_np = 0;
  for (int32_t i = 0; i < n_seqs; ++i) {
    const int32_t L = ctx_lens[i], ql = q_lens[i];
    EB_REQUIRE(ql >= 1 && L >= ql, EB_ERR_ARG, "eb_attn_plan: sequence %d has q_len %d, context %d", i, ql, L);
    const int32_t t_lo = window > 0 ? std::max(0, L - ql - window + 1) : 0;
    rg[(size_t)i].pb = t_lo / page_size;
    rg[(size_t)i].pe = (L + page_size - 1) / page_size;
    total += rg[(size_t)i].pe - rg[(size_t)i].pb;
    max_np = std::max(max_np, rg[(size_t)i].pe - rg[(size_t)i].pb);
  }
  int32_t chunk = chunk_pages;
  if (chunk == 0) {
    const int64_t target = 4ll * sm_count;
    chunk = (int32_t)std::min<int64_t>(512, std::max<int64_t>(8, (total + target - 1) / target));
    // Short ranges (windowed layers of a large batch): when the unsplit sequences already give every SM an item,
    // halving each only adds a second wave of CTAs and the merge launch, so leave them whole.
    if (n_seqs >= sm_count && max_np <= 2 * chunk) chunk = std::max(chunk, std::min(512, max_np));
  }
  EB_REQUIRE(chunk >= 1 && chunk <= 512, EB_ERR_ARG, "eb_attn_plan: chunk_pages %d outside 1..512", chunk);
  int32_t n = 0, parts = 0;
  for (int32_t i = 0; i < n_seqs; ++i) {
    const int32_t np = rg[(size_t)i].pe - rg[(size_t)i].pb;
    const int32_t k = (np + chunk - 1) / chunk;
    EB_REQUIRE(n + k <= cap_items, EB_ERR_NOMEM, "eb_attn_plan: more than %d items", cap_items);
    seq_part[i] = parts;
    const int32_t base = np / k, rem = np % k;
    int32_t p = rg[(size_t)i].pb;
    for (int32_t c = 0; c < k; ++c) {
      const int32_t sz = base + (c < rem ? 1 : 0);
      items[n].seq = i;
      items[n].page_begin = p;
      items[n].page_end = p + sz;
      items[n].part = parts;
      p += sz;
      parts += parts_per_item;
      ++n;
    }
  }
  seq_part[n_seqs] = parts;
  std::stable_sort(items, items + n, [](const eb_attn_item& a, const eb_attn_item& b) {
    return (a.page_end - a.page_begin) > (b.page_end - b.page_begin);
  });
  *n_items = n;
  *n_parts = parts;
  return EB_OK;
}

}  // extern "C"

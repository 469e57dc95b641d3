/*
 * eidola_b200.h -- C ABI of libeidola_b200.so: the decode step of a paged-KV,
 * sink-attention, FP8 block-scaled, mixture-of-experts decoder on NVIDIA B200
 * (sm_100a).
 *
 * THIS SURFACE IS NEW.  The reference project (eidola-ai/eidola) has no operator
 * API: its only engine boundaries are text-in/text-out --
 *   * server side: `trait ChatBackend { send, list_models, send_stream }`
 *     (crates/eidola-server/src/backend.rs:87-108), sole implementation an HTTPS
 *     client (`TinfoilBackend`, backend.rs:413-615);
 *   * client side: a `llama-server` child process started with the argv at
 *     crates/eidola-app-core/src/local_models.rs:1612-1626 and spoken to over
 *     loopback HTTP (crates/eidola-app-core/src/lib.rs:7155-7163).
 * Everything below is what an in-process engine behind either of those would
 * call every decode step.  Each entry point cites the reference code that would
 * sit above it; none replaces reference arithmetic, because there is none.
 *
 * Conventions
 *   * every function returns an int32 status: 0 = ok, negative = host-side
 *     validation error (nothing was launched), positive = CUDA runtime error
 *     code or a device status word read back by eb_status_read();
 *   * no exception crosses the boundary; eb_last_error() gives a log-safe
 *     message (sizes and indices only, never tensor contents -- the reference
 *     keeps payloads out of its logs, crates/eidola-server/AGENTS.md:65-66);
 *   * buffers are caller-owned unless an eb_engine owns them; pointers named
 *     d_* are device pointers, h_* are host pointers; `stream` is a
 *     cudaStream_t passed as void* (NULL = the legacy default stream);
 *   * one thread drives one handle at a time (the reference gives each engine
 *     a single owning supervisor task, local_models.rs:1633-1638).
 *
 * Tensor formats
 *   bf16   : uint16 bit patterns, round-to-nearest-even
 *   e4m3   : 1-4-3, bias 7, max 448, no infinity, saturating RNE
 *   scales : one fp32 per 128x128 block, row-major [ceil(rows/128)][ceil(cols/128)]
 *   KV page: [2 (K,V)][n_kv][page_size=16][head_dim=64] bf16, pages contiguous per layer
 */
#ifndef EIDOLA_B200_H_
#define EIDOLA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define EB_ABI_VERSION 5

/* status codes (negative: host validation) */
#define EB_OK 0
#define EB_ERR_ARG (-1)        /* null pointer, size out of range, misaligned */
#define EB_ERR_UNSUPPORTED (-2) /* shape outside what the kernels are built for */
#define EB_ERR_NOMEM (-3)       /* page pool or sequence slots exhausted (scheduler) */
#define EB_ERR_NODEVICE (-4)    /* no sm_100 device / driver entry point missing */
#define EB_ERR_STATE (-5)       /* call order (e.g. unknown sequence slot) */
/* device status word bits (positive, OR-ed) */
#define EB_DEV_WAIT_TIMEOUT 0x1000 /* a bounded wait inside a kernel gave up */
#define EB_DEV_BAD_INDEX 0x2000    /* a page id / expert id / row index was out of range and skipped */

int32_t eb_version(int32_t* abi);
/* Message for the last non-zero return on this thread. */
int32_t eb_last_error(char* buf, size_t n);

/* ---- device memory plumbing for callers without a CUDA binding ------------------
 * A Rust or C host needs these to own buffers without linking the CUDA runtime itself. */
int32_t eb_device_count(int32_t* n);
int32_t eb_device_set(int32_t device);
int32_t eb_device_info(int32_t device, int32_t* sm_count, int64_t* l2_bytes, int64_t* hbm_bytes, int32_t* cc_major,
                       int32_t* cc_minor);
/* Free and total device memory of the current device in bytes (cudaMemGetInfo). */
int32_t eb_device_mem_info(int64_t* free_bytes, int64_t* total_bytes);
int32_t eb_malloc(void** d_ptr, size_t bytes);
int32_t eb_free(void* d_ptr);
int32_t eb_host_alloc(void** h_ptr, size_t bytes); /* pinned */
int32_t eb_host_free(void* h_ptr);
int32_t eb_memset(void* d_ptr, int32_t value, size_t bytes, void* stream);
int32_t eb_copy_h2d(void* d_dst, const void* h_src, size_t bytes, void* stream);
int32_t eb_copy_d2h(void* h_dst, const void* d_src, size_t bytes, void* stream);
int32_t eb_copy_d2d(void* d_dst, const void* d_src, size_t bytes, void* stream);
int32_t eb_stream_create(void** stream);
int32_t eb_stream_destroy(void* stream);
int32_t eb_stream_sync(void* stream);
int32_t eb_device_sync(void);
int32_t eb_event_create(void** ev);
int32_t eb_event_destroy(void* ev);
int32_t eb_event_record(void* ev, void* stream);
int32_t eb_event_elapsed_ms(void* ev_start, void* ev_stop, float* ms); /* synchronises on ev_stop */
/* Writes `bytes` of a scratch buffer so that the L2 holds none of the caller's tensors. */
int32_t eb_l2_flush(void* d_scratch, size_t bytes, void* stream);
/* Every wait inside a kernel (on a shared-memory barrier fed by TMA or by the tensor core) is a bounded poll: after
 * `tries` polls the kernel raises EB_DEV_WAIT_TIMEOUT, drains its copies in flight, frees its tensor memory and
 * returns, so the context stays usable and the host decides what to do (the reference turns a stalled engine into an
 * error the same way: a 300 s readiness budget, crates/eidola-app-core/src/local_models.rs:2020-2064).  The default
 * is 2^22 polls (seconds); EIDOLA_B200_WAIT_TRIES or eb_wait_limit_set() set it for launches made afterwards. */
int32_t eb_wait_limit_set(uint32_t tries);
int32_t eb_wait_limit_get(uint32_t* tries);
/* Self-test of that discipline: one CTA polls, at most `tries` (<= 2^20) times, a barrier that nothing completes.  The
 * kernel returns, EB_DEV_WAIT_TIMEOUT appears in the status word, *h_polls receives the polls made.  Nothing hangs. */
int32_t eb_selftest_wait_expires(uint32_t tries, uint32_t* h_polls);
/* Device status word (EB_DEV_* bits) accumulated by kernels since the last read; reading clears it. */
int32_t eb_status_read(int32_t* status);

/* ---- synthetic tensors (definition: eb_synth.h) ------------------------------------
 * Fill device buffers with the seeded tensors the benchmark configurations describe. */
int32_t eb_synth_normal_bf16(void* d_out, int64_t n, uint64_t seed, uint64_t stream_id, uint64_t idx0, float scale,
                             void* stream);
int32_t eb_synth_normal_f32(void* d_out, int64_t n, uint64_t seed, uint64_t stream_id, uint64_t idx0, float scale,
                            void* stream);
int32_t eb_synth_normal_e4m3(void* d_out, int64_t n, uint64_t seed, uint64_t stream_id, uint64_t idx0, float scale,
                             void* stream);
int32_t eb_synth_uniform_f32(void* d_out, int64_t n, uint64_t seed, uint64_t stream_id, uint64_t idx0, float lo,
                             float hi, void* stream);
/* Random-init weight band [row0, row0+nrows) x cols of a [rows_total x cols] tensor ~ N(0, std), quantised to
 * e4m3 with per-128x128 scales.  row0 must be a multiple of 128. */
int32_t eb_synth_weight_fp8(void* d_codes, void* d_scales, int64_t rows_total, int64_t cols, int64_t row0,
                            int64_t nrows, uint64_t seed, uint64_t stream_id, float std, void* stream);

/* The block [row0, +nrows) x [col0, +ncols) of the same tensor (row0 and col0 multiples of 128, so its scale blocks
 * are the tensor's own): what a tensor-parallel rank holds of a column-sharded weight. */
int32_t eb_synth_weight_fp8_slice(void* d_codes, void* d_scales, int64_t rows_total, int64_t cols_total, int64_t row0,
                                  int64_t nrows, int64_t col0, int64_t ncols, uint64_t seed, uint64_t stream_id,
                                  float std, void* stream);
/* Checkpoint weights: fp32 [nrows][ld] (the first `cols` of each row) -> e4m3 codes [nrows][cols] + one fp32 scale per
 * 128x128 block (scale = block amax / 448, codes = rne(w / scale) saturating), the quantiser the seeded weights use. */
int32_t eb_quant_weight_f32(const float* d_w, int64_t ld, int64_t nrows, int64_t cols, void* d_codes, void* d_scales, void* stream);
int32_t eb_f32_to_bf16(const float* d_in, void* d_out, int64_t n, void* stream);
/* KV heads [head0, head0+n_kv_local) of a cache filled with N(0,1) values indexed by their position in the global
 * layout [pages][2][n_kv_total][page_size][head_dim], so every rank holds its slice of one global tensor. */
int32_t eb_synth_kv_heads_bf16(void* d_cache, int64_t num_pages, int32_t n_kv_total, int32_t head0, int32_t n_kv_local,
                               int32_t page_size, int32_t head_dim, uint64_t seed, uint64_t stream_id, void* stream);

/* ---- scheduler: continuous batching over a page pool (host only, no CUDA call) ------
 * Nearest reference analogue: the whole-engine admission planner `plan_evictions` /
 * `reserve_engine` (crates/eidola-app-core/src/local_models.rs:441-485, 653-701), which admits
 * engines against a byte budget in one critical section; here the unit is a 16-token page. */
typedef struct eb_sched eb_sched;

int32_t eb_sched_create(int32_t num_pages, int32_t page_size, int32_t max_seqs, int32_t max_pages_per_seq,
                        uint64_t seed, eb_sched** out);
int32_t eb_sched_destroy(eb_sched* s);
/* Admit a sequence with `context_len` tokens already to be held; returns its slot.  EB_ERR_NOMEM when the pool
 * cannot hold it (nothing is changed, like the reference planner's refusal without eviction). */
int32_t eb_sched_admit(eb_sched* s, int32_t context_len, int32_t* slot);
/* Grow a sequence to `new_len` tokens, taking pages from the shuffled free list as needed. */
int32_t eb_sched_extend(eb_sched* s, int32_t slot, int32_t new_len);
/* Roll a sequence back to `new_len` tokens (rejected draft tokens); whole pages past the end are returned. */
int32_t eb_sched_truncate(eb_sched* s, int32_t slot, int32_t new_len);
int32_t eb_sched_release(eb_sched* s, int32_t slot);
/* Admission with eviction: the reference's memory-pool planner (`plan_evictions`, crates/eidola-app-core/src/
 * local_models.rs:653-701: least recently used first, never a pinned engine nor one serving a turn, refuse without
 * unloading anything when that cannot make room) and its plan-and-reserve critical section (`reserve_engine`,
 * local_models.rs:441-485), with 16-token pages for bytes and sequences for engines.
 * eb_sched_touch records a use (`now` is any monotonic tick of the caller); eb_sched_set_flags sets pinned / in_flight
 * (-1 = leave as is); eb_sched_plan_evictions only plans (victims in LRU order; nothing changes);
 * eb_sched_admit_evicting releases the victims and admits, or returns EB_ERR_NOMEM having changed nothing. */
int32_t eb_sched_touch(eb_sched* s, int32_t slot, int64_t now);
int32_t eb_sched_set_flags(eb_sched* s, int32_t slot, int32_t pinned, int32_t in_flight);
int32_t eb_sched_plan_evictions(const eb_sched* s, int32_t context_len, int32_t* evict_slots, int32_t cap, int32_t* n_evict);
int32_t eb_sched_admit_evicting(eb_sched* s, int32_t context_len, int64_t now, int32_t* slot, int32_t* evict_slots, int32_t cap,
                                int32_t* n_evict);
int32_t eb_sched_free_pages(const eb_sched* s, int32_t* n);
int32_t eb_sched_seq_len(const eb_sched* s, int32_t slot, int32_t* len);
/* Block table of all slots: [max_seqs][max_pages_per_seq] int32, unused entries -1.  The pointer stays valid
 * until the scheduler is destroyed. */
int32_t eb_sched_block_tables(const eb_sched* s, const int32_t** h_tables, int32_t* stride);
/*
 * Pack a ragged step.  For each of n_seqs sequences (slots[i], q_lens[i] new tokens, already counted in the
 * sequence length by eb_sched_extend) write:
 *   q_off[n_seqs+1]   exclusive prefix sum of q_lens (row offsets into the flat token arrays)
 *   ctx_lens[n_seqs]  sequence length including the new tokens
 *   tok_seq[T]        index i of the sequence each token row belongs to
 *   tok_slot[T]       scheduler slot of each token row
 *   positions[T]      absolute position of each token row
 * Returns T through n_tokens.
 */
int32_t eb_sched_pack(const eb_sched* s, const int32_t* slots, const int32_t* q_lens, int32_t n_seqs, int32_t* q_off,
                      int32_t* ctx_lens, int32_t* tok_seq, int32_t* tok_slot, int32_t* positions, int32_t* n_tokens);

/* One unit of attention work: a run of logical pages of one sequence. */
typedef struct eb_attn_item {
  int32_t seq;        /* index into the step's sequence arrays */
  int32_t page_begin; /* first logical page (index into the block-table row) */
  int32_t page_end;   /* one past the last logical page */
  int32_t part;       /* first partial-result slot this item writes */
} eb_attn_item;

/*
 * The value to pass as `sm_count` to eb_attn_plan for a launch of these shapes, so that its automatic chunk size suits
 * the kernel eb_attn_paged_sink will run: decode shapes (at most 16 query rows per KV head) and verify shapes on windows
 * below 2048 tokens run one CTA per work item over all KV heads of the rank (-> sm_count); verify shapes on longer items
 * run one CTA per (work item, KV head), two per SM (-> 2 * sm_count / n_kv, at least 1).  A plan made with any other
 * value is still correct, only cut finer or coarser than the kernel likes.  No reference counterpart (the reference
 * delegates inference, crates/eidola-app-core/src/local_models.rs:1612-1626).
 */
int32_t eb_attn_plan_sm_count(int32_t sm_count, int32_t max_q_len, int32_t n_q, int32_t n_kv, int32_t window);

/*
 * Split-K plan for one attention launch.  Long contexts are cut into runs of at most `chunk_pages` pages
 * (0 = choose so that about 4 items per SM exist, at least 8 pages each; a batch of at least sm_count sequences
 * whose longest visible range is within two such runs is left unsplit); items are ordered longest first.
 *   items[cap_items], seq_part[n_seqs+1] (partial-slot range of each sequence)
 * window = 0 plans a full layer, otherwise only the pages a `window`-token sliding window can see.
 * parts_per_item = 8 / n_kv_local (warps that share a KV head write separate partials).
 */
int32_t eb_attn_plan(const int32_t* ctx_lens, const int32_t* q_lens, int32_t n_seqs, int32_t page_size,
                     int32_t window, int32_t sm_count, int32_t chunk_pages, int32_t parts_per_item,
                     eb_attn_item* items, int32_t cap_items, int32_t* n_items, int32_t* seq_part, int32_t* n_parts);

/* ---- operators (device pointers) ------------------------------------------------------ */

/* K1.  Scatter new K,V rows into one layer's paged cache.
 * d_k_new/d_v_new: [T][n_kv][head_dim] bf16, row stride in elements (>= n_kv*head_dim, multiple of 8). */
int32_t eb_kv_append(void* d_cache, int32_t num_pages, int32_t n_kv, int32_t head_dim, int32_t page_size,
                     const void* d_k_new, const void* d_v_new, int64_t row_stride, const int32_t* d_block_tables,
                     int32_t bt_stride, const int32_t* d_tok_slot, const int32_t* d_positions, int32_t n_tokens,
                     void* stream);

typedef struct eb_attn_args {
  const void* d_q;    /* [T][n_q][head_dim] bf16 */
  int64_t q_stride;   /* elements between token rows of q */
  void* d_out;        /* [T][n_q][head_dim] bf16 */
  int64_t out_stride; /* elements between token rows of out */
  const void* d_cache;
  int32_t num_pages;
  const int32_t* d_block_tables;
  int32_t bt_stride;
  const int32_t* d_seq_slots; /* [n_seqs] block-table row of each sequence */
  const int32_t* d_q_off;     /* [n_seqs+1] */
  const int32_t* d_ctx_lens;  /* [n_seqs] */
  int32_t n_seqs;
  int32_t max_q_len; /* largest q_len in the batch; max_q_len * (n_q / n_kv) <= 48 */
  const float* d_sinks; /* [n_q] learned sink logit per query head */
  int32_t window;       /* 0 = full attention */
  int32_t n_q, n_kv, head_dim, page_size; /* n_q / n_kv = 8 or 4; n_kv in {1,2,4,8}; head_dim 64; page_size 16 */
  float scale; /* 1/sqrt(head_dim) */
  const eb_attn_item* d_items;
  int32_t n_items;
  const int32_t* d_seq_part; /* [n_seqs+1] */
  int32_t n_parts;
  void* d_part_acc; /* fp32 [n_parts][max_q_len][n_q][head_dim] */
  void* d_part_ml;  /* fp32 [n_parts][max_q_len][n_q][2] */
} eb_attn_args;

/* K2+K3.  Paged sink attention (decode and k>1 verify) with split-K and log-sum-exp merge. */
int32_t eb_attn_paged_sink(const eb_attn_args* a, void* stream);
/*
 * K2+K3 for callers that cannot allocate device memory (this entry point has no counterpart in the reference
 * project).  A host that has given all device memory to its own pool, a plugin living inside another runtime's
 * allocator arena, or a thread that must never take the allocator's lock cannot hand eb_attn_paged_sink a
 * workspace; here the split-K scratch is two device arrays built into the library (16 MiB + 512 KiB, held by every
 * GPU that loads the library until the process exits).  d_part_acc / d_part_ml of the arguments are ignored.
 *   limit    : n_parts * max_q_len * n_q <= 65536 rows, else EB_ERR_NOMEM and nothing is launched (plan with a
 *              larger chunk_pages, or use eb_attn_paged_sink).  The kernels also check every partial slot the plan
 *              names against n_parts: a slot outside [0, n_parts) is skipped and EB_DEV_BAD_INDEX is raised, so a
 *              stale plan cannot write past the built-in arrays;
 *   d_status : caller-owned device int32 that receives EB_DEV_* bits (OR-ed in).  NULL = a word inside the library,
 *              read and cleared by eb_attn_static_status_read (which allocates nothing) and also folded into what
 *              eb_status_read reports (that one allocates its own word on first use);
 *   calls no cudaMalloc, cudaFree or other allocating routine.  The first call on a device resolves the addresses
 *   of the built-in arrays (cudaGetSymbolAddress, once per device, with that device current; concurrent first
 *   calls from several host threads are safe): make that first call before any stream capture begins;
 *   every call on a device shares the same scratch, which keeps the previous call's contents.  Nothing in it has
 *   to start at zero (each partial row is written before it is read), but two calls that overlap on the GPU --
 *   different streams, or the same scratch from two threads -- race on it: serialise them.
 */
int32_t eb_attn_paged_sink_static(const eb_attn_args* a, int32_t* d_status, void* stream);
/* EB_DEV_* bits raised by eb_attn_paged_sink_static calls on the current device that passed d_status = NULL; reading
 * clears them.  Allocates nothing (no counterpart in the reference project either). */
int32_t eb_attn_static_status_read(int32_t* status);
/* Workspace sizes for the two partial buffers of eb_attn_args. */
int32_t eb_attn_workspace(int32_t n_parts, int32_t max_q_len, int32_t n_q, int32_t head_dim, size_t* acc_bytes,
                          size_t* ml_bytes);

/* K8 (part).  Quantise bf16 activations to e4m3 with one fp32 scale per (128-row block, 128-column block).
 * Dense: d_seg_off = NULL, blocks are rows [128b, 128b+128).  Grouped: rows are grouped in n_groups segments
 * d_seg_off[n_groups+1] (device) and blocks restart at every segment start, numbered consecutively over the
 * segments.  d_scales: [n_blocks][ceil(cols/128)], n_blocks <= rows/128 + n_groups. */
int32_t eb_quant_act_block128(const void* d_x, int64_t ldx, int32_t rows, int32_t cols, const int32_t* d_seg_off,
                              int32_t n_groups, void* d_codes, void* d_scales, void* stream);

/* The same, reading row d_row_map[r] of a [src_rows x cols] matrix for output row r (token -> expert gather). */
int32_t eb_quant_gather_block128(const void* d_x, int64_t ldx, int32_t src_rows, const int32_t* d_row_map, int32_t rows,
                                 int32_t cols, const int32_t* d_seg_off, int32_t n_groups, void* d_codes,
                                 void* d_scales, void* stream);
/* The same on act = bf16(silu(gate) * up), where row r of d_gate_up holds [gate(cols) | up(cols)] bf16. */
int32_t eb_quant_silu_mul_block128(const void* d_gate_up, int64_t ld, int32_t rows, int32_t cols,
                                   const int32_t* d_seg_off, int32_t n_groups, void* d_codes, void* d_scales,
                                   void* stream);

typedef struct eb_gemm_args {
  const void* d_x8;  /* [rows][K] e4m3 activations */
  const float* d_sx; /* [row blocks][ceil(K/128)] */
  const void* d_w8;  /* [n_groups][N][K] e4m3 weights */
  const float* d_sw; /* [n_groups][ceil(N/128)][ceil(K/128)] */
  void* d_y;         /* [rows][N] bf16 */
  int64_t ldy;       /* elements between rows of y */
  int32_t rows, N, K;
  int32_t n_groups;           /* 1 = dense */
  const int32_t* d_seg_off;   /* grouped: [n_groups+1] row range of each group (device) */
  void* d_work;               /* eb_gemm_workspace() bytes; dense: optional (enables split K) */
  int32_t tile_tokens;        /* 0 = choose; else 16, 32, 64 or 128 tokens per tile */
  int32_t splits;             /* dense: 0 = choose, else K splits (needs d_work) */
  int32_t tiles_ready;        /* grouped: 1 = d_work already holds eb_gemm_group_tiles() output for these segments */
  size_t work_bytes;          /* bytes the caller owns at d_work; a call that would need more is refused (explicit
                                 splits, grouped) or falls back to fewer K splits (splits = 0) */
  int32_t w_tiled;            /* 0: d_w8 is row-major [n_groups][N][K]; 1: d_w8 holds the 16 KiB tiles eb_weight_tile_fp8
                                 writes (same results bit for bit; HBM serves a tile as one contiguous read) */
} eb_gemm_args;

/* Weight layout for streaming.  A GEMM stage is 128 weight rows x 128 bytes of K; in a row-major matrix those are 128
 * separate 128-byte reads 1 K apart.  eb_weight_tile_fp8 rewrites [n_groups][N][K] e4m3 codes as
 * [n_groups][ceil(N/128)][ceil(K/128)][128 rows][128 bytes] (zero padded), so a stage is 16 KiB of consecutive bytes;
 * pass the result with w_tiled = 1.  Done once per weight tensor, e.g. when a checkpoint is loaded.  The block scales
 * keep their layout.  eb_weight_tiled_bytes gives the size of the tiled buffer. */
int32_t eb_weight_tiled_bytes(int32_t n_groups, int32_t N, int32_t K, size_t* bytes);
int32_t eb_weight_tile_fp8(const void* d_w8, int32_t n_groups, int32_t N, int32_t K, void* d_tiled, void* stream);
/* K4.  Y = X * W^T, e4m3 x e4m3 -> fp32 with per-128x128 block scales, bf16 out (tcgen05 tensor cores).
 * The weights (d_w8, d_sw) must be complete when the call is made: the kernel may fetch them before the work queued
 * ahead of it on the stream has finished (activations and scales of X are read only after it has). */
int32_t eb_gemm_fp8_block(const eb_gemm_args* a, void* stream);
/* K6.  The same per group g on rows [d_seg_off[g], d_seg_off[g+1]) with weights W[g]; activation scale blocks
 * restart at each segment start (the numbering eb_quant_act_block128 uses). */
int32_t eb_gemm_fp8_grouped(const eb_gemm_args* a, void* stream);
int32_t eb_gemm_workspace(int32_t rows, int32_t N, int32_t n_groups, size_t* bytes);
/* Dense GEMM that leaves split-K partials for a fused consumer: when it chose splits_used > 1 the fp32 partials
 * [splits_used][rows][N] are in d_work and d_y is untouched; when splits_used == 1 d_y holds the bf16 result. */
int32_t eb_gemm_fp8_block_partial(const eb_gemm_args* a, int32_t* splits_used, void* stream);
/* Measured ceiling of the FP8 tensor path on the current device: one CTA per SM issues `blocks` groups of four
 * tcgen05.mma.kind::f8f6f4 (128 x 256 x 32) back to back on operands resident in shared memory, no loads, no
 * epilogue; best of `reps` timed launches after a warm-up.  tflops = 2 * 128 * 256 * 128 * blocks * SMs / time: the
 * denominator "fraction of FP8 peak" is reported against (sample the SM clock beside it: the figure scales with it). */
int32_t eb_fp8_mma_peak(int32_t blocks, int32_t reps, float* best_ms, double* tflops);
/* Token-tile table of a grouped GEMM, built once and shared by GEMMs over the same segments (tiles_ready = 1). */
int32_t eb_gemm_group_tiles(const int32_t* d_seg_off, int32_t n_groups, int32_t rows, int32_t tile_tokens, void* d_work,
                            void* stream);

/* ---- MoE routing (K5, K7) ---------------------------------------------------------------- */

/* Router: logits = x * Wr^T (bf16 inputs, fp32 accumulation in a fixed order, so the choice is reproducible bit for
 * bit), top_k by value with ties to the lower expert, weights = softmax over the selected logits.
 * d_idx [T][top_k] int32, d_wts [T][top_k] fp32, d_logits [T][E] fp32 or NULL. */
int32_t eb_moe_route(const void* d_x, const void* d_wr, int32_t T, int32_t E, int32_t H, int32_t top_k, int32_t* d_idx,
                     float* d_wts, float* d_logits, void* stream);
/* Token -> expert permutation (stable by expert, then token, then slot): d_seg_off[E+1], d_perm_row[T*top_k] (row
 * of slot (t,j) in expert order), d_row_token[T*top_k] (token of each permuted row). */
int32_t eb_moe_permute(const int32_t* d_idx, int32_t T, int32_t top_k, int32_t E, int32_t* d_seg_off,
                       int32_t* d_perm_row, int32_t* d_row_token, void* stream);
/* The same, also writing the token-tile table of the grouped GEMMs over these segments into d_group_work
 * (what eb_gemm_group_tiles would build for rows = T*top_k and tile_tokens), so they run with tiles_ready = 1. */
int32_t eb_moe_permute_tiles(const int32_t* d_idx, int32_t T, int32_t top_k, int32_t E, int32_t* d_seg_off,
                             int32_t* d_perm_row, int32_t* d_row_token, int32_t tile_tokens, void* d_group_work,
                             void* stream);
/* x[t] = bf16(x[t] + bf16(sum_j w[t][j] * y[perm_row[t][j]])): weighted combine fused with the residual add. */
int32_t eb_moe_combine(const void* d_y, const int32_t* d_perm_row, const float* d_wts, int32_t T, int32_t top_k,
                       int32_t H, void* d_x, void* stream);

/* ---- per-token glue (K8) ---------------------------------------------------------------- */

int32_t eb_rmsnorm(const void* d_x, const float* d_g, int32_t T, int32_t H, float eps, void* d_y, void* stream);
/* cos/sin table [max_pos][head_dim/2], angle = pos * theta^(-2i/head_dim) evaluated in double (host buffers). */
int32_t eb_rope_table(int32_t max_pos, int32_t head_dim, double theta, float* h_cos, float* h_sin);
/* Rotate-half rotary embedding, in place, of n_heads heads starting at d_x in each token row. */
int32_t eb_rope(void* d_x, int64_t row_stride, int32_t n_heads, int32_t head_dim, const int32_t* d_positions, int32_t T,
                const float* d_cos, const float* d_sin, int32_t max_pos, void* stream);
int32_t eb_residual_add(void* d_x, const void* d_y, int64_t n, void* stream);
/* Fused consumers of a dense GEMM.  `d_part`/`splits`: fp32 split-K partials [splits][T][N] summed in split order
 * and rounded to bf16 first (splits = 1: d_y_bf16 is read instead).
 * eb_qkv_rope_append: rotary embedding of the q and k heads of the fused [q | k | v] row, q written to d_qkv (row
 * stride N), k and v appended to the paged cache.
 * eb_oproj_residual_rmsnorm: x = bf16(x + o); h = rmsnorm(x) * g. */
int32_t eb_qkv_rope_append(const float* d_part, int32_t splits, void* d_qkv, int32_t T, int32_t n_q, int32_t n_kv,
                           int32_t head_dim, const int32_t* d_positions, const float* d_cos, const float* d_sin,
                           int32_t max_pos, void* d_cache, int32_t num_pages, int32_t page_size,
                           const int32_t* d_block_tables, int32_t bt_stride, const int32_t* d_tok_slot, void* stream);
int32_t eb_oproj_residual_rmsnorm(const float* d_part, int32_t splits, const void* d_o_bf16, void* d_x, const float* d_g,
                                  int32_t T, int32_t H, float eps, void* d_h, void* stream);
/* x = bf16(x + bf16(sum over n_planes planes)); h = rmsnorm(x) * g.  The planes ([n_planes][plane_stride elements], the
 * first T*H of each used) are the partial products of the ranks of a tensor-parallel group, fp32 or bf16; they are added
 * in plane order in fp32 and the sum is rounded once. */
int32_t eb_planes_residual_rmsnorm(const void* d_planes, int32_t planes_are_bf16, int32_t n_planes, int64_t plane_stride, void* d_x,
                                   const float* d_g, int32_t T, int32_t H, float eps, void* d_h, void* stream);
/* The same with explicit row geometry: a row of d_qkv has row_elems elements, the K heads start at k_col0 and the V
 * heads at v_col0 (a tensor-parallel rank whose K/V heads share a 128-row scale block with a neighbour computes the
 * whole block and uses its part). */
int32_t eb_qkv_rope_append_ex(const float* d_part, int32_t splits, void* d_qkv, int32_t row_elems, int32_t k_col0,
                              int32_t v_col0, int32_t T, int32_t n_q, int32_t n_kv, int32_t head_dim,
                              const int32_t* d_positions, const float* d_cos, const float* d_sin, int32_t max_pos,
                              void* d_cache, int32_t num_pages, int32_t page_size, const int32_t* d_block_tables,
                              int32_t bt_stride, const int32_t* d_tok_slot, void* stream);
/* d_out[i] = sum over splits of d_part[s][i] (fp32), or the fp32 image of d_bf16 when d_part is NULL: the buffer an
 * all-reduce sums across ranks. */
int32_t eb_sum_planes_f32(const float* d_part, int32_t splits, const void* d_bf16, int64_t n, float* d_out, void* stream);
/* Expert parallelism: d_out[i] = d_idx[i] - e0 when that is one of this rank's e_local experts, else -1;
 * the permutation that skips the -1 slots (perm_row = -1); the fp32 partial mix of this rank's experts. */
int32_t eb_moe_localize(const int32_t* d_idx, int32_t n, int32_t e0, int32_t e_local, int32_t* d_out, void* stream);
int32_t eb_moe_permute_tiles_local(const int32_t* d_idx_local, int32_t T, int32_t top_k, int32_t e_local, int32_t* d_seg_off,
                                   int32_t* d_perm_row, int32_t* d_row_token, int32_t tile_tokens, void* d_group_work,
                                   void* stream);
int32_t eb_moe_combine_f32(const void* d_y, const int32_t* d_perm_row, const float* d_wts, int32_t T, int32_t top_k, int32_t H,
                           float* d_out, void* stream);
/* The same partial mix rounded once to bf16 (the operand of a bf16 reduce-scatter). */
int32_t eb_moe_combine_bf16(const void* d_y, const int32_t* d_perm_row, const float* d_wts, int32_t T, int32_t top_k, int32_t H,
                            void* d_out, void* stream);
/* x = bf16(x + bf16(sum_j w_j y[perm_row])) as eb_moe_combine, then h = rmsnorm(x) * g for the next consumer. */
int32_t eb_moe_combine_rmsnorm(const void* d_y, const int32_t* d_perm_row, const float* d_wts, int32_t T, int32_t top_k,
                               int32_t H, void* d_x, const float* d_g, float eps, void* d_h, void* stream);
/* The same with the bound of d_perm_row's values given explicitly (rows of d_y): the tokens may be a slice of a batch
 * whose rows are numbered over the whole batch. */
int32_t eb_moe_combine_rmsnorm_ex(const void* d_y, const int32_t* d_perm_row, const float* d_wts, int32_t T, int32_t top_k,
                                  int32_t H, int64_t n_rows, void* d_x, const float* d_g, float eps, void* d_h, void* stream);
int32_t eb_embed(const void* d_table, int32_t V, int32_t H, const int32_t* d_tokens, int32_t T, void* d_x, void* stream);
/* Greedy argmax over bf16 logits [T][ld], ties to the lower id; d_margin (top1 - top2) may be NULL. */
int32_t eb_argmax(const void* d_logits, int32_t T, int64_t V, int64_t ld, int32_t* d_tok, float* d_margin, void* stream);
/* Vocabulary-parallel argmax.  Partial: over columns [0, V) of d_logits (a rank's slice, whose first column is token id
 * v_off) write per row a candidate {top1 value, top2 value, top1 id as int bits, 0} to d_cand[T][4].  Merge: n_parts
 * candidate sets laid out [n_parts][part_stride rows][4], slices in ascending id order -> greedy token (ties to the
 * lower id) and top1 - top2 margin, identical to eb_argmax over the concatenated logits. */
int32_t eb_argmax_partial(const void* d_logits, int32_t T, int64_t V, int64_t ld, int32_t v_off, float* d_cand, void* stream);
int32_t eb_argmax_merge(const float* d_cand, int32_t n_parts, int64_t part_stride, int32_t T, int32_t* d_tok, float* d_margin,
                        void* stream);

/* Temperature / nucleus (top-p) sampling over bf16 logits [T][ld], one token per row, for rows whose d_scale is > 0
 * (the others are left alone: a greedy row keeps what eb_argmax wrote to d_tok).  The reference server's request type
 * carries `temperature` and `top_p` (crates/eidola-server/src/types.rs:24-30) and forwards them to a remote engine; this
 * is what an engine behind that boundary does with them.  Per row: d_scale = log2(e) / temperature as fp32;
 * d_top_p_q24 = top_p in units of 2^-24 (>= 2^24: the whole vocabulary); d_rand32 = one uniform 32-bit number
 * (eb_sample_rand32(seed, position) gives a counter-based one).  The token is a pure function of those and the logits:
 * weights W_v = trunc(2^31 * 2^((x_v - max) * scale)) from separately rounded fp32 operations, the nucleus = every
 * token whose logit is at least the largest threshold with tail mass >= max(1, sum(W) * top_p), and the token = the
 * first one, in id order, whose running nucleus mass exceeds (mass * rand32) >> 32 -- integer arithmetic throughout, so
 * the CPU checker reproduces it bit for bit.  Rows without a finite maximum are left alone. */
int32_t eb_sample_top_p(const void* d_logits, int32_t T, int64_t V, int64_t ld, const float* d_scale, const uint32_t* d_top_p_q24,
                        const uint32_t* d_rand32, int32_t* d_tok, void* stream);
uint32_t eb_sample_rand32(uint64_t seed, uint64_t counter); /* host: splitmix64 of (seed, counter), upper half */

/* ---- engine: the whole decode step ------------------------------------------------------------
 * What an in-process implementation of the reference's engine boundary would drive once per generated token:
 * the reference client posts to `llama-server` and reads tokens back as SSE chunks
 * (crates/eidola-app-core/src/lib.rs:7155-7163, 7232-7340); the server relays a provider's chunks
 * (crates/eidola-server/src/backend.rs:481-615).  Tokenisation, chat templating and sampling policy stay above
 * this call; the engine takes token ids and returns the greedy next token of every row. */
typedef struct eb_config {
  int32_t n_layers, hidden, n_q_heads, n_kv_heads, head_dim;
  int32_t window;       /* sliding window of even layers (odd layers attend to everything) */
  int32_t n_experts, top_k, inter, vocab;
  int32_t page_size, num_pages, max_seqs, max_pages_per_seq;
  int32_t max_tokens;   /* token rows per step (sum of q_len) */
  int32_t max_q_len;    /* new tokens per sequence per decode / verify step: 1 = decode, k+1 = verify k drafts; also the
                           run of tokens one attention work entry covers (prefill chunks are cut into such runs) */
  float rope_theta, rms_eps, init_std;
  uint64_t seed;        /* weights are a pure function of (shape, seed) */
  int32_t debug;        /* bit 0: keep per-layer routing indices / hidden states readable and allow teacher forcing;
                           bit 1: time attention, GEMM and LM-head calls of each step with CUDA events */
  int32_t window_ring;  /* 1: sliding-window layers keep only a ring of ceil((window + chunk)/page_size) + 1 pages per
                           sequence (logical page p lives in ring page p mod ring) instead of the whole context; chunk =
                           eb_engine_chunk_tokens, which a ring holds down to min(max_tokens, 256) */
} eb_config;

typedef struct eb_engine eb_engine;

/* ---- communicator (NCCL, bound at run time with dlopen) ---------------------------------------
 * Rank 0 makes a 128-byte id, hands it to the other ranks by any channel, every rank (its device current) creates. */
typedef struct eb_comm eb_comm;
int32_t eb_comm_unique_id(void* h_id128);
int32_t eb_comm_create(const void* h_id128, int32_t rank, int32_t size, eb_comm** out);
int32_t eb_comm_destroy(eb_comm* c);
int32_t eb_comm_info(const eb_comm* c, int32_t* rank, int32_t* size);
int32_t eb_comm_allreduce_f32(eb_comm* c, void* d_buf, int64_t count, void* stream);
/* In-place all-gather of 1..3 buffers in one NCCL group: rank r's bytes_per_rank[i] bytes sit at offset
 * r * bytes_per_rank[i] of buffer i before the call, every rank holds all slices after it. */
int32_t eb_comm_allgather(eb_comm* c, int32_t n_bufs, void* const* d_bufs, const int64_t* bytes_per_rank, void* stream);
/* In-place fp32 reduce-scatter: d_buf holds size * count_per_rank floats; on return rank r's slice
 * [r * count_per_rank, (r + 1) * count_per_rank) holds the sum over ranks, the other slices are undefined. */
int32_t eb_comm_reduce_scatter_f32(eb_comm* c, void* d_buf, int64_t count_per_rank, void* stream);
/* The same on bf16 elements: half the bytes, the sum rounded to bf16 on the way. */
int32_t eb_comm_reduce_scatter_bf16(eb_comm* c, void* d_buf, int64_t count_per_rank, void* stream);
/* 0 = healthy.  A host whose step does not return within its own deadline, or that reads a non-zero value, aborts
 * the communicator and rebuilds it (failure handling stays on the host; kernels never wait on a peer). */
int32_t eb_comm_async_error(eb_comm* c, int32_t* err);
int32_t eb_comm_abort(eb_comm* c);

/* ---- symmetric peer memory (NVLink / NVSwitch stores) ------------------------------------------------------------
 * Every rank of a communicator allocates an arena of `bytes` and maps its peers' arenas (CUDA IPC; the handles travel
 * once through the communicator).  eb_symm_push copies rows from the local arena straight into the peers' arenas with
 * plain stores and then raises this rank's flag on every peer; eb_symm_wait polls, with the library's bounded-wait
 * discipline, the flags the peers raise here.  An all-gather or the data movement of a reduce-scatter is one push and
 * one wait (two small kernels) instead of a library collective; sums are left to the consumer kernel, which adds the
 * ranks' planes in a fixed order.  Nothing ever loads from a peer.  A rank that stops pushing makes its peers' waits
 * run out: EB_DEV_WAIT_TIMEOUT appears in the status word and the step's results must be discarded. */
typedef struct eb_symm eb_symm;
int32_t eb_symm_create(eb_comm* c, size_t bytes, eb_symm** out);
int32_t eb_symm_destroy(eb_symm* s);
/* Base address, in this process, of rank `rank`'s arena (the own rank's is ordinary device memory). */
int32_t eb_symm_ptr(const eb_symm* s, int32_t rank, void** ptr, size_t* bytes);
/* Segment i copies, for every destination rank p, min(bytes[i], src_valid[i] - p * src_step[i]) bytes from local offset
 * src_off[i] + p * src_step[i] to offset dst_off[i] + my_rank * dst_step[i] of rank p's arena (all multiples of 4;
 * src_valid NULL = everything; self_copy: also to the own arena).  At most 4 segments.  *seq identifies the collective. */
int32_t eb_symm_push(eb_symm* s, int32_t n_segs, const int64_t* src_off, const int64_t* src_step, const int64_t* dst_off,
                     const int64_t* dst_step, const int64_t* bytes, const int64_t* src_valid, int32_t self_copy, int32_t* seq,
                     void* stream);
/* C2, expert-parallel dispatch and return (the all-to-all pair) as row stores.  Rows are numbered globally -- position in
 * the expert-major order over ALL experts, which every rank computes from the gathered routing (eb_moe_permute) -- so a
 * row sits at the same offset in every arena and no counts are exchanged.
 * dispatch: for each token t in [t0, t0 + nt) of this rank's slice and each slot j, the row src_off + t * row_bytes goes
 *           to the rank that holds expert d_idx[t][j] (experts_per_rank consecutive experts per rank), at row d_perm[t][j]
 *           of dst_off.
 * return  : every row i of this rank's experts' range [d_seg_off[first_expert], d_seg_off[first_expert + experts_per_rank])
 *           goes from src_off + i * row_bytes to the same row of dst_off on the rank that owns token d_row_token[i]
 *           (tokens are dealt to ranks in chunks of chunk_tokens).
 * Both raise the flags like eb_symm_push; eb_symm_wait(seq) on the receiving side. */
int32_t eb_symm_dispatch_rows(eb_symm* s, int64_t src_off, int64_t dst_off, int32_t row_bytes, const int32_t* d_idx,
                              const int32_t* d_perm, int32_t t0, int32_t nt, int32_t top_k, int32_t experts_per_rank,
                              int32_t n_experts, int32_t n_rows, int32_t* seq, void* stream);
int32_t eb_symm_return_rows(eb_symm* s, int64_t src_off, int64_t dst_off, int32_t row_bytes, const int32_t* d_row_token,
                            const int32_t* d_seg_off, int32_t first_expert, int32_t experts_per_rank, int32_t chunk_tokens,
                            int32_t n_rows, int32_t* seq, void* stream);
/* Returns (in stream order) once every peer's push `seq` has arrived here, or the bounded wait has run out.  `patience`
 * (1..64) multiplies the wait limit: the first collective of a step also absorbs the skew between the ranks' host
 * loops, the later ones only the skew between their kernels. */
int32_t eb_symm_wait(eb_symm* s, int32_t seq, int32_t patience, void* stream);
/* Producers of a whole-batch exchange that store their result straight into every rank's arena (this rank's plane at
 * dst_off + rank * plane_step, its own arena included) and raise the collective's flags themselves, so no eb_symm_push
 * launch follows them: the sum of `splits` fp32 planes of n elements (the arithmetic of eb_sum_planes_f32), and the
 * bf16 mix of this rank's experts' rows (the arithmetic of eb_moe_combine_bf16).  `seq` receives the collective's
 * sequence number for eb_symm_wait / eb_planes_residual_rmsnorm_after. */
int32_t eb_sum_planes_f32_to_peers(eb_symm* s, int64_t dst_off, int64_t plane_step, const float* d_part, int32_t splits, int64_t n,
                                   int32_t* seq, void* stream);
int32_t eb_moe_combine_bf16_to_peers(eb_symm* s, int64_t dst_off, int64_t plane_step, const void* d_y, const int32_t* d_perm_row,
                                     const float* d_wts, int32_t T, int32_t top_k, int32_t H, int32_t* seq, void* stream);
/* Quantises this rank's column band of an operand that every rank assembles (the attention output before a replicated O
 * projection): x [rows][cols] bf16 -> e4m3 codes and 128x128 block scales, stored straight into EVERY rank's arena, the
 * codes at codes_off + rank * cols with row pitch ld_codes, the scales at scales_off + rank * cols / 128 (floats) with
 * ld_scales scales per row block; the launch raises the collective's flags itself (seq for eb_symm_wait).  With
 * slice_rows > 0 (a multiple of 128) rows [p * slice_rows, +slice_rows) go to rank p alone, the owner of that token slice;
 * with 0 all rows go to all ranks.  The codes and scales are those of eb_quant_act_block128 on the same band. */
int32_t eb_quant_act_block128_to_peers(eb_symm* s, const void* d_x, int64_t ldx, int32_t rows, int32_t cols, int64_t codes_off,
                                       int64_t ld_codes, int64_t scales_off, int32_t ld_scales, int32_t slice_rows, int32_t* seq,
                                       void* stream);
/* eb_planes_residual_rmsnorm on planes that the ranks of `s` pushed as collective `seq`: every CTA waits, bounded, for its
 * peers' flags itself, so no eb_symm_wait launch is needed between the push and this call.  s == NULL: no wait. */
int32_t eb_planes_residual_rmsnorm_after(eb_symm* s, int32_t seq, int32_t patience, const void* d_planes, int32_t planes_are_bf16,
                                         int32_t n_planes, int64_t plane_stride, void* d_x, const float* d_g, int32_t T, int32_t H,
                                         float eps, void* d_h, void* stream);

int32_t eb_engine_create(const eb_config* cfg, eb_engine** out);
/* Tensor-parallel heads + expert-parallel experts over tp_size ranks (one process per GPU): rank r holds query heads
 * [r*n_q/tp, ...), KV heads [r*n_kv/tp, ...) with their slice of every KV page (page ids are the same on all ranks),
 * the matching rows of W_qkv and columns of W_o, experts [r*E/tp, ...) and a band of whole 128-row blocks of the
 * LM head.  Every rank is given the same steps and returns the same tokens; the model is the same tensor for every
 * tp_size (weights are slices of the single-GPU tensors).  The LM head is vocabulary-parallel: each rank leaves one
 * argmax candidate per token, the candidates are gathered and merged.
 *
 * Per layer the partial [tokens, hidden] products of the O projection and of the rank's experts have to be summed over
 * the ranks.  Three forms, chosen per step from its token count (every form gives the same bits):
 *   up to 512 tokens   every rank receives every rank's whole partial and adds them itself in rank order, so residual,
 *                      norm and routing run on all rows everywhere and nothing is gathered (two exchanges per layer);
 *   larger steps       the partials are summed over token slices (tp_size equal chunks of whole 128-row scale blocks);
 *                      the owner of a slice adds the residual, normalises, routes and quantises its rows, and gathers
 *                      return the normalised rows, the routing and the e4m3 codes with their block scales;
 *   from 1024 tokens   on four ranks and more the expert step instead sends each token's normalised row to the ranks of
 *                      its experts and the expert outputs back to the token's owner (dispatch / return of rows).
 * The exchanges are this library's own kernels over a symmetric peer-memory arena (eb_symm_*: plain stores into the
 * peers' memory, a flag per sender, a consumer kernel that waits for the flags with a bounded number of polls and
 * raises EB_DEV_WAIT_TIMEOUT instead of hanging); `comm` carries the set-up (exchange of the memory handles) and, with
 * EIDOLA_B200_TP_NCCL=1, the exchanges themselves as NCCL reduce-scatter / all-gather calls.  EIDOLA_B200_TP_WHOLE=0 and
 * EIDOLA_B200_EP_A2A=0|1 force one of the forms (A/B runs and tests).
 *
 * EIDOLA_B200_NVTX=1 (any engine): NVTX ranges around every step and its phases, for timeline tools.
 *
 * From four ranks on (peer-memory transport; EIDOLA_B200_TP_OGATHER=1|0 forces it on or off) the O projection has no
 * partial products at all: every rank keeps the whole W_o, quantises its heads' columns of the attention output straight
 * into the other ranks' copies of the operand (eb_quant_act_block128_to_peers: all rows to all ranks for steps of up to
 * 512 tokens, a token slice to its owner otherwise) and multiplies full-K rows itself.  One byte per (token, head column)
 * crosses the links instead of a [tokens, hidden] partial per rank, and the projection's bits are the single-GPU ones. */
int32_t eb_engine_create_tp(const eb_config* cfg, int32_t tp_rank, int32_t tp_size, eb_comm* comm, eb_engine** out);
int32_t eb_engine_destroy(eb_engine* e);
/* Device bytes held by weights, KV pages and workspaces. */
int32_t eb_engine_memory(const eb_engine* e, int64_t* weight_bytes, int64_t* kv_bytes, int64_t* work_bytes);
/*
 * Replace the seeded weights by a checkpoint in GGUF, the container the reference's client downloads and keeps on disk
 * (crates/eidola-app-core/src/local_models.rs:29-34, 1310-1385).  Tensors (F32, F16 or BF16; rows of `cols` elements):
 *   token_embd.weight [vocab][hidden]            output.weight [vocab][hidden]            output_norm.weight [hidden]
 *   blk.L.attn_norm.weight [hidden]              blk.L.ffn_norm.weight [hidden]           blk.L.attn_sinks.weight [n_q_heads]
 *   blk.L.attn_qkv.weight [(n_q + 2 n_kv) * head_dim][hidden]   (q heads, then k heads, then v heads)
 *   blk.L.attn_output.weight [hidden][n_q * head_dim]
 *   blk.L.ffn_gate_inp.weight [experts][hidden]                 (router)
 *   blk.L.ffn_gate_up_exps.weight [experts][2 * inter][hidden]  (gate rows, then up rows)
 *   blk.L.ffn_down_exps.weight [experts][hidden][inter]
 * The linear layers are quantised on the device to e4m3 with 128x128 block scales (eb_quant_weight_f32) and stored as
 * tiles; embeddings and router become bf16; norms and sinks stay fp32.  A tensor-parallel rank reads only its own rows,
 * columns and experts.  Tensor types read: F32, F16, BF16, and the block formats Q4_0, Q8_0 and MXFP4 (32 elements of a
 * row per scale; decoded to fp32 on the host, then quantised like the others); the other quantised GGUF types are
 * refused.  Returns EB_ERR_ARG naming the tensor when one is missing or has the wrong shape; the engine's weights are
 * then partly replaced and it must be reloaded or destroyed.
 */
int32_t eb_engine_load_gguf(eb_engine* e, const char* path);
/* Host only (no device): n elements from element elem0 of tensor `tensor` of a GGUF file as fp32, through the reader the
 * loader uses; ggml_type / n_elements (may be NULL) receive the tensor's stored type and size; n == 0 only asks for those. */
int32_t eb_gguf_read_f32(const char* path, const char* tensor, int64_t elem0, int64_t n, float* h_out, int32_t* ggml_type,
                         int64_t* n_elements);
/* Stand-in for prefill: fill every KV page of every layer with seeded N(0,1) values (element i of layer l is
 * eb_normal(seed, 20000 + l, i)), so a sequence admitted with a context length has keys and values to attend to. */
int32_t eb_engine_kv_fill_synth(eb_engine* e);
/* Scheduler of this engine (continuous batching): admit / release between steps. */
int32_t eb_engine_seq_admit(eb_engine* e, int32_t context_len, int32_t* slot);
/* The same through eb_sched_admit_evicting: idle sequences are released, least recently stepped first, to make room
 * (h_evicted receives their slots; their owners must re-admit and prefill them if they come back).  A sequence is
 * "used" whenever a step includes it. */
int32_t eb_engine_seq_admit_evicting(eb_engine* e, int32_t context_len, int32_t* slot, int32_t* h_evicted, int32_t cap,
                                     int32_t* n_evicted);
int32_t eb_engine_seq_pin(eb_engine* e, int32_t slot, int32_t pinned);
int32_t eb_engine_seq_release(eb_engine* e, int32_t slot);
/* Cut a sequence back to new_len tokens (rejected drafts; the common prefix of a conversation's next turn).  With
 * window_ring a cut deeper than the rings still cover (about eb_engine_chunk_tokens tokens below the longest the
 * sequence has been) is refused with EB_ERR_UNSUPPORTED and changes nothing. */
int32_t eb_engine_seq_truncate(eb_engine* e, int32_t slot, int32_t new_len);
/* Roll n sequences back in one call (after a verify step: new length = old length + accepted drafts + 1). */
int32_t eb_engine_seq_truncate_many(eb_engine* e, const int32_t* h_slots, const int32_t* h_new_lens, int32_t n);
int32_t eb_engine_seq_len(const eb_engine* e, int32_t slot, int32_t* len);
int32_t eb_engine_sched(eb_engine* e, eb_sched** sched); /* borrowed; lives as long as the engine */
/*
 * One step for n_seqs sequences: sequence i appends q_lens[i] tokens (h_tokens, flat, in sequence order), every
 * layer runs, and h_next[row] receives the greedy token after each of the T = sum(q_lens) rows (h_margin: top-1
 * minus top-2 logit, may be NULL).  Host buffers; the call returns after the results have arrived.
 * q_lens[i] may be anything from 1 to eb_engine_chunk_tokens (T <= max_tokens): runs longer than max_q_len (prefill
 * chunks) are cut into attention work entries of max_q_len tokens on the same block-table row, each causal among its own
 * tokens and seeing everything before it, so a whole prompt can go through in one step.
 */
int32_t eb_engine_step(eb_engine* e, const int32_t* h_slots, const int32_t* h_q_lens, int32_t n_seqs,
                       const int32_t* h_tokens, int32_t* h_next, float* h_margin);
/*
 * Prefill: run the prompts of n_seqs admitted sequences (h_n_tokens[i] tokens each, flat in h_tokens in sequence order)
 * through every layer, so that their K and V are in the paged cache, in chunks of up to eb_engine_chunk_tokens tokens
 * per sequence and max_tokens rows per step (sequences in order, each taking what it still needs or what is left of
 * the step) -- the same kernels, pages and block tables as decode and draft verification (a chunk is causal among its
 * own tokens and sees everything before it).  h_next[i] / h_margin[i] receive the greedy token and
 * top-2 margin after the LAST prompt token of sequence i: the first generated token.  What the reference's client
 * sends as `messages` and its engine turns into a prompt (crates/eidola-app-core/src/lib.rs:10812-10825) ends up here
 * as token ids.  steps_run / device_ms (may be NULL): steps taken and their summed device time.
 */
int32_t eb_engine_prefill(eb_engine* e, const int32_t* h_slots, const int32_t* h_n_tokens, int32_t n_seqs, const int32_t* h_tokens,
                          int32_t* h_next, float* h_margin, int32_t* steps_run, float* device_ms);
/* Most new tokens one sequence may bring to a step: max_tokens, or min(max_tokens, 256) with window_ring (never less than
 * max_q_len). */
int32_t eb_engine_chunk_tokens(const eb_engine* e, int32_t* tokens);
/* Sampling for one live sequence, from its next step on: temperature > 0 draws every new token of the sequence with
 * eb_sample_top_p (scale = log2(e) / temperature in fp32, top_p clamped to [0, 1], rand32 = eb_sample_rand32(seed,
 * absolute position of the token drawn), so a sequence's tokens do not depend on what shares its steps); temperature
 * <= 0 is greedy, the state of every newly admitted sequence.  h_margin stays the top-1 minus top-2 logit.  The request
 * fields this serves: crates/eidola-server/src/types.rs:24-30.  Single-GPU engines only: EB_ERR_UNSUPPORTED under tensor
 * parallelism, whose LM head is split over the vocabulary. */
int32_t eb_engine_seq_sampling(eb_engine* e, int32_t slot, float temperature, float top_p, uint64_t seed);
/* The same split in two so a caller can overlap host work: launch, then wait for the results. */
int32_t eb_engine_step_launch(eb_engine* e, const int32_t* h_slots, const int32_t* h_q_lens, int32_t n_seqs,
                              const int32_t* h_tokens);
int32_t eb_engine_step_wait(eb_engine* e, int32_t* h_next, float* h_margin);
/* Milliseconds the last step spent on the device (CUDA events around its kernels) and kernels it launched. */
int32_t eb_engine_last_step_stats(const eb_engine* e, float* device_ms, int32_t* kernel_launches);
/* Bytes the last step copied host -> device (the staging block: tokens, packing arrays, block-table patches, the two
 * attention plans) and device -> host (greedy tokens and margins). */
int32_t eb_engine_last_step_copies(const eb_engine* e, int64_t* h2d_bytes, int64_t* d2h_bytes);
/* Switch the per-call timing of debug bit 1 on or off between steps (the events add a millisecond or two to a step, so
 * a benchmark times its steps with it off and takes the breakdown from a few extra steps with it on). */
int32_t eb_engine_profile(eb_engine* e, int32_t on);
/* debug bit 1: device milliseconds of the last step by category (8 floats): [0] attention on full layers, [1] attention
 * on windowed layers, [2] QKV and O projections, [3] expert GEMMs, [4] LM head, [5] collectives (tensor-parallel
 * engines), [6] router, [7] activation quantisers.  What is left of the step is norms, rotary/append, permutation,
 * combine, argmax and the gaps between kernels. */
int32_t eb_engine_last_step_breakdown(const eb_engine* e, float* ms8);
/* The stream the engine launches on (borrowed), so a caller can record its own events around steps. */
int32_t eb_engine_stream(eb_engine* e, void** stream);
/* debug bit 0 only: copy out the last step's logits [T][vocab] bf16 and layer routing indices [T][top_k]. */
int32_t eb_engine_read_logits(eb_engine* e, void* h_logits, int64_t bytes);
int32_t eb_engine_read_routing(eb_engine* e, int32_t layer, int32_t* h_idx, int64_t bytes);
/* Copy out the residual stream [T][hidden] bf16 as it stood after `layer` (debug = 1; layer = -1: embeddings). */
int32_t eb_engine_read_hidden(eb_engine* e, int32_t layer, void* h_x, int64_t bytes);
/* debug bit 0: work buffers of the LAST layer of the last step, so a parity test can tell attention from what follows
 * it: which = 0 the fused projection rows [T][local q | k | v width] bf16 (the q heads rotated; the k and v columns
 * are not kept, they went to the cache), which = 1 the attention output [T][local q heads * head_dim] bf16. */
int32_t eb_engine_debug_read_last(eb_engine* e, int32_t which, void* h_out, int64_t bytes);
/* Teacher forcing for parity tests (debug = 1): before `layer` runs (layer = n_layers: before the final norm) the
 * residual stream of the next steps with exactly `rows` token rows is replaced by h_x [rows][hidden] bf16.  FP8
 * activation quantisation amplifies a one-ulp difference into percent-level differences a layer later, so a
 * layer is compared with a CPU restatement on identical inputs.  h_x = NULL clears the override. */
int32_t eb_engine_debug_force_hidden(eb_engine* e, int32_t layer, const void* h_x, int32_t rows);

#ifdef __cplusplus
}
#endif
#endif /* EIDOLA_B200_H_ */

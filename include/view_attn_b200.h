/*
 * view_attn_b200.h -- C ABI of the B200 (sm_100a) cache-view attention / Gated DeltaNet kernels.
 *
 * Every entry point takes plain device pointers and sizes, launches on the given CUDA stream,
 * allocates no device memory, keeps no reference to caller memory and never throws: it returns 0
 * or a negative VA_ERR_* code.  The caller (PyTorch host code, or any other runtime) owns all
 * memory.  The only driver objects the library creates are one non-blocking side stream and two
 * events per device, on the first va_view_decode call whose plan carries shared-block tiles
 * (`groups`); va_view_decode_static creates none.  Kernels that need more than 48 KB of shared
 * memory opt in with cudaFuncSetAttribute on the launching call.
 * Device-side faults (a page index outside the pool, a bounded wait that ran out) are reported
 * through the caller-supplied `status` word: 0 = clean, otherwise the first VA_DEV_* code seen.
 *
 * The citations name the reference code each entry point replaces
 * (paths relative to python/minisgl/ in dvmazur/async_llm).
 */
#ifndef VIEW_ATTN_B200_H_
#define VIEW_ATTN_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VA_OK 0
#define VA_ERR_BAD_ARG (-1)      /* null pointer, negative size, misaligned pointer            */
#define VA_ERR_UNSUPPORTED (-2)  /* head_dim / GQA group / page size outside the built kernels */
#define VA_ERR_CAPACITY (-3)     /* plan larger than the scratch or table capacity given       */
#define VA_ERR_LAUNCH (-4)       /* CUDA launch error (see va_last_cuda_error)                 */

#define VA_DEV_BAD_PAGE 1        /* page index outside [0, num_pages)   */
#define VA_DEV_BAD_ROW 2         /* query row / partial slot out of range */
#define VA_DEV_WAIT_EXPIRED 3    /* a bounded device-side wait gave up  */

typedef void* va_stream_t; /* cudaStream_t */

/* Library / device facts ------------------------------------------------------------------ */

/* ABI version of this header (bumped on any struct change). */
int va_abi_version(void);
/* Text of the last CUDA error seen by this library on the calling thread ("" if none). */
const char* va_last_cuda_error(void);
/* Number of SMs of the current device (the planners size their work lists from it). */
int va_sm_count(void);

/* Geometry shared by the attention entry points --------------------------------------------- */

typedef struct VaPool {
  void* k;              /* bf16 [num_slots, num_kv_heads, head_dim] of ONE layer             */
  void* v;              /* same shape; slot = page * page_size + offset                      */
  int64_t num_slots;    /* num_pages * page_size (incl. the dummy page)                      */
  int32_t page_size;
  int32_t num_q_heads;
  int32_t num_kv_heads;
  int32_t head_dim;     /* 128 or 256                                                        */
  int32_t rotary_dim;   /* <= head_dim, even; dims beyond it pass through unrotated          */
  int32_t max_pos;      /* rows of cos_sin                                                   */
  const float* cos_sin; /* fp32 [max_pos, rotary_dim]: cos in the first half, sin in the 2nd */
  float sm_scale;       /* 1/sqrt(head_dim) unless the caller says otherwise                 */
} VaPool;

/* 1. Rotate-and-store of new keys/values ---------------------------------------------------
 * Replaces: SharedCacheAttention.forward lines shared_cache/attention.py:645-649
 * (`_rope(k, positions)` then `kv_cache.store_kv`), MHAKVCache.store_kv kvcache/mha_pool.py:45-56
 * and the scatter kernel kernel/csrc/jit/store.cu:25-57.
 *   k, v      bf16 [n, num_kv_heads*head_dim] rows with the given row strides (elements)
 *   positions int32 [n] block-relative RoPE position of each new key, or NULL = store k as is
 *   out_loc   int32 [n] physical slot; a negative slot skips the row (graph padding)
 */
int va_store_kv(const VaPool* pool, const void* k, int64_t k_row_stride, const void* v,
                int64_t v_row_stride, const int32_t* positions, const int32_t* out_loc, int32_t n,
                int32_t* status, va_stream_t stream);

/* 2. Stand-alone RoPE delta rotation ---------------------------------------------------------
 * Replaces: apply_rope_correction shared_cache/rope_correction.py:15-54 and
 * SharedCacheAttention._rope shared_cache/attention.py:241-255 (partial rotary included).
 *   x, out  bf16 [n, heads, head_dim] contiguous (out may alias x);  delta int32 [n] signed.
 */
int va_rope_rotate(const void* x, void* out, const int32_t* delta, int32_t n, int32_t heads,
                   int32_t head_dim, int32_t rotary_dim, const float* cos_sin, int32_t max_pos,
                   va_stream_t stream);

/* 3. View decode -----------------------------------------------------------------------------
 * Replaces: the decode branch of SharedCacheAttention.forward shared_cache/attention.py:651-703
 * (query copies + rotation, per-segment FlashInfer paged decode, pad-scatter, merge_states).
 *
 * The plan is a device-resident int32 table built by the host planner (one H2D copy per step):
 *   page_indices  flat page numbers of every segment
 *   items         [num_items][VA_ITEM_WORDS]  one streamed key range of one (query row, kv head):
 *                   [0] offset of the segment's first page in page_indices
 *                   [1] first token, counted from the start of that first page
 *                   [2] number of keys
 *                   [3] query row (worker)          [4] signed RoPE delta of the query
 *                   [5] partial slot to write       [6] kv head      [7] reserved (0)
 *   lane_off      [num_lanes+1]  items[lane_off[i]:lane_off[i+1]] is the run of lane i;
 *                 num_lanes is a multiple of va_decode_lane_width(head_dim), at most
 *                 va_decode_lanes(head_dim)
 *   row_part_off  [num_rows*num_kv_heads+1]  the partial slots of (query row r, kv head h) are
 *                 row_part_off[r*num_kv_heads+h] : row_part_off[r*num_kv_heads+h+1]
 * Scratch (G = num_q_heads/num_kv_heads, one GQA group per partial):
 *          partial_o fp32 [num_partials, G, head_dim]  unnormalised output,
 *          partial_ml fp32 [num_partials, G, 2]        running max (log2 units) and running sum.
 */
#define VA_ITEM_WORDS 8
#define VA_PHASE_SKIP_STREAM 1 /* do not launch the streaming (partials) pass */
#define VA_PHASE_SKIP_MERGE 2  /* do not launch the merge pass                */
#define VA_PHASE_SKIP_GROUPS 4 /* do not launch the dense tiles of `groups`  */
#define VA_PHASE_GROUPS_FORKED 8 /* va_view_decode_fork_groups launched the dense tiles of `groups` earlier on this
                                    stream: join them before the merge pass, do not launch them again */

struct VaDensePlan; /* section 4 */

typedef struct VaDecodePlan {
  const int32_t* page_indices;
  const int32_t* items;
  const int32_t* lane_off;
  const int32_t* row_part_off;
  int32_t num_items;
  int32_t num_lanes;
  int32_t num_rows;
  int32_t num_partials;
  int32_t num_page_indices;
  int32_t phase_mask; /* 0 = whole step; VA_PHASE_* bits leave a pass out (per-kernel timing) */
  /* Optional: key ranges read by many query rows at once (a block shared by several requests),
   * planned as dense tiles in partial mode (section 4).  They run concurrently with the streaming
   * pass on an internal side stream that forks from / joins `stream` through events (capturable
   * in a CUDA graph); their partial slots share the scratch below and are merged with the rest.
   * num_lanes may then be smaller than va_decode_lanes() (a multiple of the warps per CTA), so
   * that the tiles find free SMs. */
  const struct VaDensePlan* groups;
} VaDecodePlan;

/* Largest number of independent streaming lanes (warps) the decode kernel runs for this
 * head_dim on the current device (SM count x lanes per CTA), and the lanes per CTA. */
int va_decode_lanes(int32_t head_dim);
int va_decode_lane_width(int32_t head_dim);

/*   q    bf16 [num_rows, num_q_heads*head_dim] UNROTATED, row stride in elements
 *   out  bf16 [num_rows, num_q_heads*head_dim]
 */
int va_view_decode(const VaPool* pool, const VaDecodePlan* plan, const void* q,
                   int64_t q_row_stride, void* out, int64_t out_row_stride, float* partial_o,
                   float* partial_ml, int32_t* status, va_stream_t stream);

/* The dense tiles of a decode step ahead of the rest.  The tiles of blocks that many requests read
 * do not depend on this step's new keys unless one of those blocks is written in the step (the
 * caller knows: a write target that is also a grouped block).  When they do not, the caller may
 * launch them BEFORE it stores the new keys:
 *     va_view_decode_fork_groups(...)   tiles forked from `stream` onto the library's side stream
 *     va_store_kv(...)                  on `stream`
 *     va_view_decode(...)               same plan with VA_PHASE_GROUPS_FORKED in phase_mask: the streaming
 *                                       pass becomes resident under the store kernel (programmatic
 *                                       dependent launch), the tiles are joined before the merge pass
 * The reference has no counterpart (it runs its per-segment FlashInfer calls in order,
 * shared_cache/attention.py:624-703); this only reorders launches of the same step. */
int va_view_decode_fork_groups(const VaPool* pool, const VaDecodePlan* plan, const void* q, int64_t q_row_stride,
                               float* partial_o, float* partial_ml, int32_t* status, va_stream_t stream);

/* 4. Dense-tile view attention ----------------------------------------------------------------
 * Replaces: SharedCacheAttention._forward_prefill_batch shared_cache/attention.py:705-752 (the
 * per-(token, segment) query copies, the two FlashInfer paged-prefill calls and merge_states), and
 * serves the decode of blocks shared by many requests (shared_cache/attention.py:651-703).
 *
 * A TILE is up to 128/G query entries (G = num_q_heads/num_kv_heads) of one kv head walking a
 * list of SEGMENTS.  Tables (device int32):
 *   tiles    [num_tiles][8]    {entry_begin, entry_count, seg_begin, seg_count, kv_head, mode, q_key, 0}
 *                              mode 0: write final bf16 rows to out[entry.q_row]
 *                              mode 1: write split-K partials to slot entry.part (layout of
 *                                      va_view_decode's scratch; merged by va_view_decode)
 *                              q_key   0, or a caller-chosen id promising that every single-segment
 *                                      tile carrying the same id has the same entries' (q_row, rel),
 *                                      kv_head and segment loc_base: a CTA that runs two such tiles
 *                                      back to back (CTA c runs tiles c, c + num_ctas, ...) keeps
 *                                      the rotated queries it staged for the first one
 *   entries  [num_entries][4]  {q_row, rel, part, 0}
 *   segments [num_segments][8] {page_off, tok_begin, n_keys, loc_base, causal_base, 0, 0, 0}
 *                              the query of an entry is rotated by rel + loc_base; with
 *                              causal_base >= 0 the entry sees keys [0, causal_base + rel] only
 *                              (end-aligned causal mask of the self segment), else all n_keys.
 */
typedef struct VaDensePlan {
  const int32_t* page_indices;
  const int32_t* tiles;
  const int32_t* entries;
  const int32_t* segments;
  int32_t num_page_indices;
  int32_t num_tiles;
  int32_t num_entries;
  int32_t num_segments;
  int32_t num_partials;
  int32_t num_rows; /* rows of q / out */
  int32_t num_ctas; /* > 0: run this many persistent CTAs, CTA c takes tiles c, c+num_ctas, ... */
  int32_t engine;   /* VA_DENSE_ENGINE_*: which tensor-core path runs the tiles                 */
  /* Optional interleaved-mRoPE query positions (shared_cache/attention.py:118-127,516-537): device
   * int32 [3, num_rows], the (time, height, width) position of every query row, used instead of
   * entry.rel for the rotation (entry.rel stays the token index of the causal mask); rotary
   * frequency f reads axis 1 when f % 3 == 1 and f < mrope_lim_h, axis 2 when f % 3 == 2 and
   * f < mrope_lim_w, else axis 0.  NULL = entry.rel on every axis.  tcgen05 engine only. */
  const int32_t* q_pos3;
  int32_t mrope_lim_h;
  int32_t mrope_lim_w;
} VaDensePlan;

#define VA_DENSE_ENGINE_MMA_SYNC 0 /* warp-level mma.sync, operands through registers           */
#define VA_DENSE_ENGINE_TCGEN05 1  /* tcgen05.mma from one thread, accumulators in TMEM         */

int va_view_dense(const VaPool* pool, const VaDensePlan* plan, const void* q, int64_t q_row_stride,
                  void* out, int64_t out_row_stride, float* partial_o, float* partial_ml,
                  int32_t* status, va_stream_t stream);

/* 5. Gated DeltaNet over an ordered block list ---------------------------------------------
 * Block summaries are fp32 tensors in block convention, one per (block, layer):
 *   A_hat [num_v_heads, dk, dk]   B_hat [num_v_heads, dv, dk]      S_out^T = S_in^T A_hat + B_hat
 * (shared_cache/gdn_affine.py:1-24).  Pointer tables are device int64 arrays of device addresses;
 * 0 means "this block has no summary for the layer" (skipped in a chain; identity / zero for a
 * write block).  head_k_dim = head_v_dim = 128.  q and k may carry num_k_heads < num_v_heads
 * heads (value head h reads key head h / (num_v_heads/num_k_heads)); both are L2-normalised in
 * fp32 inside the kernels (eps inside the rsqrt) and q is scaled by q_scale.
 */

/* 5a. Fused decode step.  Replaces, per GDN layer and step: compose_first/compose_level
 * (kernel/gdn_compose.py:14-97), the transposition to the model convention, the one-token
 * recurrence whose stepped state is discarded (models/qwen3_5_delta.py:124-163, :474-481) and the
 * per-token affine capture (shared_cache/gdn.py:213-269, kernel/gdn_prefill.py:53-131).
 * The new summaries go to FRESH slabs (write_a/write_b must not alias any input), so readers of
 * the previous summary are never disturbed (shared_cache/gdn_decode.py:112-121). */
/* Storage type of block summaries (shared_cache/gdn.py:40-45, state_dtype): fp32, or bf16 storage
 * with fp32 arithmetic -- values are widened when read and rounded once when a summary is stored
 * (shared_cache/gdn.py:249-269, shared_cache/gdn_affine.py:113-122). */
#define VA_SUMMARY_F32 0
#define VA_SUMMARY_BF16 1

typedef struct VaGdnStep {
  const void* q;            /* bf16 [W, num_k_heads, 128]                         */
  const void* k;            /* bf16 [W, num_k_heads, 128]                         */
  const void* v;            /* bf16 [W, num_v_heads, 128]                         */
  const float* g;           /* fp32 [W, num_v_heads] log decay (alpha = exp g)    */
  const float* beta;        /* fp32 [W, num_v_heads]                              */
  void* out;                /* bf16 [W, num_v_heads, 128]                         */
  const int64_t* chain_a;   /* [W, depth] A_hat of each view block, view order    */
  const int64_t* chain_b;   /* [W, depth] B_hat                                   */
  const int64_t* read_a;    /* [W] write block's current A_hat (0 = identity)     */
  const int64_t* read_b;    /* [W] write block's current B_hat (0 = zero)         */
  const int64_t* write_a;   /* [W] fresh A_hat slab                               */
  const int64_t* write_b;   /* [W] fresh B_hat slab                               */
  int32_t num_workers;
  int32_t depth;
  int32_t num_k_heads;
  int32_t num_v_heads;
  int32_t head_k_dim;
  int32_t head_v_dim;
  float l2_eps;
  float q_scale;
  int32_t* status;
  /* elements between consecutive workers' rows of q / k / v (they may lie inside the wider
   * [q | k | v] rows a layer's conv step wrote); 0 = dense */
  int64_t q_row_stride;
  int64_t k_row_stride;
  int64_t v_row_stride;
  int32_t summary_dtype;    /* VA_SUMMARY_*: storage type of every A_hat / B_hat named above */
} VaGdnStep;

int va_gdn_step(const VaGdnStep* args, va_stream_t stream);

/* 5b. Initial recurrent state of each worker from its chain:
 * state[w, h] = (fold of the chain)^T as [dk, dv], zeros if no block has a summary.
 * Replaces SharedCacheGDN.compose_initial_recurrent_state shared_cache/gdn.py:127-180 and
 * GDNDecodeBuffers.compose shared_cache/gdn_decode.py:190-203. */
int va_gdn_compose(const int64_t* chain_a, const int64_t* chain_b, float* state, int32_t num_workers,
                   int32_t depth, int32_t num_heads, int32_t head_k_dim, int32_t head_v_dim,
                   int32_t summary_dtype, va_stream_t stream);

/* 5c. Prefill scan of a batch of requests (tokens request-major, request r owns rows
 * seg_off[r]:seg_off[r+1]): the gated delta rule from state0, the output rows, and the write
 * block's new summary from one joint pass over [S | A_hat | B_hat].  Replaces
 * chunk_gated_delta_rule + capture (models/qwen3_5_delta.py:41-121, :349-441) and the joint
 * pass of GDNPrefillBuffers.core_and_capture shared_cache/gdn_prefill.py:63-85. */
typedef struct VaGdnPrefill {
  const void* q;            /* bf16 [N, num_k_heads, 128]; q, k, v 16-byte aligned for the CHUNK engines */
  const void* k;
  const void* v;            /* bf16 [N, num_v_heads, 128]                          */
  const float* g;           /* fp32 [N, num_v_heads]                               */
  const float* beta;
  void* out;                /* bf16 [N, num_v_heads, 128]                          */
  const int32_t* seg_off;   /* [R+1]                                               */
  const float* state0;      /* fp32 [R, num_v_heads, dk, dv] or NULL (zeros)       */
  const int64_t* init_a;    /* [R] write block's previous A_hat (0 = identity)     */
  const int64_t* init_b;    /* [R] previous B_hat (0 = zero)                       */
  const int64_t* write_a;   /* [R] new A_hat slab (0 = not wanted)                 */
  const int64_t* write_b;
  float* final_state;       /* fp32 [R, num_v_heads, dk, dv] or NULL               */
  int32_t num_requests;
  int32_t num_k_heads;
  int32_t num_v_heads;
  int32_t head_k_dim;
  int32_t head_v_dim;
  float l2_eps;
  float q_scale;
  int32_t engine;           /* VA_GDN_ENGINE_*                                     */
  /* Scratch of the CHUNK engine (device memory of the caller, 16-byte aligned, at least
   * va_gdn_prefill_scratch_bytes(num_tokens, num_v_heads)): the state-independent half of every
   * chunk (normalised K and Q, W, U, the causal score tile, the decays) is computed once, all
   * chunks in parallel, and parked there before the three states are walked in order.
   * Required by VA_GDN_ENGINE_CHUNK and VA_GDN_ENGINE_CHUNK_TC, ignored by VA_GDN_ENGINE_SCAN. */
  int32_t max_segment_tokens; /* longest request, 0 = unknown (num_tokens is used)  */
  void* scratch;
  int64_t scratch_bytes;
  int64_t num_tokens;       /* N (rows of q/k/v); needed with scratch              */
  int32_t summary_dtype;    /* VA_SUMMARY_*: storage type of init_a/b and write_a/b */
  int32_t* status;          /* device word for VA_DEV_* findings (a bounded wait of the CHUNK_TC
                               engine that ran out), or NULL                                       */
} VaGdnPrefill;

/* SCAN: token by token in fp32 (exact restatement of the recurrence, state in registers).
 * CHUNK: 64 tokens at a time on the tensor cores (UT transform of _chunk_gated_delta_rule,
 * models/qwen3_5_delta.py:85-114): bf16 operands, fp32 accumulation and fp32 state; mma.sync.
 * CHUNK_TC: the same chunk pre-pass, the state walked with tcgen05 products (state resident in
 * TMEM, transposed so that the 128 feature rows are the M dimension). */
#define VA_GDN_ENGINE_SCAN 0
#define VA_GDN_ENGINE_CHUNK 1
#define VA_GDN_ENGINE_CHUNK_TC 2

int64_t va_gdn_prefill_scratch_bytes(int64_t num_tokens, int32_t num_v_heads);
int va_gdn_prefill(const VaGdnPrefill* args, va_stream_t stream);

/* 6. View decode without caller-supplied scratch ------------------------------------------------
 * No counterpart in the reference.  Same step as va_view_decode, for callers that cannot allocate
 * device memory (a process that gave all free HBM to its KV pool at start-up; a host without a
 * device allocator): the split-K scratch is a fixed array inside the library, present on every GPU
 * that loads it.  Limits: num_partials * G * head_dim <= 2048*8*256 floats and num_partials * G <=
 * 2048*8 (G = num_q_heads/num_kv_heads; num_partials = the larger of the plan's and its `groups`'),
 * else VA_ERR_CAPACITY; every argument check of va_view_decode runs before the first launch, so a
 * refused call launches nothing.  The first
 * call on a device looks up the array's device address and should be made outside stream capture.
 * All calls on one GPU share the array: calls that may overlap on the GPU race; calls queued on one
 * stream do not.  The array keeps the previous call's contents and needs no clearing (every slot a
 * plan names is written before it is read).  Dense tiles of `plan->groups` run on `stream` itself. */
int va_view_decode_static(const VaPool* pool, const VaDecodePlan* plan, const void* q,
                          int64_t q_row_stride, void* out, int64_t out_row_stride, int32_t* status,
                          va_stream_t stream);

/* 7. Host planner of the decode step -------------------------------------------------------------
 * Replaces: the table building of SharedCacheAttention.prepare shared_cache/attention.py:282-448
 * (indptr / indices / last_page_len per wrapper), for the work list of section 3 and the shared-block
 * tiles of section 4.  Host code only: no CUDA call is made and no GPU is needed.
 *
 * Input: the step's sub-requests in reference order (one per (worker, non-empty block of its view),
 * then the implicit-self ones), each as
 *   sub_worker   query row           sub_loc      signed RoPE distance of the query to the block
 *   sub_len      keys (post-append)  sub_page_off offset of the block's first page in `pages`
 *   sub_tok0     first token inside that first page
 *   sub_key      >= 0: identity of the block (equal for every reader of one block); < 0: private
 * and `pages`, the flat page numbers.  Blocks read by at least group_min_readers sub-requests and
 * at least group_min_keys long become dense tiles in partial mode; the SMs are split between the
 * streaming lanes and the tiles by the modelled cost (keys / rate) of either side.
 *
 * Output: one int32 blob [pages | items | lane_off | row_part_off | tiles | entries | segments],
 * every section starting on a multiple of 4 words, described by VaPlanLayout (offsets in words).
 * The layout is always filled in; when blob_words < layout->total_words nothing is written to
 * `blob` and VA_ERR_CAPACITY is returned, so a caller can size the blob from a first call.
 * Copy the blob to the device and point VaDecodePlan / VaDensePlan at its sections. */
typedef struct VaPlanParams {
  int32_t num_workers;
  int32_t num_kv_heads;
  int32_t readers_per_tile;    /* query entries of one dense tile: 128 / (num_q_heads/num_kv_heads) */
  int32_t num_sms;             /* SMs the step may use                                             */
  int32_t lane_width;          /* va_decode_lane_width(head_dim)                                   */
  int32_t group_min_readers;   /* 0: never plan dense tiles                                        */
  int32_t group_min_keys;
  int32_t dense_tiles_per_cta; /* key chunks are sized so that every dense CTA runs this many tiles */
  int32_t min_item_keys;       /* a lane's quota never drops below this many keys                  */
  int32_t cut_slack_keys;      /* a lane cut this close to a segment boundary moves onto it        */
  int32_t fixed_stream_lanes;  /* > 0: the lane count is frozen (captured graph)                   */
  int32_t fixed_dense_sms;     /* with fixed_stream_lanes > 0: frozen dense CTA count, 0 = no tiles */
  double stream_rate;          /* keys per microsecond of one (reader, kv head) unit on one SM     */
  double dense_rate;           /* keys per microsecond of one (reader group, kv head) tile row     */
} VaPlanParams;

typedef struct VaPlanLayout {
  int64_t total_words;
  int64_t quota;      /* keys per streaming lane   */
  int64_t total_keys; /* keys streamed by the lanes */
  int32_t off_pages, num_pages;
  int32_t off_items, num_items;
  int32_t off_lane_off, num_lanes;
  int32_t off_row_part_off, num_groups; /* num_workers * num_kv_heads (+1 offsets) */
  int32_t off_tiles, num_tiles;
  int32_t off_entries, num_entries;
  int32_t off_segments, num_segments;
  int32_t num_partials;
  int32_t dense_sms; /* CTAs of the dense tiles (VaDensePlan.num_ctas), 0 = no tiles */
} VaPlanLayout;

int va_plan_decode(const VaPlanParams* params, int32_t num_subs, const int32_t* sub_worker,
                   const int32_t* sub_loc, const int32_t* sub_len, const int32_t* sub_page_off,
                   const int32_t* sub_tok0, const int32_t* sub_key, const int32_t* pages,
                   int32_t num_pages, int32_t* blob, int64_t blob_words, VaPlanLayout* layout);

/* The same step described by its views, as the serving engine holds it: the distinct blocks with
 * their post-append token count and span, every worker's view as a list of block indices, and the
 * workers whose write block is outside their view.  Expands the views into sub-requests with the
 * reference's rules -- an empty block is skipped; the query's distance to a block is the span from
 * the block's start to the end of the view, minus one; a write block outside the view is one key
 * at the new token's slot (shared_cache/attention.py:282-368) -- and schedules them as
 * va_plan_decode does.  `pages` holds the blocks' page runs back to back (block_pages[b] pages of
 * block b); a page allocated for this step's token (block_pending_page[b] >= 0) is appended to its
 * block's run and the implicit-self pages after all runs by the planner, so the page section of
 * the blob is the step's complete page pool.
 * sub_out (optional) receives five rows of `sub_stride` words, sub_stride >= view_start[W] +
 * num_aux: worker, loc, segment index within the worker, length, block (-1 for implicit self) of
 * every sub-request, paged ones first (worker-major), then the implicit-self ones. */
typedef struct VaViewStep {
  int32_t num_workers;
  int32_t num_blocks;
  int32_t num_aux;
  int32_t page_size;
  const int32_t* view_start;     /* [num_workers + 1] */
  const int32_t* view_block;     /* [view_start[num_workers]] */
  const int32_t* block_len;      /* [num_blocks] tokens after this step's append         */
  const int32_t* block_span;     /* [num_blocks] position span after this step's append  */
  const int32_t* block_pages;        /* [num_blocks] pages the block holds before this step    */
  const int32_t* block_pending_page; /* [num_blocks] page allocated for this step, -1 = none; may be NULL */
  const int32_t* pages;              /* [sum of block_pages] page numbers                      */
  const int32_t* aux_worker;     /* [num_aux] */
  const int32_t* aux_loc;        /* [num_aux] span of the write block                    */
  const int64_t* aux_slot;       /* [num_aux] token slot of the new key                  */
} VaViewStep;

typedef struct VaViewSubs {
  int32_t num_main;     /* paged sub-requests                    */
  int32_t num_aux;      /* implicit-self sub-requests            */
  int32_t max_segments; /* most segments any worker's query sees */
} VaViewSubs;

int va_plan_views(const VaPlanParams* params, const VaViewStep* step, int32_t* blob, int64_t blob_words,
                  VaPlanLayout* layout, int32_t* sub_out, int64_t sub_stride, VaViewSubs* subs_info);

/* Tile table of a batched view-conditioned prefill (host code).  Replaces the per-request tile
 * bookkeeping of SharedCacheAttention.prepare_prefill_batch (shared_cache/attention.py:450-622 builds
 * one FlashInfer plan per context depth instead).  `requests` holds (seg_begin, seg_count,
 * row_offset, num_new) per request, `segments` the 8-word segment rows of VaDensePlan.  Writes
 * `entries` ([num_rows, 4]: row, relative position) and `tiles` ([*num_tiles_out, 8]: entry_begin,
 * entry_count, seg_begin, seg_count, kv head): tiles of per_tile consecutive new tokens per
 * (request, kv head), heaviest first (keys walked x rows; stable), every other round of
 * min(max_ctas, tiles) rows reversed.  VA_ERR_CAPACITY (with *num_tiles_out set) if tile_capacity is
 * too small. */
int va_plan_prefill_tiles(const int32_t* segments, int32_t num_segments, const int32_t* requests,
                          int32_t num_requests, int32_t per_tile, int32_t num_kv_heads, int32_t max_ctas,
                          int32_t* entries, int32_t num_rows, int32_t* tiles, int32_t tile_capacity,
                          int32_t* num_tiles_out);

/* Address tables of a GDN forward over the views (host code, no CUDA call).  Replaces the pointer
 * tables GDNDecodeBuffers.prepare assembles per chain level (shared_cache/gdn_decode.py:62-167:
 * prefix_links / terminal_sinks over the chains, then per-layer pointer lists) and the
 * "most recent conv window along the reversed chain" rule of SharedCacheGDN.prior_conv_states
 * (shared_cache/gdn.py:182-207).  The caller numbers the distinct blocks of the step (row 0 = no
 * block) and hands over their per-layer addresses:
 *   block_addr [num_blocks + 1, layers, 2]  (A_hat, B_hat) of a block's summary, 0 = none
 *   block_conv [num_blocks + 1, layers]     conv window, 0 = none; NULL = no conv / write rows
 *   chain_idx  [workers, depth]             rows of block_addr in view order, 0 past the chain's end
 *   target_idx [workers]                    row of each worker's write block
 *   write_*_base [workers] + layer * write_*_stride (bytes): the fresh slabs of a worker's layers
 * and gets `tab` [8, layers, workers, depth] int64, zero-filled and then: row 0 / 1 = chain A_hat /
 * B_hat per view position; rows 2..7 (read a, read b, conv read, write a, write b, conv write) in
 * [..., 0].  Conv read = the window of the LAST block of the chain that has one, per layer. */
int va_gdn_plan_tables(const int64_t* block_addr, const int64_t* block_conv, const int32_t* chain_idx,
                       const int32_t* target_idx, const int64_t* write_a_base, int64_t write_a_stride,
                       const int64_t* write_b_base, int64_t write_b_stride, const int64_t* conv_write_base,
                       int64_t conv_write_stride, int32_t num_blocks, int32_t layers, int32_t workers,
                       int32_t depth, int64_t* tab);

/* 8. Block merge / append ------------------------------------------------------------------------
 * Replaces: SharedCacheSession._copy_slots + _shift_keys_ (shared_cache/session.py:489-528), which
 * loop over the layers in Python (index_select / index_copy_ per layer for K and V, then
 * index_select + fp32 rotation + index_copy_ for the keys of the right-hand block).
 * One launch for all layers: token i's K and V rows move from slot src_slots[i] to dst_slots[i]
 * (device int32 arrays) in every layer; the keys of tokens [shift_begin, n) are rotated by `shift`
 * positions on the way (stored bf16 widened to fp32, rotated, rounded once: the reference's
 * arithmetic).  `pool` describes layer 0; layer l starts layer_stride elements further in both the
 * K and the V pool.  The source and destination slot sets must be disjoint. */
int va_block_copy(const VaPool* pool, int32_t num_layers, int64_t layer_stride, const int32_t* src_slots,
                  const int32_t* dst_slots, int32_t n, int32_t shift_begin, int32_t shift,
                  int32_t* status, va_stream_t stream);

/* Replaces: the per-layer compose_gdn_affines calls of _finish_block_merge
 * (shared_cache/session.py:441-462; shared_cache/gdn_affine.py:104-127).  For every pair i:
 *   out_a[i] = a_first[i] a_second[i]          out_b[i] = b_first[i] a_second[i] + b_second[i]
 * per head, fp32 sums.  The six arguments are device int64 arrays of device addresses of
 * [num_v_heads, 128, 128] tensors of the storage type summary_dtype (VA_SUMMARY_*; bf16 results are
 * rounded once, after the fp32 add: shared_cache/gdn_affine.py:113-122); outputs must not alias
 * inputs. */
int va_gdn_compose_pairs(const int64_t* a_first, const int64_t* b_first, const int64_t* a_second,
                         const int64_t* b_second, const int64_t* out_a, const int64_t* out_b,
                         int32_t num_pairs, int32_t num_v_heads, int32_t head_k_dim, int32_t head_v_dim,
                         int32_t summary_dtype, va_stream_t stream);

/* 9. Interleaved 3-axis mRoPE ----------------------------------------------------------------------
 * Replaces: SharedCacheAttention._rope_mrope shared_cache/attention.py:257-280 and, for the store
 * form, the mRoPE branch of forward (shared_cache/attention.py:645-649 with batch.mrope_positions).
 *   pos       int32 [pos_axes, n]: pos_axes 1 = the same position on all three axes (text tokens),
 *             3 = (time, height, width) rows
 *   lim_h, lim_w  3 * mrope_section[1], 3 * mrope_section[2]: rotary frequency f reads the height
 *             axis when f % 3 == 1 and f < lim_h, the width axis when f % 3 == 2 and f < lim_w,
 *             else the time axis
 *   cos_sin   fp32 [max_pos, rotary_dim], row p = cos | sin of p * inv_freq
 * Arithmetic is the reference's bf16 tensor arithmetic (cos, sin, both products and the sum each
 * rounded to bf16).  va_mrope_rotate: x, out bf16 [n, heads, head_dim] contiguous, out may alias x.
 * va_store_kv_mrope: like va_store_kv, keys rotated this way on their way into the pool. */
int va_mrope_rotate(const void* x, void* out, const int32_t* pos, int32_t pos_axes, int32_t n,
                    int32_t heads, int32_t head_dim, int32_t rotary_dim, const float* cos_sin,
                    int32_t max_pos, int32_t lim_h, int32_t lim_w, va_stream_t stream);
int va_store_kv_mrope(const VaPool* pool, const void* k, int64_t k_row_stride, const void* v,
                      int64_t v_row_stride, const int32_t* pos, int32_t pos_axes, const int32_t* out_loc,
                      int32_t n, int32_t lim_h, int32_t lim_w, int32_t* status, va_stream_t stream);

/* 10. GDN layer steps around the recurrent core (decode) --------------------------------------
 * va_gdn_decode_pre replaces, in Qwen3_5GatedDeltaNet._forward_ar_decode
 * (models/qwen3_5_delta.py:453-461), the conv-window concatenation, the new conv state slice,
 * _decode_conv_silu (:232-245) and _gates (:296-299) -- one launch instead of about twenty.
 *   qkv        bf16 [W, conv_dim] rows (row stride in elements): this step's projections
 *   prior_conv bf16 [W, conv_dim, k] previous conv state, or NULL for zeros
 *   conv_weight bf16 [conv_dim, k];  a, b bf16 [W, Hv];  a_log, dt_bias fp32 [Hv]
 *   qkv_out    bf16 [W, conv_dim]  SiLU(sum_t window[t] * weight[t]), fp32 products and sum
 *   conv_out   bf16 [W, conv_dim, k]  the last k entries of [prior | qkv]
 *   beta_out   bf16 [W, Hv] sigmoid(b);  g_out fp32 [W, Hv] = -exp(a_log) * softplus(a + dt_bias)
 *   beta_f32_out  optional fp32 [W, Hv]: beta_out widened, the form va_gdn_step reads
 *   prior_conv_ptrs / conv_out_ptrs  optional device int64 [W]: the states as separate [conv_dim, k]
 *                 tensors named by address (0 = zeros for a prior state, 0 = do not write the new
 *                 state: a padding row of a fixed-capacity batch) instead of the dense arrays --
 *                 the blocks' own tensors, so that no gather / scatter launch is needed
 *                 (replaces gather_rows / scatter_rows of shared_cache/gdn_decode.py) */
typedef struct VaGdnDecodePre {
  const void* qkv;
  int64_t qkv_row_stride;
  const void* prior_conv;
  const void* conv_weight;
  const void* a;
  const void* b;
  const float* a_log;
  const float* dt_bias;
  void* qkv_out;
  void* conv_out;
  void* beta_out;
  float* g_out;
  float* beta_f32_out;
  const int64_t* prior_conv_ptrs;
  const int64_t* conv_out_ptrs;
  int32_t num_workers;
  int32_t conv_dim;
  int32_t conv_kernel; /* 1..8 */
  int32_t num_v_heads;
  int64_t a_row_stride; /* elements between workers' rows of a / b (columns of a wider      */
  int64_t b_row_stride; /* projection output are read in place); 0 = num_v_heads            */
} VaGdnDecodePre;

int va_gdn_decode_pre(const VaGdnDecodePre* args, va_stream_t stream);

/* Replaces _GatedRMSNorm.forward (models/qwen3_5_delta.py:248-263):
 *   out = bf16(weight * x * rsqrt(mean(x^2) + eps) * silu(gate)), fp32 inside.
 *   x, out bf16 [rows, dim] contiguous; weight fp32 [dim]; dim a multiple of 32, <= 1024.
 *   gate bf16: row r lies at gate + (r / rows_per_token) * gate_token_stride + (r % rows_per_token) * dim
 *   (the z columns of a wider projection output are read in place); rows_per_token <= 0 = dense rows. */
int va_gdn_gated_rmsnorm(const void* x, const void* gate, const float* weight, void* out, int64_t rows,
                         int32_t dim, float eps, int32_t rows_per_token, int64_t gate_token_stride,
                         va_stream_t stream);

/* Replaces, per request of a GDN prefill (Qwen3_5GatedDeltaNet._forward_ar_prefill_one,
 * models/qwen3_5_delta.py:399-419), the transpose / concatenation with the prior conv tail,
 * _prefill_conv_silu (:215-229: products rounded to bf16, fp32 sum and SiLU) and the new conv
 * state -- all requests of the batch in one launch.
 *   qkv       bf16 [T, conv_dim] rows of all requests, request r = rows seg_off[r] : seg_off[r+1]
 *   prior_conv bf16 [R, conv_dim, k] or NULL (zeros);  conv_weight bf16 [conv_dim, k]
 *   seg_off   device int32 [R + 1]; a request with an empty range is skipped, tokens beyond
 *             seg_off[R] are left alone (padding of a fixed-capacity batch)
 *   qkv_out   bf16 [T, conv_dim];  conv_out bf16 [R, conv_dim, k] = last k of [prior | inputs]
 *   prior_conv_ptrs / conv_out_ptrs  optional device int64 [R]: the states as separate [conv_dim, k]
 *             tensors named by address (0 = zeros for a prior state, 0 = do not write the new state)
 *             instead of the dense arrays, as in VaGdnDecodePre */
typedef struct VaGdnPrefillConv {
  const void* qkv;
  int64_t qkv_row_stride;
  const void* prior_conv;
  const void* conv_weight;
  const int32_t* seg_off;
  void* qkv_out;
  void* conv_out;
  const int64_t* prior_conv_ptrs;
  const int64_t* conv_out_ptrs;
  int32_t num_requests;
  int32_t num_tokens;
  int32_t conv_dim;
  int32_t conv_kernel; /* 1..8 */
} VaGdnPrefillConv;

int va_gdn_prefill_conv(const VaGdnPrefillConv* args, va_stream_t stream);

/* 11. Gated full-attention layer steps around the view attention ---------------------------------
 * The fused qkv projection of the reference's gated attention layer writes rows
 *   [ head 0: q | gate ] ... [ head Hq-1: q | gate ] [ k heads ] [ v heads ]       (2*Hq + 2*Hkv) * D wide
 * (models/qwen3_5_attn.py:47-52,103-109).
 * va_attn_qk_norm replaces the q / gate split copies and the two per-head RMSNorm calls
 * (models/qwen3_5_attn.py:105-114; layers/norm.py:8-22, FlashInfer's `gemma_rmsnorm` when
 * weight_plus_one, else `rmsnorm`): q_out [n, Hq*D] and k_out [n, Hkv*D] bf16 =
 *   x * rsqrt(mean(x^2) + eps) * (weight + (weight_plus_one ? 1 : 0)), fp32 inside, one rounding.
 * gate and v are read where they lie by the later steps (no copy).  head_dim 128 or 256.
 * va_attn_output_gate replaces _sigmoid_output_gate (models/qwen3_5_attn.py:21-23,136):
 *   out = bf16(float(o) * sigmoid(float(gate))), gate read in place from the projection rows. */
typedef struct VaAttnQkNorm {
  const void* qkv;        /* bf16 rows, row stride in elements (multiple of 8)  */
  int64_t qkv_row_stride;
  const float* q_weight;  /* fp32 [head_dim]                                     */
  const float* k_weight;  /* fp32 [head_dim]                                     */
  void* q_out;            /* bf16 [n, num_q_heads * head_dim]                    */
  void* k_out;            /* bf16 [n, num_kv_heads * head_dim]                   */
  int32_t n;
  int32_t num_q_heads;
  int32_t num_kv_heads;
  int32_t head_dim;
  float eps;
  int32_t weight_plus_one;
} VaAttnQkNorm;

int va_attn_qk_norm(const VaAttnQkNorm* args, va_stream_t stream);
int va_attn_output_gate(const void* o, const void* qkv, int64_t qkv_row_stride, void* out, int32_t n,
                        int32_t num_q_heads, int32_t head_dim, va_stream_t stream);

/* 12. Decoder-layer glue (used by the full-model workload) ------------------------------------------
 * va_add_rmsnorm replaces RMSNormFused.forward (layers/norm.py:25-43; FlashInfer
 * `fused_add_rmsnorm` / `gemma_fused_add_rmsnorm`): residual <- residual + delta (fp32 sum, stored as
 * bf16, in place), out <- sum * rsqrt(mean(sum^2) + eps) * (weight + (weight_plus_one ? 1 : 0)), one
 * rounding.  delta NULL: no add (RMSNorm.forward, layers/norm.py:8-22).  All rows bf16 [n, dim]
 * contiguous, weight bf16 [dim], dim a multiple of 8, at most 16384, 16-byte aligned pointers.
 * va_silu_mul replaces silu_and_mul (layers/activation.py:9-12): out[n, inter] =
 * bf16(silu(gate) * up), gate = columns [0, inter) and up = columns [inter, 2 inter) of rows
 * row_stride elements apart; fp32 inside. */
int va_add_rmsnorm(void* residual, const void* delta, const void* weight, void* out, int32_t n, int32_t dim,
                   float eps, int32_t weight_plus_one, va_stream_t stream);
int va_silu_mul(const void* gate_up, int64_t row_stride, void* out, int32_t n, int32_t inter, va_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* VIEW_ATTN_B200_H_ */

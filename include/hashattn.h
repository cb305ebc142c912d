/*
 * hashattn.h — C ABI of libhashattn.so: the HashAttention sparse-decode hot path for
 * NVIDIA B200 (sm_100a).
 *
 * The library replaces, for one attention layer and one decode step, what the reference
 * does in torch inside hashattention/hashattention_llama.py:
 *     USA.forward / k_embedding / q_embedding      (:151-226)  -> ha_hash_decode, ha_hash_prefill
 *     compute_mask_multi, usa_eval_mode == 'simple' (:401-446)  -> ha_score_select
 *     masked softmax(QK^T/sqrt(d)) . V              (:578-623)  -> ha_sparse_decode
 *     the three in sequence                         (:571-623)  -> ha_decode_step
 *
 * Conventions
 *   - Every function returns an int status (HA_OK == 0) and never throws.
 *   - Unless a parameter is documented as a host pointer, every pointer is a DEVICE pointer.
 *   - Nothing is allocated or freed inside the library; temporaries live in a caller-provided
 *     workspace of ha_workspace_bytes() bytes that was prepared once by ha_workspace_init().
 *   - All work is ordered on the given CUDA stream; the library creates no streams or events of
 *     its own, and no entry point synchronises with the host except ha_decode_step_host
 *     (documented there).
 *   - Kernels validate page ids and sizes before touching memory; a violation is reported
 *     through the 4-byte device word `status` (0 == clean) instead of a fault.
 *
 * Data layout in HBM (all little-endian, row-major, dimension names left to right)
 *   K pages, V pages : [num_pages][num_kv_heads][page_size][head_dim]   bf16
 *   hash pages       : [num_pages][num_kv_heads][page_size][gqa_group]  u32
 *                      one 16-byte word per token per kv-head holding the packed 32-bit key
 *                      code of each of the gqa_group(=4) query heads of that kv-head.
 *                      bit i of a code == 1 iff output i of the head's hash MLP is > 0
 *                      (LSB == output 0; efficiency/kernels/torchatt.py:35-36,159).
 *   page_table       : [batch][max_pages] i32, entry p = page id of tokens [p*page_size, ...)
 *   seq_lens         : [batch] i32, number of cached tokens INCLUDING the one being decoded
 *   q, out           : [batch][num_q_heads][head_dim] bf16 (num_q_heads = num_kv_heads*gqa_group,
 *                      query head h belongs to kv-head h / gqa_group)
 *   k_new, v_new     : [batch][num_kv_heads][head_dim] bf16 (post-RoPE key of the new token)
 *   hash weights     : per side (q or k) [num_q_heads][W0 128x128 | W1 128x128 | W2 32x128]
 *                      row-major [out][in] exactly as torch.nn.Linear stores them, bf16 or f32
 *                      (HA_WEIGHTS_*), 36864 elements per head;
 *                      biases [num_q_heads][128 + 128 + 32] f32.
 */
#ifndef HASHATTN_H_
#define HASHATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HA_ABI_VERSION 5

/* status codes (return values and contents of the device status word) */
#define HA_OK 0
#define HA_ERR_BAD_ARG 1         /* null pointer, non-positive size, inconsistent shape      */
#define HA_ERR_UNSUPPORTED_DIM 2 /* head_dim != 128, gqa_group != 4, page_size != 256, ...   */
#define HA_ERR_WORKSPACE 3       /* workspace missing or smaller than ha_workspace_bytes()   */
#define HA_ERR_LAUNCH 4          /* the CUDA runtime refused a launch or a copy              */
#define HA_ERR_TIMEOUT 5         /* a bounded device-side wait ran out                       */
#define HA_ERR_BAD_PAGE 6        /* device: page id outside [0, num_pages)                   */
#define HA_ERR_BAD_SEQ_LEN 7     /* device: seq_len < 1 or beyond max_pages * page_size      */
#define HA_ERR_SEL_OVERFLOW 8    /* device: heavy budget exceeds sel_stride                  */
#define HA_ERR_SCRATCH_LIMIT 9   /* problem needs more than HA_STATIC_SCRATCH_BYTES of scratch */

#define HA_WEIGHTS_BF16 0
#define HA_WEIGHTS_F32 1
#define HA_HASH_LSH (-1) /* ha_hash_weights_t.num_layers: the LSH baseline, lth_num_layers == 0 of the reference */

/* Shape of one layer's paged cache as seen by ONE GPU (after any kv-head partitioning). */
typedef struct ha_shape {
    int32_t batch;        /* B: sequences decoded together                                   */
    int32_t num_kv_heads; /* kv heads held by this GPU                                       */
    int32_t gqa_group;    /* query heads per kv head; must be 4                              */
    int32_t head_dim;     /* must be 128                                                     */
    int32_t page_size;    /* tokens per page; must be 256                                    */
    int32_t max_pages;    /* columns of page_table                                           */
    int32_t num_pages;    /* pages in the K / V / hash pools (bound for page ids)            */
    int32_t sel_stride;   /* row pitch (elements) of sel_idx: >= largest heavy budget        */
} ha_shape_t;

/* Budgets of compute_mask_multi (hashattention/hashattention_llama.py:423-443).
 * heavy_budget <= 1.0 is a fraction of seq_len, > 1.0 an absolute token count; the product
 * is formed in double precision and truncated, as Python's int(k * heavy_budget) does.
 * eval_mode selects what is kept among the candidates:
 *   HA_EVAL_SIMPLE  usa_eval_mode == 'simple' (:436-438): the hb best, ties by lowest index.
 *   HA_EVAL_DEPTH   any other usa_eval_mode (:439-443): every candidate whose score is at least
 *                   max(best score - retrieve_depth, score of the hb-th best); a variable
 *                   number, all ties included. (One mismatching bit lowers the reference's
 *                   +-1 span by 2, hence its `2 * usa_retrieve_depth`.) hb == 0 keeps nothing
 *                   (the reference raises there). sel_stride must cover the largest set.      */
#define HA_EVAL_SIMPLE 0
#define HA_EVAL_DEPTH 1
typedef struct ha_budget {
    int32_t init_budget;   /* sink tokens  [0, init)                                          */
    int32_t recent_budget; /* recent tokens [S - recent, S)                                   */
    double heavy_budget;
    int32_t eval_mode;      /* HA_EVAL_SIMPLE or HA_EVAL_DEPTH                                */
    int32_t retrieve_depth; /* usa_retrieve_depth, only read in HA_EVAL_DEPTH; |depth| <= 64  */
} ha_budget_t;

typedef struct ha_hash_weights {
    const void* wq;    /* query-side weights, layout above                                   */
    const float* bq;   /* query-side biases                                                  */
    const void* wk;    /* key-side weights                                                   */
    const float* bk;   /* key-side biases                                                    */
    int32_t dtype;     /* HA_WEIGHTS_BF16 or HA_WEIGHTS_F32                                  */
    int32_t num_layers; /* lth_num_layers of the reference (hashattention_llama.py:99-127): 3 (or 0,
                         * meaning 3): Linear-SiLU-Linear-SiLU-Linear; 2: Linear(128,128)-SiLU-
                         * Linear(128,32), stored in the W0 and W2 slots; 1: Linear(128,32), stored in
                         * the W2 slot. Unused slots are ignored. The layout per head stays
                         * [W0 | W1 | W2] and [b0 | b1 | b2].
                         * HA_HASH_LSH: the LSH baseline (lth_num_layers == 0 there, :75-84, :130-139): one
                         * Linear(129,32) per head over [x, sqrt(relu(M^2 - |x|^2))], M = 1e-3 + the largest
                         * norm of the call; columns 0..127 of its weight in the W2 slot, column 128 in
                         * b0[0..31], its bias in b2; the key and the query side are the same function.  */
    void* lsh_state;    /* HA_HASH_LSH only, else ignored: device buffer of 2 * num_kv_heads 32-bit words that
                         * belongs to the cache - float m[num_kv_heads], the largest key norm cached per
                         * kv-head (set by ha_hash_prefill, raised by decode steps), then int32
                         * stale[num_kv_heads]. A step whose new keys raise m re-hashes that kv-head's
                         * cache, as the reference (which re-hashes every key on every step) implies.      */
} ha_hash_weights_t;

int ha_abi_version(void);
const char* ha_status_str(int status);

/* Process-wide dispatch options (no reference counterpart; the library reads no environment
 * variables). For experiments and tests: results never depend on them, only which kernels run
 * (the one exception, a failure-injection value, is marked).
 *   HA_OPT_CLUSTER_GATHER  -1 library decides, 0 / 1: thread-block-cluster variant of the gather
 *   HA_OPT_CLUSTER_SELECT  -1 library decides (at most 8 (sequence, kv-head) units of at most 65536
 *                          tokens), 0 never, 1 whenever the sequences fit: single-pass cluster kernel
 *                          for scoring + selection
 *   HA_OPT_PLAN_HANDOVER   -1 / 1 inside a step the selection kernel takes the plan of each (sequence,
 *                          kv-head) as soon as the scoring kernel has finished it (a ready word per unit in
 *                          the workspace, polled with a bound), 0 it waits for the whole scoring kernel.
 *                          2 is a failure-injection hook for tests of that bound: the selection waits, the
 *                          scoring kernel does not announce anything, every waiting CTA gives up after its
 *                          poll limit (about a second), the step's status is HA_ERR_TIMEOUT, its output is
 *                          undefined and the workspace has to be cleared again with ha_workspace_init.   */
#define HA_OPT_CLUSTER_GATHER 0
#define HA_OPT_CLUSTER_SELECT 1
#define HA_OPT_PLAN_HANDOVER 2
#define HA_OPT_COUNT_ 3
int ha_set_option(int option_key, int value); /* HA_ERR_BAD_ARG for an unknown key */
int ha_get_option(int option_key);

/* Bytes of workspace needed by any entry point below for this shape and these budgets
 * (0 if either is invalid). Host-only arithmetic. */
size_t ha_workspace_bytes(const ha_shape_t* shape, const ha_budget_t* budget);

/* Zeroes the workspace, in particular the arrival counters, histogram totals and ready words of the scoring kernel.
 * REQUIRED once after allocating the workspace, and again after a step that did not run to its end (a kernel was
 * aborted, the status word read HA_ERR_TIMEOUT, or a step returned HA_ERR_LAUNCH half-way): the kernels leave
 * these words at zero themselves and keep no other state in the workspace between calls.                        */
int ha_workspace_init(const ha_shape_t* shape, const ha_budget_t* budget, void* workspace,
                      size_t workspace_bytes, void* stream);

/* Decode-time hash encoder + cache append.
 * Replaces USA.q_embedding for the new query and USA.k_embedding for the new key
 * (hashattention/hashattention_llama.py:204-226, 411-414) and Cache.update (:573-576).
 *   - q_codes[b][h]  <- packed sign bits of q-MLP_h(q[b][h])
 *   - the 4 codes of k-MLP_{4j..4j+3}(k_new[b][j]) are written to the hash page slot of token
 *     seq_lens[b]-1; k_new / v_new rows are copied to the same slot of the K / V pages.
 *   - k_new == NULL skips the key side (query-only encode).
 *   - preact_dbg (optional, may be NULL): [batch][2][num_q_heads][32] f32 final-layer
 *     pre-activations, side 0 = query, side 1 = key.                                       */
int ha_hash_decode(const ha_shape_t* shape, const ha_hash_weights_t* weights,
                   const void* q, const void* k_new, const void* v_new,
                   void* k_pages, void* v_pages, uint32_t* hash_pages,
                   const int32_t* page_table, const int32_t* seq_lens,
                   uint32_t* q_codes, float* preact_dbg, int32_t* status, void* stream);

/* Prefill key-hash build: encodes every cached key of every sequence.
 * Replaces USA.k_embedding over the whole cache (hashattention/hashattention_llama.py:204-214;
 * the reference recomputes it on every decode step at :405-406).
 * Tokens [first_token[b], seq_lens[b]) of sequence b are encoded (first_token == NULL: from 0). */
int ha_hash_prefill(const ha_shape_t* shape, const ha_hash_weights_t* weights,
                    const void* k_pages, uint32_t* hash_pages,
                    const int32_t* page_table, const int32_t* seq_lens,
                    const int32_t* first_token, int32_t* status, void* stream);

/* Hamming scoring + budget selection (both usa_eval_modes, see ha_budget_t; the text below
 * describes HA_EVAL_SIMPLE).
 * Replaces the +-1 dot product of USA.forward (hashattention/hashattention_llama.py:171-187)
 * and compute_mask_multi (:423-438). score = popcount(~(q_code ^ k_code)) in 0..32, which
 * equals (span + 32) / 2 of the reference. Candidates are tokens [lo, hi) with
 * lo = min(init, S), hi = max(lo, S - recent); the heavy set is the min(hb, hi - lo) best
 * candidates, ties at the threshold broken by lowest token index.
 *   - sel_idx[b][h][0 .. sel_cnt[b][h]) <- heavy token indices, each once; ordered by chunks of
 *     the sequence (1024 to 32768 tokens, depending on the kernel that ran), not ascending
 *     inside a chunk: the set is the contract, not the order
 *   - scores_dbg (optional, may be NULL): [batch][num_q_heads][max_pages*page_size] u8      */
int ha_score_select(const ha_shape_t* shape, const ha_budget_t* budget,
                    const uint32_t* q_codes, const uint32_t* hash_pages,
                    const int32_t* page_table, const int32_t* seq_lens,
                    int32_t* sel_idx, int32_t* sel_cnt, uint8_t* scores_dbg,
                    void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* ha_score_select without a workspace, for callers that cannot hand the library any scratch
 * memory of their own. (No counterpart in the reference; it exists for hosts such as an
 * inference-server plugin whose enqueue hook may not allocate, or a process whose memory pool
 * already owns the whole device, where a cudaMalloc for the workspace is either forbidden or
 * fails.) Same inputs, outputs, results and status codes as ha_score_select; the per-chunk
 * score histograms, the plan and the score bytes live in a buffer of HA_STATIC_SCRATCH_BYTES that
 * is part of the library image: every GPU that loads libhashattn.so carries it until the process ends.
 *   - Returns HA_ERR_SCRATCH_LIMIT, launching nothing, when this shape needs more than that
 *     (ha_static_scratch_needed() tells how much a shape needs).
 *   - Calls no allocator of any kind. The first call on each device looks the buffer's device
 *     address up (cudaGetSymbolAddress) and keeps it; make that first call outside any stream
 *     capture.
 *   - All calls on a device share the one buffer, which keeps whatever the last call left. The
 *     one part that must start at zero (the scoring kernel's arrival counters and histogram totals) is cleared by
 *     every call on `stream` before its kernels; every other word is written before it is read.
 *     Two calls whose kernels may overlap on the GPU - different streams, no ordering between
 *     them - overwrite each other: order them.                                                  */
#define HA_STATIC_SCRATCH_BYTES (4u << 20)
size_t ha_static_scratch_needed(const ha_shape_t* shape);
int ha_score_select_static(const ha_shape_t* shape, const ha_budget_t* budget,
                           const uint32_t* q_codes, const uint32_t* hash_pages,
                           const int32_t* page_table, const int32_t* seq_lens,
                           int32_t* sel_idx, int32_t* sel_cnt, int32_t* status, void* stream);

/* The two halves of ha_decode_step after the encoder, as stages of their own (profiling, or a
 * host that interleaves other work): ha_score_plan streams the hash pages, leaves one score byte
 * per token and query head, the per-chunk histograms and the selection plan (thresholds, tie
 * quotas, per-chunk output offsets) in the workspace and writes sel_cnt; ha_select_attend, called
 * next on the same stream with the same workspace, selects (sel_idx <- heavy token indices, as
 * ha_score_select) and attends (out, as ha_sparse_decode) chunk by chunk in one kernel.
 * References: hashattention/hashattention_llama.py:171-187, 423-443 and :578-623.            */
int ha_score_plan(const ha_shape_t* shape, const ha_budget_t* budget,
                  const uint32_t* q_codes, const uint32_t* hash_pages,
                  const int32_t* page_table, const int32_t* seq_lens, int32_t* sel_cnt,
                  void* workspace, size_t workspace_bytes, int32_t* status, void* stream);
int ha_select_attend(const ha_shape_t* shape, const ha_budget_t* budget,
                     const void* q, const void* k_pages, const void* v_pages,
                     const int32_t* page_table, const int32_t* seq_lens,
                     int32_t* sel_idx, float sm_scale, void* out,
                     void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* Sparse GQA flash-decode over sink + heavy + recent tokens.
 * Replaces hashattention/hashattention_llama.py:578-623 (repeat_kv, QK^T/sqrt(d), mask fill,
 * fp32 softmax, .V); masked positions contribute exactly 0 there, so the result equals a
 * softmax over the selected set. fp32 accumulation, bf16 output.                            */
int ha_sparse_decode(const ha_shape_t* shape, const ha_budget_t* budget,
                     const void* q, const void* k_pages, const void* v_pages,
                     const int32_t* page_table, const int32_t* seq_lens,
                     const int32_t* sel_idx, const int32_t* sel_cnt, float sm_scale,
                     void* out, void* workspace, size_t workspace_bytes,
                     int32_t* status, void* stream);

/* One whole decode step of one layer: ha_hash_decode -> ha_score_select -> ha_sparse_decode
 * enqueued back to back on `stream` (hashattention/hashattention_llama.py:571-623).
 * q_codes [batch][num_q_heads], sel_idx [batch][num_q_heads][sel_stride] and
 * sel_cnt [batch][num_q_heads] are caller-owned device buffers that hold the intermediate
 * results afterwards.                                                                       */
int ha_decode_step(const ha_shape_t* shape, const ha_budget_t* budget,
                   const ha_hash_weights_t* weights,
                   const void* q, const void* k_new, const void* v_new,
                   void* k_pages, void* v_pages, uint32_t* hash_pages,
                   const int32_t* page_table, const int32_t* seq_lens,
                   uint32_t* q_codes, int32_t* sel_idx, int32_t* sel_cnt, float sm_scale,
                   void* out, void* workspace, size_t workspace_bytes,
                   int32_t* status, void* stream);

/* Multi-token decode: 2 <= q_len <= 128 new tokens per sequence in one call (the reference sends
 * them through the same sparse path: hashattention/hashattention_llama.py:529, with the causal /
 * recent diagonal of compute_mask_multi :423-428). The caller lays the step out as ROWS, one per
 * (sequence, new token): shape->batch = number of rows; q, k_new, v_new, out, q_codes, sel_idx,
 * sel_cnt are indexed by row; page_table row r repeats the page list of the row's sequence;
 * seq_lens[r] = position of the row's token + 1 (what that query may see, its own key included and
 * appended by this call); budget_lens[r] = length of the sequence after the whole chunk, the k of
 * int(k * heavy_budget) (:431-434). Every row is then exactly one ha_decode_step problem.
 * Requires recent_budget >= q_len - 1: a token of the chunk is then never a selection candidate
 * of a later row of the same call (its hash word is written by this call).                      */
int ha_decode_step_rows(const ha_shape_t* shape, const ha_budget_t* budget,
                        const ha_hash_weights_t* weights,
                        const void* q, const void* k_new, const void* v_new,
                        void* k_pages, void* v_pages, uint32_t* hash_pages,
                        const int32_t* page_table, const int32_t* seq_lens, const int32_t* budget_lens,
                        uint32_t* q_codes, int32_t* sel_idx, int32_t* sel_cnt, float sm_scale,
                        void* out, void* workspace, size_t workspace_bytes,
                        int32_t* status, void* stream);

/* Number of kernels one ha_decode_step call enqueues for this shape and budget (the library picks
 * between a single-pass cluster selection and scoring + fused selection/attention); 0 for an
 * invalid shape. For launch accounting; no reference counterpart. (With the LSH baseline, HA_HASH_LSH,
 * a step enqueues one kernel more: the re-hash pass that returns at once unless the key norm bound rose.) */
int ha_decode_step_launches(const ha_shape_t* shape, const ha_budget_t* budget);
/* The kernels of that step by name, in launch order, as a static string (for labelling measurements). */
const char* ha_decode_step_path(const ha_shape_t* shape, const ha_budget_t* budget);

/* ha_decode_step for a caller whose per-step tensors live in HOST memory.
 * q_host, k_new_host, v_new_host (inputs) and out_host (result) are HOST pointers; q_dev,
 * k_new_dev, v_new_dev, out_dev are device staging buffers of the same sizes.
 * If all host buffers are page-locked and device-addressable (cudaHostAlloc / cudaHostRegister,
 * torch pin_memory) the kernels use them in place: the encoder kernel reads the inputs over the
 * bus once (keeping a device copy of q in q_dev), the last kernel stores the result into
 * out_host and, if status_host is page-locked too, the step's last kernel stores the status word
 * into status_host; else that word is copied. Otherwise the inputs are copied to the staging
 * buffers, ha_decode_step runs on those, and `out` is copied back. Either way the host buffers
 * must stay untouched until the stream has reached the end of the call. If `synchronize` is
 * non-zero the call waits for the stream and returns the device status word (HA_OK if clean).
 * status_host is a host int32 receiving that word.                                          */
int ha_decode_step_host(const ha_shape_t* shape, const ha_budget_t* budget,
                        const ha_hash_weights_t* weights,
                        const void* q_host, const void* k_new_host, const void* v_new_host,
                        void* out_host, int32_t* status_host,
                        void* q_dev, void* k_new_dev, void* v_new_dev, void* out_dev,
                        void* k_pages, void* v_pages, uint32_t* hash_pages,
                        const int32_t* page_table, const int32_t* seq_lens,
                        uint32_t* q_codes, int32_t* sel_idx, int32_t* sel_cnt, float sm_scale,
                        void* workspace, size_t workspace_bytes,
                        int32_t* status, void* stream, int synchronize);

/* Helper for a host model's decode step (one new token per sequence): splits the fused projection
 * qkv [batch][num_q_heads + 2 * num_kv_heads][128] bf16 (query heads, then key heads, then value
 * heads) into the contiguous q [batch][num_q_heads][128], k_new and v_new [batch][num_kv_heads][128]
 * that ha_decode_step takes, applying the rotary position embedding (rotate-half convention,
 * angle = positions[b] * rope_theta^(-2i/128), fp32) to q and k on the way. Replaces
 * apply_rotary_pos_emb + the view / transpose of hashattention/hashattention_llama.py:551-571 for
 * q_len == 1. positions: [batch] int64 on the device.                                          */
int ha_rope_split(const void* qkv, const int64_t* positions, int32_t batch, int32_t num_q_heads,
                  int32_t num_kv_heads, float rope_theta, void* q, void* k_new, void* v_new, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HASHATTN_H_ */
